#!/usr/bin/env python
"""Checks the baseline the comparisons rest on: the NCCL header version equals the version of the library the
benchmarks load, torch's bundled NCCL is reported, and (with --run, on a GPU box) benchmark_nccl passes its own
correctness check and clears a bus-bandwidth floor at 128 MiB, the NCCL size sweep (build/bin/nccl_sweep, the
stand-in for nccl-tests) produces a monotone, complete set of rows, and the peer-copy speed of light
(build/bin/p2p_bandwidth, the stand-in for nvbandwidth) clears its floors in one and in both directions.

Reference counterparts: tests/validate_nccl_version.sh, tests/validate_nccl_tests.sh, tests/validate_nvbandwidth.sh,
tests/run_nccl_baseline.sh (nccl-tests and nvbandwidth themselves are not available offline here)."""
from __future__ import annotations

import argparse
import ctypes
import json
import re
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def header_version(path: str = "/usr/include/nccl.h"):
    text = Path(path).read_text()
    parts = [int(re.search(rf"#define NCCL_{k}\s+(\d+)", text).group(1)) for k in ("MAJOR", "MINOR", "PATCH")]
    return parts[0] * 10000 + parts[1] * 100 + parts[2]


def system_library_path() -> str:
    """The libnccl the C++ benchmarks link against (not the copy torch bundles, which a Python process
    that imported torch has already loaded under the same soname)."""
    out = subprocess.run(["ldconfig", "-p"], capture_output=True, text=True).stdout
    for line in out.splitlines():
        if "libnccl.so.2 " in line and "=>" in line:
            return line.split("=>")[1].strip()
    return "libnccl.so.2"


def library_version(name: str = ""):
    lib = ctypes.CDLL(name or system_library_path())
    v = ctypes.c_int(0)
    lib.ncclGetVersion(ctypes.byref(v))
    return v.value


def check_p2p(record: dict, floor: float) -> list:
    """Problems with one line of p2p_bandwidth output (empty list = fine)."""
    if "unavailable" in record:
        return [record["unavailable"]]
    bad = []
    for key in ("copy_engine_unidirectional_gbs", "copy_engine_bidirectional_per_direction_gbs", "sm_remote_store_gbs",
                "sm_remote_load_gbs", "bulk_pull_gbs", "bulk_push_gbs"):
        v = record.get(key)
        if v is None or v < floor:
            bad.append(f"{key} = {v} below the floor of {floor} GB/s")
    return bad


def check_nccl_sweep(rows: list, floor: float) -> list:
    """Problems with the rows of nccl_sweep: every power of two present once per dtype, times positive and
    non-decreasing from 1 MiB on, and the largest message at or above the bandwidth floor."""
    bad = []
    by_dtype = {}
    for r in rows:
        by_dtype.setdefault(r["dtype"], []).append(r)
    if not by_dtype:
        return ["no rows"]
    for dtype, rs in by_dtype.items():
        rs.sort(key=lambda r: r["bytes"])
        sizes = [r["bytes"] for r in rs]
        if any(b != sizes[0] << i for i, b in enumerate(sizes)):
            bad.append(f"{dtype}: sizes are not consecutive powers of two: {sizes}")
        if any(r["us"] <= 0 for r in rs):
            bad.append(f"{dtype}: non-positive time")
        big = [r for r in rs if r["bytes"] >= (1 << 20)]
        if any(b["us"] < a["us"] * 0.8 for a, b in zip(big, big[1:])):
            bad.append(f"{dtype}: time per call shrinks with the message size")
        if rs[-1]["bytes"] >= (128 << 20) and rs[-1]["busbw_gbps"] < floor:
            bad.append(f"{dtype}: {rs[-1]['busbw_gbps']} GB/s at {rs[-1]['bytes']} bytes, floor {floor}")
    return bad


def validate_p2p(floor: float) -> bool:
    out = subprocess.run([str(ROOT / "build" / "bin" / "p2p_bandwidth"), str(256 << 20), "5"], capture_output=True,
                         text=True, timeout=600)
    line = next((ln for ln in out.stdout.splitlines() if ln.startswith("{")), "{}")
    bad = check_p2p(json.loads(line), floor)
    print("p2p_bandwidth:", "OK " + line if not bad else "; ".join(bad))
    return not bad


def validate_nccl_sweep(gpus: int, floor: float) -> bool:
    out = subprocess.run([sys.executable, "-m", "yali_b200.launch", "-np", str(gpus), str(ROOT / "build" / "bin" / "nccl_sweep"),
                          "4096", str(256 << 20), "fp32"], capture_output=True, text=True, timeout=900, cwd=str(ROOT))
    rows = [json.loads(ln) for ln in out.stdout.splitlines() if ln.startswith("{")]
    bad = check_nccl_sweep(rows, floor) if out.returncode == 0 else [f"nccl_sweep exited {out.returncode}: {out.stderr[-200:]}"]
    print(f"nccl_sweep: {len(rows)} rows,", "OK" if not bad else "; ".join(bad))
    return not bad


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--run", action="store_true", help="also run build/bin/benchmark_nccl (needs GPUs)")
    ap.add_argument("--gpus", type=int, default=2)
    ap.add_argument("--floor-gbps", type=float, default=300.0)
    ap.add_argument("--p2p-floor-gbps", type=float, default=500.0)
    args = ap.parse_args()
    ok = True
    hv, lv = header_version(), library_version()
    print(f"nccl.h version {hv}, libnccl.so.2 version {lv}: {'OK' if hv == lv else 'MISMATCH'}")
    ok &= hv == lv
    try:
        import torch
        print("torch bundles NCCL", ".".join(map(str, torch.cuda.nccl.version())))
    except Exception as e:  # noqa: BLE001
        print("torch NCCL version unavailable:", e)
    if args.run:
        exe = ROOT / "build" / "bin" / "benchmark_nccl"
        out = subprocess.run([str(exe), str(32 << 20), "20", "1", "auto", "0", "cuda-events", "fp32", str(args.gpus)],
                             capture_output=True, text=True, timeout=600)
        passed = "Correctness: PASSED" in out.stdout
        bw = next((json.loads(l)["busbw_gbps"] for l in out.stdout.splitlines() if l.startswith("{")), 0.0)
        print(f"benchmark_nccl 128 MiB: correctness {'PASSED' if passed else 'FAILED'}, {bw:.1f} GB/s "
              f"(floor {args.floor_gbps})")
        ok &= passed and bw >= args.floor_gbps
        ok &= validate_p2p(args.p2p_floor_gbps)
        ok &= validate_nccl_sweep(args.gpus, args.floor_gbps)
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
