#!/usr/bin/env python
"""Checks the baseline the comparisons rest on: the NCCL header version equals the version of the library the
benchmarks load, torch's bundled NCCL is reported, and (with --run, on a GPU box) benchmark_nccl passes its own
correctness check and clears a bus-bandwidth floor at 128 MiB.

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


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--run", action="store_true", help="also run build/bin/benchmark_nccl (needs GPUs)")
    ap.add_argument("--gpus", type=int, default=2)
    ap.add_argument("--floor-gbps", type=float, default=300.0)
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
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
