#!/usr/bin/env python
"""Five sizes, a few runs each, this library against NCCL with the C++ benchmarks (`make bench` first).

    python bench/quick_benchmark.py [--gpus 2] [--runs 3] [--dtype fp32] [--processes]

Both binaries get the same positional arguments (elements calls verify mode lanes timing dtype gpus); the
reference's quick_benchmark passes its timing mode in the `verify` position (scripts/quick_benchmark.py:145-151),
which silently ran the two sides in different timing modes; here the argument list is built once for both.
`--processes` uses the one-process-per-GPU binaries under `python -m yali_b200.launch`."""
from __future__ import annotations

import argparse
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
from yali_b200.utils.stats import summarise  # noqa: E402

SIZES = [4 << 10, 64 << 10, 1 << 20, 64 << 20, 1 << 30]


def run(binary: str, elems: int, args) -> float:
    argv = [str(ROOT / "build" / "bin" / binary), str(elems), str(args.calls), "0", "auto", "0", "cuda-events",
            args.dtype]
    if args.processes:
        argv = [sys.executable, "-m", "yali_b200.launch", "-np", str(args.gpus)] + argv
    else:
        argv.append(str(args.gpus))
    out = subprocess.run(argv, capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    for line in out.stdout.splitlines():
        if line.startswith("{"):
            return json.loads(line)["busbw_gbps"]
    raise RuntimeError(f"{binary} produced no result line:\n{out.stdout[-500:]}{out.stderr[-500:]}")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=2)
    ap.add_argument("--runs", type=int, default=3)
    ap.add_argument("--calls", type=int, default=100)
    ap.add_argument("--dtype", default="fp32")
    ap.add_argument("--processes", action="store_true")
    args = ap.parse_args()
    esz = 4 if args.dtype == "fp32" else 2
    suffix = "_mpi" if args.processes else ""
    print(f"{'size':>8} {'yali GB/s':>12} {'nccl GB/s':>12} {'speed-up':>9} {'yali CV%':>9}")
    for size in SIZES:
        y = [run("benchmark_yali" + suffix, size // esz, args) for _ in range(args.runs)]
        n = [run("benchmark_nccl" + suffix, size // esz, args) for _ in range(args.runs)]
        sy, sn = summarise(y), summarise(n)
        print(f"{size:>8} {sy.mean:>12.2f} {sn.mean:>12.2f} {sy.mean / sn.mean:>8.2f}x {sy.cv_pct:>9.2f}")


if __name__ == "__main__":
    main()
