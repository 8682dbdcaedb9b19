#!/usr/bin/env python
"""Orchestrates a benchmark campaign into one output directory: build, system information, peer-copy
speed of light, examples as smoke tests, the size sweep of every variant against NCCL per dtype
(repeated `runs` times), per-dtype CSVs and the markdown summary.

    python bench/run_sweep.py --gpus 8 --mode standard --out results/$(date +%F)

Modes (sizes x dtypes x runs): quick (5 sizes, fp32, 1 run), standard (4 KiB-2 GiB, fp32/fp16/bf16, 2 runs),
full (standard with 5 runs), extensive (10 runs).
Reference counterpart: scripts/sweep.py (build -> system info -> nvbandwidth -> examples -> sweeps ->
graphs -> summary.md); the nsys phase is replaced by `YALI_PROFILE_KERNELS=1` and the committed ncu
summaries, the PNG graphs by CSVs."""
from __future__ import annotations

import argparse
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
from yali_b200.utils import hw_info  # noqa: E402

MODES = {
    "quick": dict(min_bytes=4096, max_bytes=1 << 30, dtypes="fp32", runs=1, step=16),
    "standard": dict(min_bytes=4096, max_bytes=2 << 30, dtypes="fp32,fp16,bf16", runs=2, step=2),
    "full": dict(min_bytes=4096, max_bytes=2 << 30, dtypes="fp32,fp16,bf16", runs=5, step=2),
    "extensive": dict(min_bytes=4096, max_bytes=2 << 30, dtypes="fp32,fp16,bf16", runs=10, step=2),
}


def sh(cmd, **kw):
    print("+", " ".join(map(str, cmd)), flush=True)
    return subprocess.run(cmd, cwd=str(ROOT), **kw)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=2)
    ap.add_argument("--mode", choices=list(MODES), default="quick")
    ap.add_argument("--out", default="results/latest")
    ap.add_argument("--port", type=int, default=29541)
    ap.add_argument("--skip-build", action="store_true")
    args = ap.parse_args()
    m = MODES[args.mode]
    out = Path(args.out)
    out.mkdir(parents=True, exist_ok=True)
    if not args.skip_build:
        if sh(["make", "lib", "bench", "examples"]).returncode != 0:
            return 1
    (out / "system_info.json").write_text(json.dumps(hw_info.system_info(), indent=1, default=str))
    p2p = sh([str(ROOT / "build/bin/p2p_bandwidth")], capture_output=True, text=True)
    (out / "p2p_bandwidth.json").write_text(p2p.stdout)
    ex = sh([str(ROOT / "build/bin/example_simple")], capture_output=True, text=True)
    (out / "examples.log").write_text(ex.stdout + ex.stderr)
    runs = []
    for i in range(m["runs"]):
        f = out / f"sweep_run{i}.jsonl"
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", str(args.port + i), "bench/sweep.py", "--dtypes",
               m["dtypes"], "--nccl", "--min-bytes", str(m["min_bytes"]), "--max-bytes", str(m["max_bytes"]),
               "--out", str(f)] + (["--tuning-out", str(out / "tuning.json")] if i == 0 else [])
        if sh(cmd, stdout=subprocess.DEVNULL).returncode != 0:
            print("sweep run failed", file=sys.stderr)
            return 1
        runs.append(str(f))
    return sh([sys.executable, "bench/report.py", "--out", str(out)] + runs).returncode


if __name__ == "__main__":
    sys.exit(main())
