#!/usr/bin/env python
"""Orchestrates a benchmark campaign into one output directory: build, system information, peer-copy
speed of light, examples as smoke tests, the size sweep of every variant per dtype and the NCCL sweep
with the same timing code (both repeated `runs` times), per-dtype CSVs, the markdown summary, line
charts (SVG), a per-kernel summary of the device-side timeline and an index of everything written.

    python bench/run_sweep.py --gpus 8 --mode standard --out results/$(date +%F)

Modes (sizes x dtypes x runs): quick (5 sizes, fp32, 1 run), standard (4 KiB-2 GiB, fp32/fp16/bf16, 2 runs),
full (standard with 5 runs), extensive (10 runs).
Reference counterpart: scripts/sweep.py (build -> system info -> nvbandwidth -> examples -> sweeps ->
profiler -> graphs -> summary.md -> index.md).  Its nsys phase (kernel durations out of an sqlite export)
becomes `profiler_summary.json`, built from the %globaltimer stamps the kernels write themselves; its
matplotlib PNGs become dependency-free SVGs (bench/plots.py)."""
from __future__ import annotations

import argparse
import json
import os
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


GRAPH_MAX_BYTES = 4 << 20  # up to here both arms time one CUDA-graph replay of all calls


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
        if sh(["make", "lib", "bench", "examples"]).returncode != 0:  # includes build/bin/nccl_sweep
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
               m["dtypes"], "--graph-max-bytes", str(GRAPH_MAX_BYTES), "--min-bytes", str(m["min_bytes"]), "--max-bytes", str(m["max_bytes"]),
               "--out", str(f)] + (["--tuning-out", str(out / "tuning.json")] if i == 0 else [])
        if sh(cmd, stdout=subprocess.DEVNULL).returncode != 0:
            print("sweep run failed", file=sys.stderr)
            return 1
        # NCCL with the same timing code (C++, one process per GPU), appended to the same file.
        nccl = sh([sys.executable, "-m", "yali_b200.launch", "-np", str(args.gpus), str(ROOT / "build/bin/nccl_sweep"),
                   str(m["min_bytes"]), str(m["max_bytes"]), m["dtypes"], str(GRAPH_MAX_BYTES)], capture_output=True,
                  text=True, env={**os.environ, "MASTER_PORT": str(args.port + 100 + i)})
        with open(f, "a") as fh:
            fh.write("".join(ln + "\n" for ln in nccl.stdout.splitlines() if ln.startswith("{")))
        runs.append(str(f))
    rc = sh([sys.executable, "bench/report.py", "--out", str(out)] + runs).returncode
    write_profiler_summary(runs, out)
    write_index(out, args, m)
    return rc


def write_profiler_summary(runs, out: Path) -> None:
    """Per kernel and message size: calls sampled and p50 / p99 / max of the device time per call.  The
    reference gets the same table from an nsys trace (scripts/sweep.py:1198-1496)."""
    agg = {}
    for run in runs:
        for line in Path(run).read_text().splitlines():
            if not line.startswith("{"):
                continue
            r = json.loads(line)
            if r.get("impl") != "yali_b200" or "dev_p50_us" not in r:
                continue
            k = agg.setdefault(r["kernel"], {}).setdefault(f'{r["dtype"]}:{r["bytes"]}', {"calls": 0, "p50_us": [], "p99_us": [], "max_us": 0.0})
            k["calls"] += r.get("dev_samples", 0)
            k["p50_us"].append(r["dev_p50_us"])
            k["p99_us"].append(r["dev_p99_us"])
            k["max_us"] = max(k["max_us"], r["dev_max_us"])
    for sizes in agg.values():
        for v in sizes.values():
            v["p50_us"] = round(sum(v["p50_us"]) / len(v["p50_us"]), 2)
            v["p99_us"] = round(sum(v["p99_us"]) / len(v["p99_us"]), 2)
    (out / "profiler_summary.json").write_text(json.dumps(
        {"source": "device-side timeline: %globaltimer at first-CTA entry and last-CTA exit of every call, max over ranks",
         "kernels": agg}, indent=1))


def write_index(out: Path, args, mode: dict) -> None:
    files = sorted(p.name for p in out.iterdir() if p.is_file() and p.name != "index.md")
    groups = [("Summary", [f for f in files if f in ("summary.md",)]),
              ("System", [f for f in files if f in ("system_info.json", "p2p_bandwidth.json", "examples.log")]),
              ("Tables (per implementation, world size and dtype)", [f for f in files if f.endswith(".csv")]),
              ("Charts", [f for f in files if f.endswith(".svg")]),
              ("Device-side timeline per kernel", [f for f in files if f == "profiler_summary.json"]),
              ("Raw runs and tuning table", [f for f in files if f.endswith(".jsonl") or f == "tuning.json"])]
    lines = ["# Benchmark campaign", "", f"GPUs: {args.gpus}; mode: {args.mode} (sizes {mode['min_bytes']} - {mode['max_bytes']} "
             f"bytes, dtypes {mode['dtypes']}, {mode['runs']} run(s)).", ""]
    for title, fs in groups:
        if fs:
            lines += [f"## {title}", ""] + [f"* [{f}]({f})" for f in fs] + [""]
    (out / "index.md").write_text("\n".join(lines))


if __name__ == "__main__":
    sys.exit(main())
