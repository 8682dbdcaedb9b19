#!/usr/bin/env python
"""Joins a sweep of this library (JSON lines from bench/sweep.py) with an nccl-tests `all_reduce_perf` log into
one ratio table (CSV + markdown) and checks that the bandwidth ratio agrees with the inverse time ratio.

    python bench/consolidate_eval.py --sweep sweep.jsonl --nccl-log all_reduce_perf.log --out eval

Reference counterpart: tests/consolidate_eval.py (joins a yali_sweep.csv with an nccl-tests stdout log)."""
from __future__ import annotations

import argparse
import csv
import json
import re
from pathlib import Path
from typing import Dict, Tuple


def parse_nccl_tests_log(text: str) -> Dict[int, Tuple[float, float]]:
    """size_bytes -> (out-of-place time_us, busbw GB/s) from nccl-tests' table."""
    rows = {}
    for line in text.splitlines():
        f = line.split()
        # size count type redop root time algbw busbw #wrong time algbw busbw #wrong
        if len(f) >= 9 and f[0].isdigit() and re.match(r"^-?\d+$", f[4] if f[4] != "none" else "0"):
            try:
                rows[int(f[0])] = (float(f[5]), float(f[7]))
            except ValueError:
                continue
    return rows


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--sweep", required=True)
    ap.add_argument("--nccl-log", required=True)
    ap.add_argument("--variant", default="auto")
    ap.add_argument("--out", default="eval")
    args = ap.parse_args()
    nccl = parse_nccl_tests_log(Path(args.nccl_log).read_text())
    ours = {}
    for line in Path(args.sweep).read_text().splitlines():
        if line.startswith("{"):
            r = json.loads(line)
            if r["impl"] == "yali_b200" and r["variant"] == args.variant:
                ours[r["bytes"]] = (r["us"], r["busbw_gbps"])
    rows = []
    for size in sorted(set(ours) & set(nccl)):
        (yt, yb), (nt, nb) = ours[size], nccl[size]
        bw_ratio, t_ratio = yb / nb if nb else 0.0, nt / yt if yt else 0.0
        rows.append({"bytes": size, "yali_us": yt, "nccl_us": nt, "yali_busbw": yb, "nccl_busbw": nb,
                     "bw_ratio": round(bw_ratio, 3), "time_ratio": round(t_ratio, 3),
                     "consistent": abs(bw_ratio - t_ratio) <= 0.05 * max(bw_ratio, t_ratio, 1e-9)})
    out = Path(args.out)
    out.mkdir(parents=True, exist_ok=True)
    if rows:
        with open(out / "ratio.csv", "w", newline="") as f:
            w = csv.DictWriter(f, fieldnames=list(rows[0].keys()))
            w.writeheader()
            w.writerows(rows)
    md = ["| bytes | yali us | nccl us | yali GB/s | nccl GB/s | speed-up |", "|---|---|---|---|---|---|"]
    md += [f"| {r['bytes']} | {r['yali_us']} | {r['nccl_us']} | {r['yali_busbw']} | {r['nccl_busbw']} | {r['bw_ratio']}x |"
           for r in rows]
    (out / "ratio.md").write_text("\n".join(md) + "\n")
    bad = [r["bytes"] for r in rows if not r["consistent"]]
    print(f"{len(rows)} sizes joined; bandwidth and time ratios disagree at: {bad if bad else 'none'}")


if __name__ == "__main__":
    main()
