#!/usr/bin/env python
"""Turns sweep output (JSON lines from bench/sweep.py, one file per run) into per-dtype CSVs with
run-level statistics and a markdown summary with the speed-up over NCCL per size.

    python bench/report.py --out report_dir run1.jsonl [run2.jsonl ...]

Reference counterpart: the CSV / summary.md / graph phases of scripts/sweep.py (654-680, 702-1193,
1501-1798).  The charts are SVG files written by bench/plots.py (no plotting dependency)."""
from __future__ import annotations

import argparse
import csv
import json
import sys
from collections import defaultdict
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))
sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
from yali_b200.utils.stats import summarise  # noqa: E402

LINK_MEASURED_GBS = 770.0
LINK_NOMINAL_GBS = 900.0


def human(n: int) -> str:
    for unit, s in ((1 << 30, "G"), (1 << 20, "M"), (1 << 10, "K")):
        if n >= unit and n % unit == 0:
            return f"{n // unit}{s}"
    return str(n)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("runs", nargs="+")
    ap.add_argument("--out", default="report")
    args = ap.parse_args()
    out = Path(args.out)
    out.mkdir(parents=True, exist_ok=True)
    samples = defaultdict(list)  # (impl, world, dtype, variant, bytes) -> [busbw per run]
    times = defaultdict(list)
    tails = defaultdict(list)  # device-timed p99 / p50 per call
    for run in args.runs:
        for line in Path(run).read_text().splitlines():
            if not line.startswith("{"):
                continue
            r = json.loads(line)
            key = (r["impl"], r["world"], r["dtype"], r["variant"], r["bytes"])
            samples[key].append(r["busbw_gbps"])
            times[key].append(r["us"])
            if r.get("dev_p50_us"):
                tails[key].append(r["dev_p99_us"] / r["dev_p50_us"])
    by_file = defaultdict(list)
    for (impl, world, dtype, variant, nbytes), vals in sorted(samples.items()):
        st = summarise(vals)
        by_file[(impl, world, dtype)].append({
            "variant": variant, "size": human(nbytes), "bytes": nbytes, "mean_gbps": round(st.mean, 3),
            "stddev_gbps": round(st.stddev, 3), "min_gbps": round(st.min, 3), "max_gbps": round(st.max, 3),
            "cv_pct": round(st.cv_pct, 3), "p50": round(st.p50, 3), "p90": round(st.p90, 3), "p95": round(st.p95, 3),
            "p99": round(st.p99, 3), "sol_pct_measured_link": round(100 * st.mean / LINK_MEASURED_GBS, 1),
            "sol_pct_nominal_link": round(100 * st.mean / LINK_NOMINAL_GBS, 1),
            "mean_us": round(sum(times[(impl, world, dtype, variant, nbytes)]) / len(vals), 2), "runs": st.samples})
    for (impl, world, dtype), rows in by_file.items():
        with open(out / f"{impl}_w{world}_{dtype}.csv", "w", newline="") as f:
            w = csv.DictWriter(f, fieldnames=list(rows[0].keys()))
            w.writeheader()
            w.writerows(rows)
    lines = ["# Sweep summary", "",
             "Bus bandwidth in GB/s (NCCL convention, bytes*2(n-1)/n/t), device-timed, max over ranks; mean over "
             f"{max(len(v) for v in samples.values())} run(s). SoL against the measured {LINK_MEASURED_GBS:.0f} GB/s "
             f"per-direction peer copy ({LINK_NOMINAL_GBS:.0f} nominal).", ""]
    worlds = sorted({k[1] for k in samples})
    for world in worlds:
        for dtype in sorted({k[2] for k in samples if k[1] == world}):
            lines += [f"## {world} ranks, {dtype}", "",
                      "| size | auto | flash | stream | nvls | stream_direct | NCCL | auto / NCCL | auto % of measured link | "
                      "auto p99/p50 (device) |",
                      "|---|---|---|---|---|---|---|---|---|---|"]
            sizes = sorted({k[4] for k in samples if k[1] == world and k[2] == dtype})
            for b in sizes:
                def g(impl, variant):
                    v = samples.get((impl, world, dtype, variant, b))
                    return sum(v) / len(v) if v else None
                cells = [g("yali_b200", v) for v in ("auto", "flash", "stream", "nvls", "stream_direct")] + [g("nccl", "nccl")]
                ratio = f"{cells[0] / cells[5]:.2f}x" if cells[0] and cells[5] else "-"
                sol = f"{100 * cells[0] / LINK_MEASURED_GBS:.0f} %" if cells[0] else "-"
                tl = tails.get(("yali_b200", world, dtype, "auto", b))
                tail = f"{sum(tl) / len(tl):.2f}" if tl else "-"
                lines.append("| " + human(b) + " | " + " | ".join("-" if c is None else f"{c:.1f}" for c in cells) +
                             f" | {ratio} | {sol} | {tail} |")
            lines.append("")
    from plots import make_all  # bench/plots.py
    charts = make_all(args.runs, out, LINK_MEASURED_GBS)
    if charts:
        lines += ["## Charts", ""] + [f"![{c}]({c})" for c in charts] + [""]
    (out / "summary.md").write_text("\n".join(lines))
    print(f"wrote {out}/summary.md, {len(by_file)} CSV file(s) and {len(charts)} chart(s)")


if __name__ == "__main__":
    main()
