#!/usr/bin/env python
"""Line charts of a sweep as SVG files, written without any plotting dependency (matplotlib is not a
dependency of this project): bus bandwidth against message size per variant, speed-up over NCCL, time
per call, fraction of the link's speed of light, run-to-run variation, and a dtype comparison.

    python bench/plots.py --out report_dir run1.jsonl [run2.jsonl ...]

Reference counterpart: the graph phase of scripts/sweep.py (702-1193), which draws the same families of
charts with matplotlib into PNG files."""
from __future__ import annotations

import argparse
import json
import math
from collections import defaultdict
from pathlib import Path
from typing import Dict, List, Sequence, Tuple

COLORS = ["#1f77b4", "#d62728", "#2ca02c", "#ff7f0e", "#9467bd", "#8c564b", "#17becf", "#7f7f7f", "#bcbd22", "#e377c2"]
W, H, ML, MR, MT, MB = 860, 480, 70, 170, 40, 55


def human(n: float) -> str:
    n = int(n)
    for unit, s in ((1 << 30, "G"), (1 << 20, "M"), (1 << 10, "K")):
        if n >= unit:
            return f"{n // unit}{s}"
    return str(n)


def nice_ticks(lo: float, hi: float, n: int = 6) -> List[float]:
    if hi <= lo:
        hi = lo + 1.0
    raw = (hi - lo) / n
    mag = 10 ** math.floor(math.log10(raw))
    step = min((s for s in (1, 2, 2.5, 5, 10) if s * mag >= raw), default=10) * mag
    t, out = math.floor(lo / step) * step, []
    while t <= hi + 1e-9:
        if t >= lo - 1e-9:
            out.append(round(t, 10))
        t += step
    return out


def line_chart(path: Path, title: str, ylabel: str, series: Dict[str, Sequence[Tuple[float, float]]],
               logy: bool = False, hline: Tuple[float, str] = None) -> None:
    """series: label -> [(bytes, value), ...]; x is log2(bytes)."""
    pts = [p for s in series.values() for p in s if p[1] is not None and (not logy or p[1] > 0)]
    if not pts:
        return
    xs = sorted({p[0] for p in pts})
    x0, x1 = math.log2(xs[0]), math.log2(xs[-1])
    if x1 == x0:
        x1 = x0 + 1
    ys = [p[1] for p in pts] + ([hline[0]] if hline else [])
    if logy:
        y0, y1 = math.log10(min(ys)), math.log10(max(ys))
        y0, y1 = math.floor(y0), math.ceil(y1) if y1 > y0 else y0 + 1
    else:
        y0, y1 = 0.0, max(ys) * 1.08
        if y1 <= y0:  # all values zero (for instance identical runs in a variation chart)
            y1 = 1.0

    def px(b):
        return ML + (math.log2(b) - x0) / (x1 - x0) * (W - ML - MR)

    def py(v):
        t = (math.log10(v) if logy else v)
        return H - MB - (t - y0) / (y1 - y0) * (H - MT - MB)

    o = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{W}" height="{H}" viewBox="0 0 {W} {H}" '
         'font-family="sans-serif" font-size="12">', f'<rect width="{W}" height="{H}" fill="white"/>',
         f'<text x="{W / 2}" y="22" text-anchor="middle" font-size="15">{title}</text>']
    yt = [10 ** e for e in range(int(y0), int(y1) + 1)] if logy else nice_ticks(y0, y1)
    for v in yt:
        y = py(v)
        o.append(f'<line x1="{ML}" y1="{y:.1f}" x2="{W - MR}" y2="{y:.1f}" stroke="#ddd"/>')
        o.append(f'<text x="{ML - 6}" y="{y + 4:.1f}" text-anchor="end">{v:g}</text>')
    for b in xs:
        x = px(b)
        o.append(f'<line x1="{x:.1f}" y1="{MT}" x2="{x:.1f}" y2="{H - MB}" stroke="#eee"/>')
    step = max(1, len(xs) // 11)
    for b in xs[::step]:
        o.append(f'<text x="{px(b):.1f}" y="{H - MB + 16}" text-anchor="middle">{human(b)}</text>')
    o.append(f'<rect x="{ML}" y="{MT}" width="{W - ML - MR}" height="{H - MT - MB}" fill="none" stroke="#333"/>')
    o.append(f'<text x="{(ML + W - MR) / 2}" y="{H - 12}" text-anchor="middle">message size (bytes per rank)</text>')
    o.append(f'<text x="16" y="{(MT + H - MB) / 2}" text-anchor="middle" transform="rotate(-90 16 {(MT + H - MB) / 2})">'
             f'{ylabel}</text>')
    if hline:
        y = py(hline[0])
        o.append(f'<line x1="{ML}" y1="{y:.1f}" x2="{W - MR}" y2="{y:.1f}" stroke="#555" stroke-dasharray="6 4"/>')
        o.append(f'<text x="{W - MR + 6}" y="{y + 4:.1f}" fill="#555">{hline[1]}</text>')
    for i, (label, s) in enumerate(series.items()):
        c = COLORS[i % len(COLORS)]
        good = sorted((b, v) for b, v in s if v is not None and (not logy or v > 0))
        if not good:
            continue
        o.append('<polyline fill="none" stroke="%s" stroke-width="2" points="%s"/>' %
                 (c, " ".join(f"{px(b):.1f},{py(v):.1f}" for b, v in good)))
        for b, v in good:
            o.append(f'<circle cx="{px(b):.1f}" cy="{py(v):.1f}" r="2.5" fill="{c}"/>')
        ly = MT + 14 + 18 * i
        o.append(f'<line x1="{W - MR + 8}" y1="{ly - 4}" x2="{W - MR + 30}" y2="{ly - 4}" stroke="{c}" stroke-width="2"/>')
        o.append(f'<text x="{W - MR + 36}" y="{ly}">{label}</text>')
    o.append("</svg>")
    path.write_text("\n".join(o))


def load(runs: Sequence[str]):
    """(impl, world, dtype, variant) -> {bytes: [rows of all runs]}"""
    data = defaultdict(lambda: defaultdict(list))
    for run in runs:
        for line in Path(run).read_text().splitlines():
            if line.startswith("{"):
                r = json.loads(line)
                if "busbw_gbps" in r and "bytes" in r:
                    data[(r["impl"], r["world"], r["dtype"], r["variant"])][r["bytes"]].append(r)
    return data


def mean(rows, key):
    vals = [r[key] for r in rows if r.get(key) is not None]
    return sum(vals) / len(vals) if vals else None


def make_all(runs: Sequence[str], out: Path, link_gbs: float = 770.0) -> List[str]:
    out.mkdir(parents=True, exist_ok=True)
    data = load(runs)
    written = []
    worlds = sorted({k[1] for k in data})
    for world in worlds:
        dtypes = sorted({k[2] for k in data if k[1] == world})
        for dtype in dtypes:
            keys = [k for k in data if k[1] == world and k[2] == dtype]
            label = (lambda k: "NCCL" if k[0].startswith("nccl") else k[3])
            bw = {label(k): [(b, mean(rows, "busbw_gbps")) for b, rows in data[k].items()] for k in keys}
            us = {label(k): [(b, mean(rows, "us")) for b, rows in data[k].items()] for k in keys}
            tag = f"w{world}_{dtype}"
            line_chart(out / f"bandwidth_{tag}.svg", f"All-reduce bus bandwidth, {world} x B200, {dtype}", "bus bandwidth (GB/s)",
                       bw, hline=(link_gbs, f"peer copy {link_gbs:.0f}"))
            line_chart(out / f"latency_{tag}.svg", f"Time per call, {world} x B200, {dtype}", "microseconds per call", us,
                       logy=True)
            written += [f"bandwidth_{tag}.svg", f"latency_{tag}.svg"]
            nccl = next((k for k in keys if k[0] == "nccl"), None)
            if nccl:
                base = {b: mean(rows, "us") for b, rows in data[nccl].items()}
                sp = {label(k): [(b, base[b] / mean(rows, "us")) for b, rows in data[k].items() if b in base and mean(rows, "us")]
                      for k in keys if k != nccl}
                line_chart(out / f"speedup_{tag}.svg", f"Speed-up over NCCL, {world} x B200, {dtype}", "NCCL time / our time", sp,
                           hline=(1.0, "NCCL"))
                written.append(f"speedup_{tag}.svg")
            sol = {label(k): [(b, 100.0 * mean(rows, "busbw_gbps") / link_gbs) for b, rows in data[k].items()] for k in keys}
            line_chart(out / f"sol_{tag}.svg", f"Fraction of the measured peer-copy rate, {world} x B200, {dtype}",
                       "% of peer copy rate", sol, hline=(85.0, "85 %"))
            written.append(f"sol_{tag}.svg")
            cv = {}
            for k in keys:
                pts = []
                for b, rows in data[k].items():
                    v = [r["busbw_gbps"] for r in rows]
                    if len(v) > 1:
                        m = sum(v) / len(v)
                        sd = (sum((x - m) ** 2 for x in v) / (len(v) - 1)) ** 0.5
                        pts.append((b, 100.0 * sd / m if m else 0.0))
                if pts:
                    cv[label(k)] = pts
            if cv:
                line_chart(out / f"variation_{tag}.svg", f"Run-to-run variation, {world} x B200, {dtype}",
                           "coefficient of variation (%)", cv)
                written.append(f"variation_{tag}.svg")
            dev = {label(k): [(b, mean(rows, "dev_p99_us") / mean(rows, "dev_p50_us")) for b, rows in data[k].items()
                              if mean(rows, "dev_p50_us")] for k in keys}
            dev = {k: v for k, v in dev.items() if v}
            if dev:
                line_chart(out / f"tail_{tag}.svg", f"Device-timed tail, p99 / p50 per call, {world} x B200, {dtype}",
                           "p99 / p50", dev, hline=(1.1, "1.1"))
                written.append(f"tail_{tag}.svg")
        auto = {d: [(b, mean(rows, "busbw_gbps")) for b, rows in data[k].items()]
                for d in dtypes for k in data if k[:3] == ("yali_b200", world, d) and k[3] == "auto"}
        if len(auto) > 1:
            line_chart(out / f"dtypes_w{world}.svg", f"Automatic variant by dtype, {world} x B200", "bus bandwidth (GB/s)", auto)
            written.append(f"dtypes_w{world}.svg")
    auto_w = {f"{w} ranks": [(b, mean(rows, "busbw_gbps")) for b, rows in data[k].items()]
              for w in worlds for k in data if k[0] == "yali_b200" and k[1] == w and k[3] == "auto" and k[2] == "fp32"}
    if len(auto_w) > 1:
        line_chart(out / "worlds_fp32.svg", "Automatic variant by number of GPUs, fp32", "bus bandwidth (GB/s)", auto_w)
        written.append("worlds_fp32.svg")
    return written


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("runs", nargs="+")
    ap.add_argument("--out", default="report")
    ap.add_argument("--link-gbs", type=float, default=770.0)
    args = ap.parse_args()
    for f in make_all(args.runs, Path(args.out), args.link_gbs):
        print("wrote", f)


if __name__ == "__main__":
    main()
