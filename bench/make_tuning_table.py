#!/usr/bin/env python
"""Builds a tuning table (the JSON that YALI_TUNING_FILE points at) from the result lines of
bench/sweep.py runs that timed the variants side by side:

    python bench/make_tuning_table.py --out tuning.json sweep_2gpu.jsonl sweep_4gpu.jsonl sweep_8gpu.jsonl

Per (world, element size, message size) the fastest of the forced variants wins; a variant must beat
the incumbent of the next smaller size by more than `--margin` (default 3 %) to take over, so that
timing noise does not make the table flip back and forth.  Rows of equal choice are merged into one
row per upper size bound.  The reference derived its thresholds by hand from sweeps
(src/include/yali_tuning.h:22-132); here the sweep writes them.
"""
from __future__ import annotations

import argparse
import json
from collections import defaultdict
from pathlib import Path

KERNEL_NAMES = {"flash": "flash", "stream": "stream", "nvls1": "nvls1", "nvls2": "nvls2"}


def load(paths):
    rows = []
    for p in paths:
        for line in Path(p).read_text().splitlines():
            if line.startswith("{"):
                rows.append(json.loads(line))
    return rows


def build(rows, margin: float = 0.03):
    """rows: sweep result lines.  Returns the list of table rows."""
    by_key = defaultdict(lambda: defaultdict(dict))  # (world, elem_bytes) -> bytes -> kernel -> best us
    for r in rows:
        if r.get("impl") != "yali_b200" or r.get("variant") == "auto" or r.get("emulated"):
            continue
        kernel = KERNEL_NAMES.get(r.get("kernel"))
        if kernel is None:
            continue
        esz = 4 if r["dtype"] == "fp32" else 2
        slot = by_key[(r["world"], esz)][r["bytes"]]
        if kernel not in slot or r["us"] < slot[kernel]["us"]:
            slot[kernel] = r
    table = []
    for (world, esz), sizes in sorted(by_key.items()):
        incumbent = None
        picks = []
        for size in sorted(sizes):
            cands = sizes[size]
            best = min(cands, key=lambda k: cands[k]["us"])
            if incumbent in cands and cands[incumbent]["us"] <= cands[best]["us"] * (1.0 + margin):
                best = incumbent
            incumbent = best
            picks.append((size, best, cands[best]))
        for i, (size, kernel, r) in enumerate(picks):
            last_of_run = i + 1 == len(picks) or picks[i + 1][1] != kernel
            if last_of_run:
                bound = size if i + 1 < len(picks) else 1 << 40  # the largest measured choice holds beyond it
                table.append({"world": world, "elem_bytes": esz, "max_bytes": bound, "variant": kernel, "ctas": 0,
                              "slot_bytes": 0, "busbw": r["busbw_gbps"]})
    return table


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("runs", nargs="+")
    ap.add_argument("--out", required=True)
    ap.add_argument("--margin", type=float, default=0.03)
    args = ap.parse_args()
    table = build(load(args.runs), args.margin)
    Path(args.out).write_text(json.dumps({"rows": table}, indent=1) + "\n")
    print(f"wrote {args.out}: {len(table)} row(s)")


if __name__ == "__main__":
    main()
