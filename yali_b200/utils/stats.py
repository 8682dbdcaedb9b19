"""Run-level statistics of benchmark samples (mean, spread, percentiles, CV).
Reference counterpart: `BenchStats` in scripts/sweep.py:129-179."""
from __future__ import annotations

import math
from dataclasses import asdict, dataclass
from typing import Dict, Sequence


@dataclass
class BenchStats:
    mean: float = 0.0
    stddev: float = 0.0
    min: float = 0.0
    max: float = 0.0
    p50: float = 0.0
    p90: float = 0.0
    p95: float = 0.0
    p99: float = 0.0
    cv_pct: float = 0.0
    samples: int = 0

    def as_dict(self) -> Dict[str, float]:
        return asdict(self)


def percentile(sorted_values: Sequence[float], q: float) -> float:
    """Linear-interpolated percentile of an ascending sequence (q in 0..100)."""
    if not sorted_values:
        return 0.0
    pos = q / 100.0 * (len(sorted_values) - 1)
    lo = int(math.floor(pos))
    hi = min(len(sorted_values) - 1, lo + 1)
    return sorted_values[lo] + (sorted_values[hi] - sorted_values[lo]) * (pos - lo)


def summarise(values: Sequence[float]) -> BenchStats:
    v = sorted(float(x) for x in values)
    if not v:
        return BenchStats()
    mean = sum(v) / len(v)
    var = sum((x - mean) ** 2 for x in v) / (len(v) - 1) if len(v) > 1 else 0.0
    sd = math.sqrt(var)
    return BenchStats(mean=mean, stddev=sd, min=v[0], max=v[-1], p50=percentile(v, 50), p90=percentile(v, 90),
                      p95=percentile(v, 95), p99=percentile(v, 99), cv_pct=100.0 * sd / mean if mean else 0.0,
                      samples=len(v))
