"""Integer helpers and latency statistics.

Same names and results as the reference's python/pplx_garden/utils/math.py:5-109, so
benchmark output stays comparable (percentiles use its "midpoint between neighbours"
rule, not numpy's interpolation).
"""

from __future__ import annotations

import math
from dataclasses import dataclass, fields


def round_up(n: int, m: int) -> int:
    return -(-n // m) * m


def ceil_div(n: int, m: int) -> int:
    return -(-n // m)


def floor_div(n: int, m: int) -> int:
    return n // m


def mean(xs: list[float]) -> float:
    return math.fsum(xs) / len(xs) if xs else 0.0


def stddev(xs: list[float]) -> float:
    """Sample standard deviation (n - 1 in the denominator; 0 for fewer than two samples)."""
    if len(xs) < 2:
        return 0.0
    mu = mean(xs)
    return math.sqrt(math.fsum((x - mu) ** 2 for x in xs) / (len(xs) - 1))


def mean_and_stddev(xs: list[float]) -> tuple[float, float]:
    return mean(xs), stddev(xs)


_PERCENTILES = (("p01", 0.01), ("p25", 0.25), ("p50", 0.5), ("p75", 0.75), ("p95", 0.95), ("p99", 0.99))


@dataclass
class Statistics:
    mean: float
    stddev: float
    min: float
    p01: float
    p25: float
    p50: float
    p75: float
    p95: float
    p99: float
    max: float

    @classmethod
    def create(cls, xs: list[float]) -> "Statistics":
        if not xs:
            return cls(**{f.name: 0.0 for f in fields(cls)})
        ordered = sorted(xs)
        n = len(ordered)

        def pick(p: float) -> float:
            pos = n * p
            idx = int(pos)
            if pos == idx or idx + 1 >= n:
                return ordered[min(idx, n - 1)]
            return 0.5 * (ordered[idx] + ordered[idx + 1])

        mu, sigma = mean_and_stddev(xs)
        return cls(mean=mu, stddev=sigma, min=ordered[0], max=ordered[-1],
                   **{name: pick(p) for name, p in _PERCENTILES})

    def __str__(self) -> str:
        parts = [f"mean={self.mean:.1f}±{self.stddev:.1f} μs"]
        for name in ("min", "p01", "p25", "p50", "p75", "p95", "p99", "max"):
            parts.append(f"{name}={getattr(self, name):.1f} μs")
        return ", ".join(parts)
