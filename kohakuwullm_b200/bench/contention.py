"""Was the GPU exclusive while a sample loop ran, and could the check have noticed if it was not?

Plain arithmetic on sample times (no torch), so it is testable without a GPU. Two statistics:

* ``sample_spread``            ``(p90 - p10) / median``. A quiet card shows about 5 % plus a fixed timer floor
                               (10 us) relative to the median, so the threshold depends on how long the work is;
                               below ~50 us per sample the threshold passes 25 % and the test has no power.
* ``contended_fraction``       share of samples slower than 1.1 x the median. Another process on the card shows
                               up as a tail of slow samples; more than 1 % of them means "shared, discard".
                               Blind to a uniform slowdown (a clock cap), which the clock record covers instead.
                               Needs at least 100 samples to resolve a 1 % limit.
Reference: src/kohakuwullm/bench/core/contention.py:1-78.
"""

from __future__ import annotations

import math
import statistics

SPREAD_BASE = 0.05
SPREAD_FLOOR_MS = 0.010
SPREAD_NO_POWER = 0.25
CONTENDED_FACTOR = 1.1
CONTENDED_LIMIT = 0.01


def percentile(ordered: list[float], q: float) -> float:
    """Linear-interpolated quantile of an ascending list."""
    if len(ordered) == 1:
        return ordered[0]
    pos = q * (len(ordered) - 1)
    lo = int(pos)
    hi = min(lo + 1, len(ordered) - 1)
    return ordered[lo] + (pos - lo) * (ordered[hi] - ordered[lo])


def sample_spread(times: list[float]) -> float:
    if not times:
        return float("nan")
    ordered = sorted(times)
    med = statistics.median(ordered)
    return (percentile(ordered, 0.9) - percentile(ordered, 0.1)) / med if med else float("nan")


def contended_fraction(times: list[float], factor: float = CONTENDED_FACTOR) -> float:
    if not times:
        return float("nan")
    med = statistics.median(times)
    return sum(t > factor * med for t in times) / len(times) if med else float("nan")


def contended_fraction_min_iters() -> int:
    return math.ceil(1.0 / CONTENDED_LIMIT)


def spread_threshold(median_ms: float) -> float:
    """Largest spread a quiet card is expected to show for samples of this length."""
    if not median_ms or median_ms != median_ms:
        return SPREAD_BASE
    return SPREAD_BASE + SPREAD_FLOOR_MS / median_ms


def spread_has_power(median_ms: float) -> bool:
    """False when the work is so short that timer noise alone reaches the 'no power' spread."""
    return spread_threshold(median_ms) <= SPREAD_NO_POWER


def verdict(times: list[float]) -> dict:
    """One record per sample loop: the statistics, their thresholds and a plain-word reading."""
    med = statistics.median(times) if times else float("nan")
    spread, frac = sample_spread(times), contended_fraction(times)
    certifiable = spread_has_power(med) and len(times) >= contended_fraction_min_iters()
    if not certifiable:
        word = "too short or too few samples to certify exclusivity"
    elif frac > CONTENDED_LIMIT or spread > spread_threshold(med):
        word = "contended: discard"
    else:
        word = "clean"
    return {"median_ms": med, "spread": spread, "spread_threshold": spread_threshold(med),
            "contended_fraction": frac, "contended_limit": CONTENDED_LIMIT, "n": len(times),
            "certifiable": certifiable, "verdict": word}
