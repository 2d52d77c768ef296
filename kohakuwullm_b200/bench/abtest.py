"""Loss-gap A/B analysis: is arm B's loss curve distinguishable from arm A's given the replicate noise floor?
The gap is the mean loss difference over the final ``window`` steps; the floor is the same statistic between
two runs of the SAME arm (different seeds / nondeterminism). A gap inside the floor is "within noise".
Reference: src/kohakuwullm/bench/analysis/abtest.py, loss_gap.py, admissibility.py."""

from __future__ import annotations

import statistics
from typing import Sequence


def final_window_mean(losses: Sequence[float], window: int = 100) -> float:
    tail = list(losses)[-window:]
    return statistics.fmean(tail)


def loss_gap(a: Sequence[float], b: Sequence[float], window: int = 100) -> float:
    return final_window_mean(b, window) - final_window_mean(a, window)


def windowed_gaps(a: Sequence[float], b: Sequence[float], window: int = 100) -> list[float]:
    n = min(len(a), len(b))
    return [statistics.fmean(b[i:i + window]) - statistics.fmean(a[i:i + window]) for i in range(0, n - window + 1, window)]


def noise_floor(replicates: Sequence[Sequence[float]], window: int = 100) -> float:
    """Largest absolute final-window gap between any two replicates of one arm."""
    finals = [final_window_mean(r, window) for r in replicates]
    return max(abs(x - y) for i, x in enumerate(finals) for y in finals[i + 1:]) if len(finals) > 1 else 0.0


def admissible(gap: float, floor: float, slack: float = 1.5) -> bool:
    return abs(gap) <= slack * floor
