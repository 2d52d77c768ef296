"""Training-health statistics: loss/grad-norm spike score, in-context-learning score, router entropy
and similarity. Reference: src/kohakuwullm/training/loop/health.py:14-88."""

from __future__ import annotations

import statistics
from collections import deque

import torch


class SpikeScore:
    """Robust z-score of the newest value against the median / MAD of the last ``window`` values; a score
    above ``threshold`` (7 sigma by default) is a spike."""

    def __init__(self, window: int = 1000, threshold: float = 7.0, min_history: int = 20):
        self.values: deque[float] = deque(maxlen=window)
        self.threshold, self.min_history = threshold, min_history

    def update(self, value: float) -> float:
        score = 0.0
        if len(self.values) >= self.min_history:
            med = statistics.median(self.values)
            mad = statistics.median(abs(v - med) for v in self.values) or 1e-12
            score = (value - med) / (1.4826 * mad)
        self.values.append(value)
        return score

    def is_spike(self, score: float) -> bool:
        return score > self.threshold


def icl_score(per_token_loss: torch.Tensor, early: int = 50, late: int = 500) -> float:
    """Loss at position ``late`` minus loss at position ``early`` of a document, averaged over a small
    neighbourhood: negative when the model uses its context."""
    if per_token_loss.numel() <= late:
        return float("nan")
    lo = per_token_loss[max(early - 5, 0): early + 5].float().mean()
    hi = per_token_loss[late - 5: late + 5].float().mean()
    return float(hi - lo)


def router_entropy(load: torch.Tensor) -> float:
    """Entropy of the expert load distribution divided by its maximum ``ln(E)`` (1 = perfectly even)."""
    p = load.float() / load.float().sum().clamp(min=1e-12)
    ent = -(p * torch.log(p.clamp(min=1e-12))).sum()
    return float(ent / torch.log(torch.tensor(float(load.numel()))))


def router_similarity(weight: torch.Tensor) -> float:
    """Mean absolute cosine similarity between different experts' gate vectors (0 = orthogonal)."""
    w = torch.nn.functional.normalize(weight.float(), dim=-1)
    sim = (w @ w.t()).abs()
    e = sim.shape[0]
    return float((sim.sum() - sim.diag().sum()) / max(e * (e - 1), 1))
