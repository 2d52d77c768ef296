"""Output head: projection to the vocabulary and the per-token losses.

``token_loss`` always returns fp32 per-token cross-entropy (zero on ignored positions) plus the
per-token log-sum-exp, from ONE pass over the vocabulary; ``loss`` reduces them and adds the z-loss
``z_w * sum(lse^2)``. The logits are materialised only by ``logits()`` (generation) and by the
soft-capped path. Reference: src/kohakuwullm/models/head.py:18-180.
"""

from __future__ import annotations

import torch
from torch import nn

from kohakuwullm_b200.models.components.mlp import Linear
from kohakuwullm_b200.ops.gemm import linear
from kohakuwullm_b200.ops.loss import IGNORE_INDEX, linear_cross_entropy


class LMHead(nn.Module):
    def __init__(self, dim: int, vocab_size: int, tied_weight: nn.Parameter | None = None,
                 z_loss_weight: float = 0.0, logit_soft_cap: float | None = None, chunk: int = 8192,
                 ignore_index: int = IGNORE_INDEX, kernel: str = "fused", **_unused):
        super().__init__()
        self.dim, self.vocab_size = dim, vocab_size
        self.z_loss_weight = z_loss_weight
        self.logit_soft_cap = logit_soft_cap
        self.chunk = chunk
        self.ignore_index = ignore_index
        self.kernel = kernel
        if tied_weight is None:
            self.proj = Linear(dim, vocab_size)
            self._tied = None
        else:
            self.proj = None
            self._tied = [tied_weight]  # held in a list so it is not registered twice

    @property
    def weight(self) -> torch.Tensor:
        return self.proj.weight if self.proj is not None else self._tied[0]

    @property
    def tied(self) -> bool:
        return self.proj is None

    def untie(self) -> None:
        """Give the head its own copy of the embedding (needed when they live on different stages)."""
        if self.proj is None:
            w = self._tied[0]
            self.proj = Linear(self.dim, self.vocab_size).to(device=w.device, dtype=w.dtype)
            with torch.no_grad():
                self.proj.weight.copy_(w)
            self._tied = None

    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        out = linear(hidden, self.weight).float()
        if self.logit_soft_cap:
            out = self.logit_soft_cap * torch.tanh(out / self.logit_soft_cap)
        return out

    def token_loss(self, hidden: torch.Tensor, labels: torch.Tensor):
        h2 = hidden.reshape(-1, hidden.shape[-1])
        return linear_cross_entropy(h2, self.weight, labels.reshape(-1), ignore_index=self.ignore_index,
                                    chunk=self.chunk, soft_cap=self.logit_soft_cap)

    def loss(self, hidden: torch.Tensor, labels: torch.Tensor, reduction: str = "mean"):
        """Returns ``(loss, logs)`` with ``logs = {ce, n_tokens, z_loss}`` as device tensors."""
        ce, lse = self.token_loss(hidden, labels)
        valid = labels.reshape(-1) != self.ignore_index
        n_valid = valid.sum()
        ce_sum = ce.sum()
        logs = {"ce": ce_sum.detach(), "n_tokens": n_valid}
        total = ce_sum
        if self.z_loss_weight:
            z = self.z_loss_weight * (lse.pow(2) * valid).sum()
            logs["z_loss"] = z.detach()
            total = total + z
        if reduction == "mean":
            total = total / n_valid.clamp(min=1)
        elif reduction != "sum":
            raise ValueError(f"reduction must be 'sum' or 'mean', got {reduction!r}")
        return total, logs
