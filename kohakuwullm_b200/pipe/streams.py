"""Extra tensors that travel with the hidden state across a stage boundary.

The router auxiliary loss of every MoE layer has to reach the loss on the last stage. It rides as a
``(1,)`` fp32 *accumulator stream*: stage 0 creates it (``accumulator``), every stage adds its local
terms (``accumulate``) and the last stage folds it into the loss (``reduce_accumulator``). P2P receives
need a dense gradient for every received tensor, so ``reduce_accumulator`` routes the accumulator
through an op whose gradient is always a dense ``(1,)`` tensor even when no local term touched it.
Reference: src/kohakuwupipe/parallel/streams.py:14-66.
"""

from __future__ import annotations

from typing import NamedTuple

import torch


def accumulator(device=None) -> torch.Tensor:
    return torch.zeros(1, dtype=torch.float32, device=device, requires_grad=True)


def accumulate(acc: torch.Tensor, term: torch.Tensor | None) -> torch.Tensor:
    return acc if term is None else acc + term.reshape(1).to(acc.dtype)


def reduce_accumulator(acc: torch.Tensor) -> torch.Tensor:
    """Scalar view of the accumulator whose backward always produces a dense gradient."""
    return (acc * torch.ones_like(acc)).sum()


class GradCarrier(NamedTuple):
    """What a stage sends forward: the hidden state and, optionally, the accumulator stream."""

    hidden: torch.Tensor
    aux: torch.Tensor | None = None

    def tensors(self) -> tuple[torch.Tensor, ...]:
        return (self.hidden,) if self.aux is None else (self.hidden, self.aux)


def split_streams(tensors) -> GradCarrier:
    if isinstance(tensors, torch.Tensor):
        return GradCarrier(tensors, None)
    if len(tensors) == 1:
        return GradCarrier(tensors[0], None)
    return GradCarrier(tensors[0], tensors[1])
