"""``PipelineModule``: the user-facing contract of the pipeline trainer (Lightning-like).

A subclass builds this rank's stage(s), says what crosses a stage boundary, how the last stage turns
hidden states into a SUMMED loss, and which optimizer to use. The trainer owns construction order,
schedules, optimizer stepping and checkpoints. Reference: src/kohakuwupipe/training/module.py:18-167.
"""

from __future__ import annotations

from typing import Any, Sequence

import torch
from torch import nn

from kohakuwullm_b200.pipe.plan import StagePlan


class PipelineModule:
    def __init__(self):
        self.stages: list[nn.Module] = []
        self.plans: list[StagePlan] = []
        self.rank = 0
        self.world = 1
        self.device = torch.device("cpu")
        self._metrics: dict[str, list] = {}

    # ------------------------------------------------------------------ construction
    def setup(self, plans: Sequence[StagePlan], rank: int, world: int, device) -> None:
        """Build one stage (``configure_model``) per plan this rank owns."""
        self.plans, self.rank, self.world, self.device = list(plans), rank, world, torch.device(device)
        self.stages = [self.configure_model(p, rank, world, self.device) for p in self.plans]

    def configure_model(self, plan: StagePlan, rank: int, world: int, device) -> nn.Module:
        raise NotImplementedError

    def configure_optimizers(self):
        """Return ``optimizer`` or ``(optimizer, scheduler)``; the optimizer must expose ``step`` and
        ``zero_grad`` and, for portable checkpoints, a named ``state_dict``."""
        raise NotImplementedError

    def boundary_example(self, plan: StagePlan) -> tuple[torch.Tensor, ...]:
        """Tensors with the shape / dtype of what arrives at ``plan``'s input."""
        raise NotImplementedError

    # ------------------------------------------------------------------ per step
    def set_batch(self, batch: Any) -> None:
        """Install the step's micro-batches (layouts, tokens on the first stage, labels on the last)."""
        raise NotImplementedError

    def num_microbatches(self, batch: Any) -> int:
        raise NotImplementedError

    def loss(self, output, micro_index: int) -> torch.Tensor:
        """SUM loss of one micro-batch on the last stage (the trainer divides by the token count)."""
        raise NotImplementedError

    def step_tokens(self, batch: Any) -> int:
        """Trained tokens of the whole step (every rank must return the same number)."""
        raise NotImplementedError

    def post_step(self) -> None:
        """After the optimizer step (refresh quantised weights, update router biases, ...)."""

    def validation_step(self, batch: Any):
        raise NotImplementedError

    # ------------------------------------------------------------------ metrics without host syncs
    def log(self, name: str, value) -> None:
        self._metrics.setdefault(name, []).append(value.detach() if torch.is_tensor(value) else value)

    def pop_metrics(self) -> dict[str, torch.Tensor]:
        """Mean of every logged value since the last pop, as device tensors (read them on an interval)."""
        out = {}
        for k, vals in self._metrics.items():
            ts = [v if torch.is_tensor(v) else torch.tensor(float(v)) for v in vals]
            out[k] = torch.stack([t.float().reshape(()) for t in ts]).mean()
        self._metrics.clear()
        return out

    # ------------------------------------------------------------------ checkpoint hooks
    def on_save_checkpoint(self, checkpoint: dict) -> None:
        pass

    def on_load_checkpoint(self, checkpoint: dict) -> None:
        pass

    def global_names(self) -> dict[str, str]:
        """local parameter name -> whole-model name, over all local stages."""
        return {}
