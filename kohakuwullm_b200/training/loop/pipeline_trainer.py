"""``PipelinedLMTrainer``: the language-model trainer under pipeline parallelism, with the surface of
``LMTrainer`` (preset + overrides in, ``fit`` / ``generate`` / checkpoints out).

It assembles what the pipeline entry point assembles by hand: the stage plan (analytic, measured, or a
pinned ``layers`` list), the ``LMPipelineModule`` (this rank's ``LMStage`` slices, stage-local optimizer,
MXFP8 conversion per stage), and the ``PipelineTrainer`` (schedule + loop). Weights and optimizer state are
saved under whole-model names, so a checkpoint written here loads into ``LMTrainer``, into a different split,
or into a single GPU. ``generate`` is collective: every rank drives the forward-only pipelined decode and
rank 0 ... last rank samples; all ranks return the same tokens.
Reference: src/kohakuwullm/training/loop/pipeline_trainer.py:24-257.
"""

from __future__ import annotations

from typing import Any, Iterable, Sequence

import torch
import torch.distributed as dist


class PipelinedLMTrainer:
    def __init__(self, arch: str | Any = "Kohaku-MoE-1B", arch_overrides: dict | None = None, *,
                 micro_tokens: int = 4096, num_microbatches: int = 16, schedule: str = "1f1b",
                 layers: Sequence[int] | None = None, autotune: bool = False, lr: float = 3e-4,
                 weight_decay: float = 0.1, max_grad_norm: float | None = 1.0, seed: int = 1234,
                 param_dtype: torch.dtype | None = None, callbacks=(), device=None, group=None,
                 optimizer: str = "fused_adamw", optimizer_kwargs: dict | None = None, lr_schedule: dict | None = None,
                 head_only_stage: bool = False):
        from kohakuwullm_b200.models import get_preset
        from kohakuwullm_b200.models.presets import LMArchConfig
        from kohakuwullm_b200.pipe.trainer import PipelineTrainer
        from kohakuwullm_b200.training.parallel.pipeline import plan_for
        from kohakuwullm_b200.training.parallel.uwupipe import LMPipelineModule

        self.rank = dist.get_rank(group) if dist.is_available() and dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.device, self.group = torch.device(device), group
        self.config = arch if isinstance(arch, LMArchConfig) else get_preset(arch, **(arch_overrides or {}))
        multi = schedule in ("interleaved-1f1b", "looped-bfs", "interleaved-zb", "zbv", "dualpipe-v")
        chunks = 2 if multi else 1
        costs = None
        if autotune and layers is None:
            from kohakuwullm_b200.training.parallel.autotune import broadcast_costs, measure_costs

            measured = measure_costs(self.config, micro_tokens, self.device) if self.rank == 0 else None
            costs = broadcast_costs(measured, self.config.depth, self.device)
        self.plans = plan_for(self.config, self.world * chunks, micro_tokens, layers=layers, costs=costs,
                              style="v" if schedule in ("zbv", "dualpipe-v") else "loop",
                              allow_empty_last=head_only_stage and costs is not None)
        kw = {} if param_dtype is None else {"param_dtype": param_dtype}
        self.module = LMPipelineModule(self.config, micro_tokens=micro_tokens, lr=lr, weight_decay=weight_decay,
                                       seed=seed, group=group, optimizer=optimizer, optimizer_kwargs=optimizer_kwargs,
                                       lr_schedule=lr_schedule, **kw)
        self.trainer = PipelineTrainer(self.module, self.plans, rank=self.rank, world=self.world, device=self.device,
                                       n_micro=num_microbatches, schedule=schedule, max_grad_norm=max_grad_norm,
                                       callbacks=list(callbacks), group=group)

    # ------------------------------------------------------------------ training
    @property
    def global_step(self) -> int:
        return self.trainer.loop.global_step

    def training_step(self, micro_batches):
        """One optimizer step over ``num_microbatches`` packed micro-batches (the same list on every rank)."""
        return self.trainer.loop.step(micro_batches)

    def fit(self, batches: Iterable, max_steps: int):
        return self.trainer.fit(batches, max_steps)

    # ------------------------------------------------------------------ state
    def gathered_state_dict(self) -> dict:
        """Whole-model weights on every rank, keyed by whole-model names (collective)."""
        from kohakuwullm_b200.pipe.checkpoint import gather_state_dict

        merged: dict = {}
        for stage in self.module.stages:
            merged.update(gather_state_dict(stage, stage.global_names(), group=self.group))
        return merged

    def load_gathered_state_dict(self, state: dict) -> None:
        """Load whole-model weights: every stage keeps the entries of its own layers."""
        for stage in self.module.stages:
            local = {loc: state[glob] for loc, glob in stage.global_names().items() if glob in state}
            stage.load_state_dict(local, strict=False)

    def save_checkpoint(self, path: str) -> None:
        self.trainer.save_checkpoint(path)

    def load_checkpoint(self, path: str) -> dict:
        return self.trainer.load_checkpoint(path)

    # ------------------------------------------------------------------ generation
    @torch.no_grad()
    def generate(self, prompt: torch.Tensor, max_new_tokens: int, **sampling) -> torch.Tensor:
        from kohakuwullm_b200.generation.engine import LocalGenerator, PipelineGenerator

        stage = self.module.stages[0]
        if self.world == 1:
            return PipelineGenerator(stage, 0, 1, group=self.group).generate(prompt.to(self.device), max_new_tokens, **sampling) \
                if hasattr(stage, "is_first") else LocalGenerator(stage).generate(prompt, max_new_tokens, **sampling)
        if len(self.module.stages) != 1:
            raise RuntimeError("pipelined decode drives one stage per rank; gather the weights and decode locally instead")
        gen = PipelineGenerator(stage, self.rank, self.world, group=self.group)
        return gen.generate(prompt.to(self.device), max_new_tokens, **sampling)
