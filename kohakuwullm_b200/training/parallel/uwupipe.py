"""``LMPipelineModule``: the language-model adapter of the pipeline engine.

Per stage it builds the backbone, slices it (``LMStage``), casts parameters to the training dtype
(norm / router / rotary / sink / bias stay fp32), converts the stage's linears to MXFP8 and creates a
flat-buffer fused AdamW over the stage's own parameters. Every rank receives the SAME step batch (a
list of packed micro-batches); stage 0 uses the tokens, the last stage the labels, nothing else is
moved. ``verify_same_batch`` compares a 4-number fp64 signature of the first batch across ranks.
Reference: src/kohakuwullm/training/parallel/uwupipe.py:44-313.
"""

from __future__ import annotations

from typing import Sequence

import torch
import torch.distributed as dist

from kohakuwullm_b200.data.packing import PackedBatch
from kohakuwullm_b200.models.backbone import LMBackbone
from kohakuwullm_b200.models.presets import LMArchConfig
from kohakuwullm_b200.parallel.flat import FlatParameters
from kohakuwullm_b200.pipe.module import PipelineModule
from kohakuwullm_b200.pipe.plan import StagePlan
from kohakuwullm_b200.training.optim.fused_adamw import FlatAdamW
from kohakuwullm_b200.training.optim.lowbit import cast_parameters_
from kohakuwullm_b200.training.parallel.pipeline import LMStage, model_has_router_loss


def batch_signature(batch: Sequence[PackedBatch]) -> torch.Tensor:
    toks = torch.cat([b.tokens.reshape(-1).double().cpu() for b in batch])
    labs = torch.cat([b.labels.reshape(-1).double().cpu() for b in batch])
    idx = torch.arange(1, toks.numel() + 1, dtype=torch.float64)
    return torch.stack([toks.sum(), (toks * idx).sum() / idx.sum(), labs.sum(), torch.tensor(float(toks.numel()), dtype=torch.float64)])


def verify_same_batch(batch: Sequence[PackedBatch], device, group=None) -> None:
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return
    sig = batch_signature(batch)
    if dist.get_backend(group) == "nccl":
        sig = sig.to(device)
    parts = [torch.empty_like(sig) for _ in range(dist.get_world_size(group))]
    dist.all_gather(parts, sig, group=group)
    for r, other in enumerate(parts):
        if not torch.equal(other.cpu(), parts[0].cpu()):
            raise RuntimeError(f"rank {r} loaded a different batch than rank 0: pipeline ranks must iterate "
                               f"identical data ({other.tolist()} vs {parts[0].tolist()})")


class LMPipelineModule(PipelineModule):
    def __init__(self, config: LMArchConfig, *, micro_tokens: int, lr: float = 3e-4, betas=(0.9, 0.95),
                 weight_decay: float = 0.1, param_dtype: torch.dtype | None = torch.bfloat16,
                 seed: int = 1234, lr_schedule=None, group=None, cuda_graphs: bool | None = None,
                 optimizer: str = "fused_adamw", optimizer_kwargs: dict | None = None):
        """``cuda_graphs``: replay every stage's forward + backward of a micro-batch from CUDA graphs (default: on
        for CUDA devices with the native kernels, single stage per rank, GPipe / 1F1B). ``optimizer``: the flat
        one-launch AdamW, or any registered name (``muon``, ``adamw16``, ``adamw8bit``, ...), built over this rank's
        stage with the usual grouping rules."""
        super().__init__()
        self.config, self.micro_tokens = config, micro_tokens
        self.lr, self.betas, self.weight_decay = lr, betas, weight_decay
        self.param_dtype, self.seed, self.lr_schedule, self.group = param_dtype, seed, lr_schedule, group
        self._labels: list[torch.Tensor] = []
        self._infos: list = []
        self._checked = False
        self._router_scale = 1.0            # a device scalar once the stage exists (graphs read it in place)
        self.cuda_graphs = cuda_graphs
        self.optimizer_name, self.optimizer_kwargs = optimizer, dict(optimizer_kwargs or {})

    # ------------------------------------------------------------------ construction
    def configure_model(self, plan: StagePlan, rank: int, world: int, device) -> LMStage:
        torch.manual_seed(self.seed)  # every rank builds the same whole model, then keeps its slice
        cfg = self.config.replace(mxfp8=False)
        backbone = LMBackbone(cfg)
        stage = LMStage(backbone, plan, boundary_dtype=None)
        del backbone
        stage.to(device)
        dtype = self.param_dtype if torch.device(device).type == "cuda" else None
        if dtype is not None and dtype != torch.float32:
            cast_parameters_(stage, dtype)
        if self.config.mxfp8 and torch.device(device).type == "cuda":
            from kohakuwullm_b200.models.mxfp8_swap import swap_mxfp8

            report = swap_mxfp8(stage)
            if report.blocking:
                raise RuntimeError(f"MXFP8 conversion incomplete on stage {plan.index}: {report.blocking}")
        return stage

    def configure_optimizers(self):
        params = self.stages[0] if len(self.stages) == 1 else torch.nn.ModuleList(self.stages)
        self.flat = FlatParameters(params)
        self._flat_names = {f"{i}.{k}": v for i, st in enumerate(self.stages) for k, v in st.global_names().items()}
        if self.optimizer_name == "fused_adamw":
            opt = FlatAdamW(self.flat, lr=self.lr, betas=self.betas, weight_decay=self.weight_decay)
        else:
            from kohakuwullm_b200.training.optim.build import MainGradOptimizer, build_optimizer

            inner = build_optimizer(params, self.optimizer_name, lr=self.lr, weight_decay=self.weight_decay,
                                    betas=self.betas, **self.optimizer_kwargs)
            opt = MainGradOptimizer(inner, self.flat, params)
        if self.lr_schedule is None:
            return opt
        from kohakuwullm_b200.utils.schedule import GroupLRSchedule, build_schedule

        fn = self.lr_schedule if callable(self.lr_schedule) else build_schedule(dict(self.lr_schedule))
        return opt, GroupLRSchedule(opt, fn)

    def boundary_example(self, plan: StagePlan):
        dtype = next(p for p in self.stages[0].parameters() if p.dim() >= 2).dtype
        hidden = torch.zeros(self.micro_tokens, self.config.dim, dtype=dtype, device=self.device)
        if model_has_router_loss(self.config):
            return (hidden, torch.zeros(1, dtype=torch.float32, device=self.device))
        return (hidden,)

    def first_input_example(self):
        return (torch.zeros(self.micro_tokens, dtype=torch.long, device=self.device),)

    def native_stage_fns(self, stage, plan: StagePlan, n_stages: int, n_micro: int, schedule: str):
        """``(stage_fn, loss_fn)`` for the native GPipe / 1F1B schedule with the stage replayed from CUDA graphs,
        or None to run it eagerly. One graph pair per micro-batch in flight on this stage."""
        from kohakuwullm_b200.ops import native

        on = self.cuda_graphs
        if on is None:
            on = self.device.type == "cuda" and native.available()
        if not on or self.device.type != "cuda":
            return None
        from kohakuwullm_b200.training.parallel.graphed_stage import GraphedLMStage

        slots = n_micro if schedule == "gpipe" else min(n_stages - plan.index - 1, n_micro) + 1
        graphed = GraphedLMStage(self, stage, slots, self.micro_tokens)
        return graphed, ((lambda out, mb: out) if stage.is_last else None)

    def global_names(self) -> dict[str, str]:
        if len(self.stages) == 1:
            return self.stages[0].global_names()
        return dict(self._flat_names)

    # ------------------------------------------------------------------ per step
    def set_batch(self, batch: Sequence[PackedBatch]) -> None:
        if not self._checked:
            verify_same_batch(batch, self.device, self.group)
            self._checked = True
        infos = [b.seq_info.to(self.device, non_blocking=True) for b in batch]
        self._infos = infos
        for stage in self.stages:
            stage.set_seq_info(infos)
            if stage.is_first:
                stage.set_tokens([b.tokens.to(self.device, non_blocking=True) for b in batch])
            if stage.is_last:
                self._labels = [b.labels.to(self.device, non_blocking=True) for b in batch]
        tokens = self.step_tokens(batch)
        scale = tokens / max(len(batch), 1)
        if not torch.is_tensor(self._router_scale):
            self._router_scale = torch.ones((), dtype=torch.float32, device=self.device)
        self._router_scale.fill_(scale)

    def num_microbatches(self, batch) -> int:
        return len(batch)

    def step_tokens(self, batch) -> int:
        return sum(b.trained_tokens() for b in batch)

    def loss_from(self, output, labels: torch.Tensor):
        """``(summed loss, summed cross-entropy)`` of one micro-batch's last-stage output."""
        from kohakuwullm_b200.pipe import streams

        last = next(s for s in self.stages if s.is_last)
        hidden, aux = (output if isinstance(output, (tuple, list)) else (output, None))
        loss, logs = last.head.loss(hidden, labels, reduction="sum")
        if aux is not None:
            loss = loss + streams.reduce_accumulator(aux) * self._router_scale
        return loss, logs["ce"]

    def loss(self, output, micro_index: int) -> torch.Tensor:
        loss, ce = self.loss_from(output, self._labels[micro_index])
        self.log("ce_sum", ce)
        return loss

    def forward_backward(self, schedule, batch, n_micro: int):
        from kohakuwullm_b200.pipe.schedules import NativeSchedule

        if isinstance(schedule, NativeSchedule):
            return schedule.step(n_micro)
        first = next((s for s in self.stages if s.is_first), None)
        tokens = torch.cat([b.tokens.to(self.device) for b in batch]) if first is not None else None
        target = torch.arange(n_micro, device=self.device).reshape(n_micro, 1)
        return schedule.step(tokens, target)

    def post_step(self) -> None:
        for stage in self.stages:
            if self.config.mxfp8:
                from kohakuwullm_b200.models.mxfp8_swap import refresh_mxfp8_weights

                refresh_mxfp8_weights(stage)
            stage.update_router_bias()
