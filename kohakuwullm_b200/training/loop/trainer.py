"""``LMTrainer``: the data-parallel trainer (the role of the reference's Lightning ``LMTrainer``).

Construction: architecture = preset + overrides -> ``LMBackbone`` -> ``TrainEngine`` (bf16 parameters, flat
fused AdamW, token-exact accumulation, fused gradient sync on N > 1). ``fit`` pulls optimizer-step batches
from a loader, splits each into ``grad_accum`` document-aligned micro-batches, steps, keeps exact int64
token / fp64 FLOP counters, calls callbacks, and checkpoints whole-model-named weights + optimizer state +
run state (counters, EMA loss, RNG, loader position). Nothing returns early on a rank (every rank takes
part in every collective). Reference: src/kohakuwullm/training/loop/trainer.py:42-472.
"""

from __future__ import annotations

import math
import os
import time
from typing import Any, Iterable

import torch
import torch.distributed as dist

from kohakuwullm_b200.data.packing import PackedBatch, split_packed
from kohakuwullm_b200.models import LMBackbone, get_preset
from kohakuwullm_b200.models.flops import FlopCounter
from kohakuwullm_b200.ops import native
from kohakuwullm_b200.pipe import checkpoint as ckpt
from kohakuwullm_b200.pipe.hooks import CallbackList
from kohakuwullm_b200.training.engine import TrainEngine
from kohakuwullm_b200.training.loop import resume
from kohakuwullm_b200.training.loop.tokens import TokenSnapshot, all_reduce_
from kohakuwullm_b200.utils.logging import get_logger
from kohakuwullm_b200.utils.schedule import build_schedule

log = get_logger("train")


class LMTrainer:
    def __init__(self, arch: str | Any = "Kohaku-500M", arch_overrides: dict | None = None, *, lr: float = 3e-4,
                 betas=(0.9, 0.95), weight_decay: float = 0.1, max_grad_norm: float = 1.0, grad_accum: int = 1,
                 lr_schedule: dict | None = None, param_dtype: torch.dtype | None = torch.bfloat16,
                 device=None, group=None, grad_sync: str = "auto", callbacks=(), log_interval: int = 10,
                 ema: float = 0.98, seed: int = 1234, head_kwargs: dict | None = None,
                 optimizer: str = "fused_adamw", optimizer_kwargs: dict | None = None, expert_parallel: bool = False,
                 ep_capacity_factor: float = 2.0, ep_on_overflow: str = "raise", grad_compress: str | None = None,
                 eps: float = 1e-8):
        self.rank = dist.get_rank(group) if dist.is_available() and dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
        self.group = group
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.device = torch.device(device)
        self.config = get_preset(arch, **(arch_overrides or {})) if isinstance(arch, str) else arch
        torch.manual_seed(seed)
        with torch.device(self.device):
            self.backbone = LMBackbone(self.config, head_kwargs=head_kwargs)
        sched = build_schedule(lr_schedule)
        if grad_sync == "auto":
            grad_sync = "fused" if (self.world > 1 and self.device.type == "cuda" and optimizer == "fused_adamw") else "nccl"
        dtype = param_dtype if self.device.type == "cuda" else None
        self.engine = TrainEngine(self.backbone, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, max_grad_norm=max_grad_norm,
                                  param_dtype=dtype, group=group, grad_sync=grad_sync,
                                  lr_schedule=(lambda step: lr * sched(step)), optimizer=optimizer,
                                  optimizer_kwargs=optimizer_kwargs, expert_parallel=expert_parallel,
                                  ep_capacity_factor=ep_capacity_factor, ep_on_overflow=ep_on_overflow,
                                  grad_compress=grad_compress)
        self.flops = FlopCounter(self.backbone)
        self.grad_accum, self.log_interval, self.ema_beta = grad_accum, log_interval, ema
        self.callbacks = CallbackList(callbacks)
        self.global_step = 0
        self.loss_ema: float | None = None
        self._local = TokenSnapshot()
        self._offset = TokenSnapshot()      # totals restored from a checkpoint
        self._t0 = None
        self.loader = None

    # ------------------------------------------------------------------ counters
    def snapshot(self, sync: bool = False) -> TokenSnapshot:
        """Global totals: this run's counters summed over ranks plus what the checkpoint carried."""
        local = self._local
        if self._t0 is not None:
            local = TokenSnapshot(local.seen, local.trained, local.model_flops, local.hardware_flops,
                                  time.perf_counter() - self._t0)
        total = all_reduce_(local, self.device, self.group) if sync else local
        return total + self._offset

    # ------------------------------------------------------------------ step
    def training_step(self, batch: PackedBatch) -> dict:
        if batch.seq_info.packed:
            micro = split_packed(batch, self.grad_accum) if self.grad_accum > 1 else [batch]
            lengths = batch.seq_info.lengths or tuple(batch.seq_info.seqlens.tolist())
        else:       # padded rows: split along the batch axis; FLOPs count the documents' own lengths, not the padding
            from kohakuwullm_b200.data.loader.padded import split_padded

            micro = split_padded(batch, self.grad_accum) if self.grad_accum > 1 else [batch]
            lengths = tuple(int(n) for n in batch.lengths.tolist())
        out = self.engine.step(micro)
        mf, hf = self.flops.step_flops(lengths)
        self._local = self._local + TokenSnapshot(batch.num_tokens, batch.trained_tokens(), mf, hf, 0.0)
        return out

    def fit(self, loader: Iterable[PackedBatch], max_steps: int):
        self.loader = loader
        cb = self.callbacks
        cb.on_fit_start(self)
        cb.on_train_start(self)
        self._t0 = time.perf_counter()
        try:
            it = iter(loader)
            # the stop test comes BEFORE pulling: a batch that is fetched but not trained on would be
            # skipped by a run resumed from the loader position
            while self.global_step < max_steps:
                try:
                    batch = next(it)
                except StopIteration:
                    break
                cb.on_train_batch_start(self, batch, self.global_step)
                out = self.training_step(batch)
                self.global_step += 1
                if self.global_step % self.log_interval == 0:
                    loss = float(out["loss"])      # the only host read, on the logging interval
                    if self.device.type == "cuda":
                        native.check_status()      # the device is idle here anyway: read the status word itself
                    out["loss_host"] = loss
                    if math.isfinite(loss):
                        self.loss_ema = loss if self.loss_ema is None else self.ema_beta * self.loss_ema + (1 - self.ema_beta) * loss
                    extra = {k: float(v) for k, v in self.engine.last_router_stats.items()}
                    log.info("train", step=self.global_step, loss=loss, loss_ema=self.loss_ema,
                             ppl=math.exp(min(float(out["ce"]), 20.0)), grad_norm=float(out["grad_norm"]),
                             lr=self.engine.optimizer.param_groups[0]["lr"], **extra)
                cb.on_train_batch_end(self, out, batch, self.global_step)
        except BaseException as exc:  # noqa: BLE001
            cb.on_exception(self, exc)
            raise
        cb.on_train_end(self)
        cb.on_fit_end(self)

    @torch.no_grad()
    def validate(self, loader: Iterable[PackedBatch], max_batches: int | None = None) -> dict:
        self.backbone.eval()
        ce = torch.zeros((), dtype=torch.float64, device=self.device)
        n = torch.zeros((), dtype=torch.float64, device=self.device)
        for i, batch in enumerate(loader):
            if max_batches is not None and i >= max_batches:
                break
            b = batch.to(self.device)
            _, logs = self.backbone.loss(b.tokens, b.labels, b.seq_info, reduction="sum")
            ce += logs["ce"].double()
            n += logs["n_tokens"].double()
        if self.world > 1:
            t = torch.stack([ce, n])
            dist.all_reduce(t, group=self.group)
            ce, n = t[0], t[1]
        self.backbone.train()
        loss = float(ce / n.clamp(min=1))
        return {"val/loss": loss, "val/ppl": math.exp(min(loss, 20.0)), "val/tokens": int(n)}

    def generate(self, prompt: torch.Tensor, max_new_tokens: int, **sampling) -> torch.Tensor:
        from kohakuwullm_b200.training.loop.sampling import PreviewSampler

        if getattr(self, "_preview_sampler", None) is None:
            self._preview_sampler = PreviewSampler()
        return self._preview_sampler.generate(self.backbone, prompt, max_new_tokens, **sampling)

    # ------------------------------------------------------------------ checkpoints
    def save_checkpoint(self, path: str) -> None:
        if self.device.type == "cuda":
            native.check_status()   # never write a checkpoint of a run whose kernels reported an error
        loader_state = self.loader.state_dict() if hasattr(self.loader, "state_dict") else None
        state = resume.pack_state(self.snapshot(sync=True), self.loss_ema, loader_state, self.global_step)
        extra = {resume.RESUME_KEY: state, "callbacks": self.callbacks.state_dict()}
        self._save(path, extra)

    def _save(self, path: str, extra: dict) -> None:
        # weights are replicated under DDP, so rank 0's copy is the model; what is spread over the ranks is the
        # ZeRO-sharded optimizer state and, under expert parallelism, the experts with their optimizer state
        ep_names = ckpt.expert_sharded_names(self.backbone) if self.world > 1 else set()
        sharded = self.engine.fused_sync or bool(ep_names)
        if sharded:
            opt = ckpt.gather_optimizer_state(self.engine.optimizer, None, self.group, ep_names=ep_names,
                                              module=self.backbone)
        elif self.engine.generic_optimizer:
            # an optimizer that keys its state by position: re-keyed by parameter name (replicas are identical)
            sd = ckpt.named_state_of(self.engine.optimizer, self.backbone)
            opt = {"named_optimizer_state": {k: {kk: (vv.detach().to("cpu", copy=True) if torch.is_tensor(vv) else vv)
                                                 for kk, vv in v.items()} for k, v in sd["named_optimizer_state"].items()},
                   "step": sd["step"]}
        else:
            opt = {"named_optimizer_state": self.engine.optimizer.state_dict()["named_optimizer_state"],
                   "step": self.engine.optimizer.step_count}
        weights = ckpt.local_state_dict(self.backbone)
        if ep_names:
            from kohakuwullm_b200.parallel.ep import gather_expert_state

            weights = {k: v.cpu() for k, v in gather_expert_state(weights, self.backbone, self.group).items()}
        if self.rank == 0:
            payload = {"state_dict": weights, "optimizer_states": [opt],
                       "global_step": self.global_step, "epoch": 0, "pytorch-lightning_version": ckpt.FORMAT_TAG}
            payload.update(extra)
            os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
            torch.save(payload, path + ".tmp")
            os.replace(path + ".tmp", path)
        if self.world > 1:
            dist.barrier(group=self.group)

    def load_checkpoint(self, path: str, loader=None) -> None:
        rest = ckpt.load(path, self.backbone, self.engine.optimizer, group=self.group)
        if self.engine.has_mxfp8:
            self.backbone.refresh_mxfp8()
        state = rest.get(resume.RESUME_KEY)
        if state:
            snap, self.loss_ema, loader_state, self.global_step = resume.unpack_state(state)
            self._offset, self._local = snap, TokenSnapshot()
            self.engine.global_step = self.global_step
            if "rng" in state:
                resume.restore_rng(state["rng"])
            if loader is not None and loader_state is not None and hasattr(loader, "load_state_dict"):
                loader.load_state_dict(loader_state)
        self.callbacks.load_state_dict(rest.get("callbacks", {}))
