"""``PipelineLoop`` and ``PipelineTrainer``: the step loop of the pipeline engine.

Order of one step: zero grads -> install the batch -> run the schedule (forward/backward of every
micro-batch, P2P overlapped with compute) -> [fp16: unscale + overflow vote, the only host read] ->
clip -> optimizer step with ``grad_scale = 1 / step_tokens`` -> ``post_step`` -> scheduler -> counters ->
the last rank's loss is broadcast as a device tensor (read only on logging intervals).
``PipelineTrainer`` owns construction order (module.setup -> stages -> optimizer -> schedule -> loop) and
checkpoints. Reference: src/kohakuwupipe/training/loop.py:20-388, trainer.py:66-274.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Iterable, Sequence

import torch
import torch.distributed as dist

from kohakuwullm_b200.pipe import checkpoint as ckpt
from kohakuwullm_b200.pipe.hooks import CallbackList
from kohakuwullm_b200.pipe.module import PipelineModule
from kohakuwullm_b200.pipe.plan import StagePlan
from kohakuwullm_b200.pipe.scaler import PipelineGradScaler
from kohakuwullm_b200.pipe.schedules import MULTI_CHUNK, SCHEDULES, V_STYLE, NativeSchedule, TorchSchedule


@dataclass
class StepOutput:
    loss: torch.Tensor                       # device tensor, identical on every rank
    step: int
    tokens: int
    skipped: bool = False
    extra: dict[str, torch.Tensor] = field(default_factory=dict)


class PipelineLoop:
    def __init__(self, module: PipelineModule, schedule, optimizer, scheduler=None, *, scaler=None,
                 callbacks: CallbackList | None = None, max_grad_norm: float | None = 1.0,
                 global_clip: bool = True, group=None):
        self.module, self.schedule, self.optimizer, self.scheduler = module, schedule, optimizer, scheduler
        self.scaler = scaler
        self.callbacks = callbacks or CallbackList()
        self.max_grad_norm, self.global_clip, self.group = max_grad_norm, global_clip, group
        self.global_step = 0
        self.tokens_seen = 0
        self.world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0

    # ------------------------------------------------------------------
    def _params(self):
        for stage in self.module.stages:
            yield from (p for p in stage.parameters() if p.requires_grad)

    def _grad_tensors(self):
        flat = getattr(self.optimizer, "flat", None)
        if flat is not None:
            return flat.grad_buffers()
        return [p.grad for p in self._params() if p.grad is not None]

    def _clip_coef(self, inv_tokens: float) -> torch.Tensor:
        """Device scalar ``inv_tokens * min(1, max_norm / norm)``; the norm is global over all stages
        unless ``global_clip`` is off (then it is stage-local, as in the reference)."""
        grads = self._grad_tensors()
        dev = self.module.device
        sq = self._sumsq(grads, dev)
        if self.global_clip and self.world > 1:
            dist.all_reduce(sq, group=self.group)
        norm = sq.sqrt() * inv_tokens
        coef = torch.full((1,), inv_tokens, dtype=torch.float32, device=dev)
        if self.max_grad_norm:
            coef = coef * torch.clamp(self.max_grad_norm / (norm + 1e-6), max=1.0)
        self.last_grad_norm = norm
        return coef

    def _sumsq(self, grads, dev) -> torch.Tensor:
        """Sum of squares of all gradient tensors as a (1,) fp32 device tensor. Flat fp32 gradient buffers on a
        GPU go through the deterministic two-level reduction kernel (one launch per buffer); anything else is
        summed tensor by tensor."""
        sq = torch.zeros(1, dtype=torch.float32, device=dev)
        from kohakuwullm_b200.ops import native

        fast = (torch.device(dev).type == "cuda" and native.available()
                and all(g.dtype == torch.float32 and g.is_contiguous() for g in grads))
        if fast and grads:
            import ctypes

            L = native.require()
            if getattr(self, "_sq_partial", None) is None:
                self._sq_partial = torch.empty(L.kwu_sumsq_blocks(), dtype=torch.float32, device=dev)
            for i, g in enumerate(grads):
                rc = L.kwu_sumsq_flat(native.ptr(g), ctypes.c_longlong(g.numel()), native.ptr(self._sq_partial),
                                      native.ptr(sq), ctypes.c_int(int(i > 0)), native.stream_ptr())
                native.check(rc, "sumsq_flat")
            return sq
        for g in grads:
            sq += g.float().pow(2).sum()
        return sq

    def broadcast_loss(self, loss: torch.Tensor | None) -> torch.Tensor:
        dev = self.module.device
        t = loss.detach().float().reshape(1) if loss is not None else torch.zeros(1, device=dev)
        if self.world > 1:
            dist.broadcast(t, src=dist.get_global_rank(self.group, self.world - 1) if self.group else self.world - 1,
                           group=self.group)
        return t.reshape(())

    def step(self, batch: Any) -> StepOutput:
        module, cb = self.module, self.callbacks
        if torch.device(module.device).type == "cuda":
            from kohakuwullm_b200.ops import native

            native.poll_status()   # an error a kernel of an earlier step reported (no host synchronisation)
        cb.on_train_batch_start(self, batch, self.global_step)
        self.optimizer.zero_grad(set_to_none=True)
        module.set_batch(batch)
        tokens = module.step_tokens(batch)
        n_micro = module.num_microbatches(batch)
        losses = module.forward_backward(self.schedule, batch, n_micro)
        overflow = False
        if self.scaler is not None and self.scaler.enabled:
            self.scaler.unscale_(self._grad_tensors())
            overflow = self.scaler.agree(self.group)
            self.scaler.update(overflow)
        skipped = overflow or tokens == 0
        if not skipped:
            coef = self._clip_coef(1.0 / tokens)
            cb.on_before_optimizer_step(self, self.optimizer)
            try:
                self.optimizer.step(grad_scale=coef)
            except TypeError:
                for g in self._grad_tensors():
                    g.mul_(coef.to(g.dtype))
                self.optimizer.step()
            module.post_step()
        if self.scheduler is not None:
            self.scheduler.step()
        self.global_step += 1
        self.tokens_seen += tokens
        local = None
        if losses:
            local = torch.stack([l.float().reshape(()) for l in losses]).sum() / max(tokens, 1)
        out = StepOutput(self.broadcast_loss(local), self.global_step, tokens, skipped, module.pop_metrics())
        cb.on_train_batch_end(self, out, batch, self.global_step)
        return out

    def fit(self, batches: Iterable, max_steps: int) -> list[StepOutput]:
        outs = []
        self.callbacks.on_fit_start(self)
        self.callbacks.on_train_start(self)
        try:
            it = iter(batches)
            while self.global_step < max_steps:  # test before pulling, so no fetched batch goes untrained
                try:
                    batch = next(it)
                except StopIteration:
                    break
                outs.append(self.step(batch))
        except BaseException as exc:  # noqa: BLE001  every rank's callbacks hear about it, then it propagates
            self.callbacks.on_exception(self, exc)
            raise
        self.callbacks.on_train_end(self)
        self.callbacks.on_fit_end(self)
        return outs

    def progress_state(self) -> dict:
        return {"global_step": self.global_step, "tokens_seen": self.tokens_seen}

    def load_progress_state(self, state: dict) -> None:
        self.global_step = int(state.get("global_step", 0))
        self.tokens_seen = int(state.get("tokens_seen", 0))


class PipelineTrainer:
    """Builds stages, optimizer, schedule and loop in the one order that works, and checkpoints them."""

    def __init__(self, module: PipelineModule, plans: Sequence[StagePlan], *, rank: int = 0, world: int = 1,
                 device="cpu", n_micro: int = 1, schedule: str = "1f1b", engine: str | None = None,
                 scaler: PipelineGradScaler | None = None, callbacks=(), max_grad_norm: float | None = 1.0,
                 global_clip: bool = True, group=None):
        if schedule not in SCHEDULES:
            raise ValueError(f"unknown schedule {schedule!r}; choose from {SCHEDULES}")
        self.module, self.plans_all = module, list(plans)
        self.rank, self.world, self.device, self.group = rank, world, torch.device(device), group
        self.schedule_name = schedule
        n_stages = len(self.plans_all)
        chunks = n_stages // world
        if n_stages % world:
            raise ValueError(f"{n_stages} stages do not divide over {world} ranks")
        if chunks > 1 and schedule not in MULTI_CHUNK:
            raise ValueError(f"schedule {schedule!r} runs one stage per rank, got {chunks}")
        if schedule in V_STYLE:
            local = [rank, 2 * world - 1 - rank]
        else:
            local = [rank + c * world for c in range(chunks)]
        self.local_indices = local
        module.setup([self.plans_all[i] for i in local], rank, world, self.device)
        opt = module.configure_optimizers()
        self.optimizer, self.scheduler = opt if isinstance(opt, tuple) else (opt, None)
        engine = engine or ("native" if schedule in ("gpipe", "1f1b") else "torch")
        if engine == "native":
            stage = module.stages[0]
            stage_fn = stage.forward_micro if hasattr(stage, "forward_micro") else (lambda mb, *a: stage(*a))
            loss_fn = module.loss if local[0] == n_stages - 1 else None
            # a module may hand over a replacement that replays the stage from CUDA graphs
            fns = module.native_stage_fns(stage, self.plans_all[local[0]], n_stages, n_micro, schedule) \
                if hasattr(module, "native_stage_fns") else None
            if fns is not None:
                stage_fn, loss_fn = fns
            self.schedule = NativeSchedule(
                stage_fn,
                stage_index=local[0], num_stages=n_stages, n_micro=n_micro,
                loss_fn=loss_fn,
                boundary=() if local[0] == 0 else module.boundary_example(self.plans_all[local[0]]),
                out_boundary=() if local[0] == n_stages - 1 else module.boundary_example(self.plans_all[local[0] + 1]),
                kind=schedule, group=group)
        else:
            # torch decides "this schedule trains" from the presence of a loss function, on EVERY rank: a rank
            # without one runs forward only and returns while its neighbours wait for its gradients
            loss_fn = lambda out, target: module.loss(out, int(target.reshape(-1)[0]))  # noqa: E731
            self.schedule = TorchSchedule(
                module.stages, local, num_stages=n_stages, n_micro=n_micro, loss_fn=loss_fn, kind=schedule,
                device=self.device, group=group,
                input_args=[module.first_input_example() if i == 0 else module.boundary_example(self.plans_all[i])
                            for i in local],
                # what a stage hands on has the shape of what the next one receives; the last stage returns
                # the same boundary (hidden states [+ the router-loss accumulator]) to the loss function
                output_args=[module.boundary_example(self.plans_all[min(i + 1, n_stages - 1)]) for i in local])
        self.loop = PipelineLoop(module, self.schedule, self.optimizer, self.scheduler, scaler=scaler,
                                 callbacks=CallbackList(callbacks), max_grad_norm=max_grad_norm,
                                 global_clip=global_clip, group=group)

    def fit(self, batches: Iterable, max_steps: int):
        return self.loop.fit(batches, max_steps)

    # ------------------------------------------------------------------ checkpoints
    def _stage_module(self):
        """What a checkpoint of this rank covers: the stage, or with several stages per rank a list of them whose
        parameter names (``"<local index>.<name>"``) are the keys ``module.global_names()`` maps to whole-model names."""
        if len(self.module.stages) == 1:
            return self.module.stages[0]
        if getattr(self, "_stage_list", None) is None:
            self._stage_list = torch.nn.ModuleList(self.module.stages)
        return self._stage_list

    def save_checkpoint(self, path: str) -> None:
        stage = self._stage_module()
        extra = {"progress": self.loop.progress_state(), "callbacks": self.loop.callbacks.state_dict()}
        if self.scheduler is not None and hasattr(self.scheduler, "state_dict"):
            extra["lr_schedulers"] = [self.scheduler.state_dict()]
        if self.loop.scaler is not None:
            extra["grad_scaler"] = self.loop.scaler.state_dict()
        self.loop.callbacks.on_save_checkpoint(self, extra)
        self.module.on_save_checkpoint(extra)
        ckpt.save(path, stage, self.optimizer, names=self.module.global_names(),
                  global_step=self.loop.global_step, extra=extra, group=self.group)

    def load_checkpoint(self, path: str) -> dict:
        stage = self._stage_module()
        rest = ckpt.load(path, stage, self.optimizer, names=self.module.global_names(), group=self.group)
        self.loop.load_progress_state(rest.get("progress", {"global_step": rest.get("global_step", 0)}))
        if self.scheduler is not None and rest.get("lr_schedulers"):
            self.scheduler.load_state_dict(rest["lr_schedulers"][0])
        if self.loop.scaler is not None and "grad_scaler" in rest:
            self.loop.scaler.load_state_dict(rest["grad_scaler"])
        self.loop.callbacks.load_state_dict(rest.get("callbacks", {}))
        self.loop.callbacks.on_load_checkpoint(self, rest)
        self.module.on_load_checkpoint(rest)
        return rest
