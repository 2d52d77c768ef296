"""Pipeline schedules.

Two executors share one interface (``step(first_stage_inputs, n_micro) -> list of losses``):

* ``NativeSchedule`` — GPipe and 1F1B written directly on ``torch.distributed`` point-to-point ops.
  Activations and their gradients cross a stage boundary as fixed-shape tensors (``boundary`` example
  tensors give shape and dtype). Every transfer is its own asynchronous group, issued by both ends of a
  link in the same order; sends are never waited for before the next compute, and receives are posted one
  micro-batch ahead, so on CUDA the transfers run on NCCL's own stream under the compute.
* ``TorchSchedule`` — adapter over ``torch.distributed.pipelining`` for the multi-chunk schedules
  (interleaved 1F1B, looped BFS, interleaved zero-bubble, ZB-V, DualPipe-V), always built with
  ``scale_grads=False`` because the loss is already normalised by the step's token count.

Reference: src/kohakuwupipe/training/trainer.py:37-63,143-160.
"""

from __future__ import annotations

from typing import Callable, Sequence

import torch
import torch.distributed as dist

SCHEDULES = ("gpipe", "1f1b", "interleaved-1f1b", "looped-bfs", "interleaved-zb", "zbv", "dualpipe-v")
MULTI_CHUNK = ("interleaved-1f1b", "looped-bfs", "interleaved-zb", "zbv", "dualpipe-v")
V_STYLE = ("zbv", "dualpipe-v")


def _as_tuple(x):
    return x if isinstance(x, (tuple, list)) else (x,)


class NativeSchedule:
    """GPipe / 1F1B over one stage per rank."""

    def __init__(self, stage_fn: Callable, *, stage_index: int, num_stages: int, n_micro: int,
                 loss_fn: Callable | None, boundary: Sequence[torch.Tensor],
                 out_boundary: Sequence[torch.Tensor] | None = None, kind: str = "1f1b",
                 group=None, prev_rank: int | None = None, next_rank: int | None = None):
        if kind not in ("gpipe", "1f1b"):
            raise ValueError(f"NativeSchedule runs gpipe or 1f1b, not {kind!r}")
        self.stage_fn, self.loss_fn = stage_fn, loss_fn
        self.s, self.S, self.M, self.kind = stage_index, num_stages, n_micro, kind
        self.group = group
        def describe(ts):
            return [(tuple(t.shape), t.dtype, t.device, t.requires_grad or t.is_floating_point()) for t in ts]

        # what arrives from the previous stage / what this stage sends on (gradients come back in that shape)
        self.boundary = describe(boundary)
        self.out_boundary = describe(out_boundary if out_boundary is not None else boundary)
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.prev = prev_rank if prev_rank is not None else rank - 1
        self.next = next_rank if next_rank is not None else rank + 1
        self.first, self.last = stage_index == 0, stage_index == num_stages - 1
        self._pending: list = []
        self.profile = False          # record a CUDA-event pair around every stage forward / backward
        self._spans: list = []
        self._links = self._make_links()

    def _make_links(self) -> dict:
        """One 2-rank group per neighbour link AND direction. NCCL runs the operations of one communicator in
        order on one stream, so on a shared communicator a receive that was posted ahead (and cannot finish
        before the neighbour has computed) holds back every send this rank posts after it, to either
        neighbour; with eight stages that chained the whole pipeline together. Built only when the pipeline
        spans the whole job, because every rank of the job has to take part in creating a group."""
        if not dist.is_initialized() or self.S < 3:
            return {}
        ranks = dist.get_process_group_ranks(self.group) if self.group is not None else None
        world = dist.get_world_size()
        if (ranks is not None and len(ranks) != world) or self.S != world:
            return {}
        if self.prev != dist.get_rank(self.group) - 1 or self.next != dist.get_rank(self.group) + 1:
            return {}     # a custom stage placement: keep the caller's group
        ranks = ranks or list(range(world))
        mine = {}
        for link in range(self.S - 1):
            for direction in ("act", "grad"):
                g = dist.new_group([ranks[link], ranks[link + 1]])
                if self.s in (link, link + 1):
                    mine[(link, direction)] = g
        return mine

    def _link(self, peer_is_next: bool, direction: str):
        link = self.s if peer_is_next else self.s - 1
        return self._links.get((link, direction), self.group)

    # ------------------------------------------------------------------ stage busy time
    def _span(self):
        if not (self.profile and torch.cuda.is_available()):
            return None
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        return ev

    def _close(self, kind: str, start) -> None:
        if start is not None:
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            self._spans.append((kind, start, end))

    def busy_ms(self) -> dict:
        """Device time spent inside stage forwards / backwards since ``profile`` was switched on (or since the
        last call): what is left of the step time is the pipeline bubble plus exposed transfers."""
        torch.cuda.synchronize()
        out = {"forward": 0.0, "backward": 0.0}
        for kind, a, b in self._spans:
            out[kind] += a.elapsed_time(b)
        self._spans.clear()
        return out

    # ------------------------------------------------------------------ communication
    def _empty(self, spec):
        return [torch.empty(shape, dtype=dtype, device=dev) for shape, dtype, dev, _ in spec]

    def _post_send(self, to: int, tensors) -> None:
        """Start sending ``tensors`` to rank ``to`` and return at once. Nothing waits for a send before the
        next compute: the work handles (and the tensors, which must stay alive until the transfer is done)
        are kept until the end of the step."""
        if not tensors:
            return
        bufs = [t.contiguous() for t in tensors]
        to_next = to == self.next
        group = self._link(to_next, "act" if to_next else "grad")
        works = dist.batch_isend_irecv([dist.P2POp(dist.isend, t, to, group) for t in bufs])
        self._pending.append((works, bufs))

    def _post_recv(self, frm: int, activations: bool):
        """Start receiving one boundary (activations from the previous stage, or gradients from the next) and
        return a handle; ``_take`` waits for it. Posting the receive of the NEXT micro-batch before computing
        the current one lets the transfer run under that compute."""
        bufs = self._empty(self.boundary if activations else self.out_boundary)
        group = self._link(not activations, "act" if activations else "grad")
        works = dist.batch_isend_irecv([dist.P2POp(dist.irecv, t, frm, group) for t in bufs])
        return bufs, works, activations

    @staticmethod
    def _take(handle):
        if handle is None:
            return None
        bufs, works, activations = handle
        for w in works:
            w.wait()   # NCCL: the compute stream waits for the transfer; the host does not block
        if activations:
            bufs = [t.requires_grad_() if t.is_floating_point() else t for t in bufs]
        return bufs

    def _drain_sends(self) -> None:
        for works, _bufs in self._pending:
            for w in works:
                w.wait()
        self._pending.clear()

    # ------------------------------------------------------------------ compute
    def _forward(self, mb: int, inputs, stash, losses):
        t0 = self._span()
        out = self.stage_fn(mb, *inputs) if inputs is not None else self.stage_fn(mb)
        outs = _as_tuple(out)
        if self.last:
            loss = self.loss_fn(outs if len(outs) > 1 else outs[0], mb)
            losses.append(loss.detach())
            stash[mb] = (inputs, (loss,))
            self._close("forward", t0)
            return None
        stash[mb] = (inputs, outs)
        self._close("forward", t0)
        return [o.detach() for o in outs]

    def _backward(self, mb: int, grads, stash):
        inputs, outs = stash.pop(mb)
        t0 = self._span()
        if self.last:
            outs[0].backward()
        else:
            pairs = [(o, g) for o, g in zip(outs, grads) if o.requires_grad]
            torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        self._close("backward", t0)
        if self.first or inputs is None:
            return None
        return [i.grad if i.grad is not None else torch.zeros_like(i) for i in inputs]

    # ------------------------------------------------------------------ schedules
    def step(self, n_micro: int | None = None) -> list[torch.Tensor]:
        """One optimizer step's worth of micro-batches.

        Order of the transfers on the link between two neighbouring stages (both sides issue them in this
        order, each as its own asynchronous group, so the two ends always agree and neither can block the
        other): the warm-up activations a_0 .. a_w, then alternately a_{w+1+i}, g_i for every steady
        iteration i, then the remaining gradients. Receives of activations are posted one micro-batch
        ahead (before the compute they overlap), receives of cool-down gradients likewise; the gradient of
        a steady iteration can only be asked for after that iteration's activation went out."""
        M = n_micro or self.M
        stash: dict[int, tuple] = {}
        losses: list[torch.Tensor] = []
        warm = M if self.kind == "gpipe" else min(self.S - self.s - 1, M)
        steady = M - warm
        first, last = self.first, self.last
        f = b = 0
        act = None if first else self._post_recv(self.prev, True)
        try:
            for _ in range(warm):
                inputs = self._take(act)
                act = self._post_recv(self.prev, True) if (not first and f + 1 < M) else None
                out = self._forward(f, inputs, stash, losses)
                f += 1
                if not last:
                    self._post_send(self.next, out)
            for _ in range(steady):
                inputs = self._take(act)
                act = self._post_recv(self.prev, True) if (not first and f + 1 < M) else None
                out = self._forward(f, inputs, stash, losses)
                f += 1
                grads = None
                if not last:
                    self._post_send(self.next, out)
                    grads = self._take(self._post_recv(self.next, False))
                gin = self._backward(b, grads, stash)
                b += 1
                if not first:
                    self._post_send(self.prev, gin)
            grad = self._post_recv(self.next, False) if (not last and b < M) else None
            while b < M:
                grads = self._take(grad)
                grad = self._post_recv(self.next, False) if (not last and b + 1 < M) else None
                gin = self._backward(b, grads, stash)
                b += 1
                if not first:
                    self._post_send(self.prev, gin)
        finally:
            self._drain_sends()
        return losses


class TorchSchedule:
    """``torch.distributed.pipelining`` schedule over one or several local stage modules."""

    def __init__(self, stage_modules: Sequence[torch.nn.Module], stage_indices: Sequence[int], *,
                 num_stages: int, n_micro: int, loss_fn: Callable | None, kind: str, device,
                 input_args: Sequence[tuple], output_args: Sequence | None = None, group=None):
        """``input_args`` / ``output_args``: per local stage, example tensors of what it receives and returns
        (one micro-batch). Both are given so that torch does no shape inference by running the stage: a stage
        whose forward needs per-step state (sequence layouts) cannot be run at construction time."""
        from torch.distributed import pipelining as pp

        classes = {
            "gpipe": pp.ScheduleGPipe, "1f1b": pp.Schedule1F1B,
            "interleaved-1f1b": pp.ScheduleInterleaved1F1B, "looped-bfs": pp.ScheduleLoopedBFS,
            "interleaved-zb": pp.ScheduleInterleavedZeroBubble, "zbv": pp.ScheduleZBVZeroBubble,
            "dualpipe-v": pp.ScheduleDualPipeV,
        }
        if kind not in classes:
            raise ValueError(f"unknown schedule {kind!r}; choose from {sorted(classes)}")
        outs = list(output_args) if output_args is not None else [None] * len(stage_modules)
        stages = []
        for m, i, a, o in zip(stage_modules, stage_indices, input_args, outs):
            if o is not None and isinstance(o, (tuple, list)) and len(o) == 1:
                o = o[0]          # a stage that returns one tensor
            stages.append(pp.PipelineStage(m, i, num_stages, device, input_args=a, output_args=o, group=group))
        cls = classes[kind]
        single = kind in ("gpipe", "1f1b")
        self.has_first = 0 in stage_indices
        self.has_last = (num_stages - 1) in stage_indices
        # the loss is normalised by the step's token count already: no 1/n_micro scaling
        self.schedule = cls(stages[0] if single else stages, n_microbatches=n_micro, loss_fn=loss_fn,
                            scale_grads=False)
        self.n_micro = n_micro

    def step(self, first_input: torch.Tensor | None = None, target: torch.Tensor | None = None):
        losses: list[torch.Tensor] = []
        kwargs = {}
        if self.has_last:
            kwargs = {"target": target, "losses": losses}
        if self.has_first:
            self.schedule.step(first_input, **kwargs)
        else:
            self.schedule.step(**kwargs)
        return losses


def local_stage_indices(rank: int, world: int, chunks: int, style: str = "loop") -> list[int]:
    """Global stage indices held by ``rank`` with ``chunks`` stages per rank: looped (rank, rank+W, ...)
    or folded in a V (rank and 2W-1-rank)."""
    if style == "v":
        if chunks != 2:
            raise ValueError("V-style schedules hold exactly two chunks per rank")
        return [rank, 2 * world - 1 - rank]
    return [rank + c * world for c in range(chunks)]
