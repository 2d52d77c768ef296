"""An ``LMStage`` whose forward + backward of one packed micro-batch replay from CUDA graphs.

Per in-flight slot (see ``pipe/graphed.py``) the stage keeps static layout buffers: ``cu_seqlens`` padded with
empty documents up to ``max_docs`` (they produce no attention tiles, so packs with any number of documents
replay the same graph), position ids, the tokens on the first stage and the labels on the last. The last
stage's graph includes the head and the loss, so what it returns is the micro-batch's summed loss.
Micro-batch ``mb`` uses slot ``mb % slots``; its layout is copied into the slot's buffers right before the
forward replay. Graphs are built at first use of a slot (warm-up runs accumulate into the gradient buffers and
the router statistics, which are saved before and restored after).
"""

from __future__ import annotations

import torch

from kohakuwullm_b200.models.seqinfo import SeqInfo
from kohakuwullm_b200.pipe.graphed import GraphedFn


class GraphedLMStage:
    def __init__(self, module, stage, slots: int, micro_tokens: int, max_docs: int | None = None):
        self.module, self.stage, self.slots, self.T = module, stage, max(int(slots), 1), micro_tokens
        self.max_docs = max_docs or max(8, micro_tokens // 32)
        dev = module.device
        self.device = dev
        self.cu = [torch.full((self.max_docs + 1,), micro_tokens, dtype=torch.int32, device=dev) for _ in range(self.slots)]
        self.pos = [torch.zeros(micro_tokens, dtype=torch.long, device=dev) for _ in range(self.slots)]
        self.tok = [torch.zeros(micro_tokens, dtype=torch.long, device=dev) for _ in range(self.slots)] if stage.is_first else None
        self.lab = [torch.full((micro_tokens,), -100, dtype=torch.long, device=dev) for _ in range(self.slots)] if stage.is_last else None
        self.ce = [torch.zeros((), dtype=torch.float32, device=dev) for _ in range(self.slots)] if stage.is_last else None
        self.graphs: list[GraphedFn | None] = [None] * self.slots
        self.params = [p for p in stage.parameters() if p.requires_grad]

    # ------------------------------------------------------------------ layout of one micro-batch -> slot buffers
    def _load(self, slot: int, mb: int) -> None:
        info = self.module._infos[mb]
        n_docs = info.num_seqs
        if info.total_tokens != self.T or n_docs > self.max_docs:
            raise ValueError(f"micro-batch {mb} ({info.total_tokens} tokens, {n_docs} documents) does not fit the "
                             f"captured stage ({self.T} tokens, {self.max_docs} documents)")
        cu = self.cu[slot]
        cu[: n_docs + 1].copy_(info.cu_seqlens, non_blocking=True)
        if n_docs < self.max_docs:
            cu[n_docs + 1:].fill_(self.T)
        self.pos[slot].copy_(info.position_ids, non_blocking=True)
        if self.tok is not None:
            self.tok[slot].copy_(self.stage._tokens[mb], non_blocking=True)
        if self.lab is not None:
            self.lab[slot].copy_(self.module._labels[mb], non_blocking=True)

    def _fn(self, slot: int):
        stage, module = self.stage, self.module
        info = SeqInfo(self.cu[slot], self.pos[slot], self.T, self.max_docs, None)

        def fn(*inputs):
            saved_infos, saved_tokens = stage._seq_infos, getattr(stage, "_tokens", None)
            stage._seq_infos = [info]
            if self.tok is not None:
                stage._tokens = [self.tok[slot]]
            try:
                out = stage.forward_micro(0, *inputs)
            finally:
                stage._seq_infos = saved_infos
                if saved_tokens is not None:
                    stage._tokens = saved_tokens
            if stage.is_last:
                loss, ce = module.loss_from(out, self.lab[slot])
                self.ce[slot].copy_(ce.detach().reshape(()))
                return (loss,)
            return out

        return fn

    def _sink(self, p, g):
        target = getattr(p, "main_grad", None)
        if target is not None:
            target.add_(g.reshape(target.shape).to(target.dtype))
        elif p.grad is None:
            p.grad = g.detach().clone()
        else:
            p.grad.add_(g)

    def _build(self, slot: int, inputs) -> GraphedFn:
        module = self.module
        flat = getattr(module, "flat", None)
        saved = [b.clone() for b in flat.grad_buffers()] if flat is not None else []
        routers = [b for n, b in self.stage.named_buffers() if n.endswith("load_accum")]
        saved_r = [b.clone() for b in routers]
        g = GraphedFn(self._fn(slot), inputs, self.params, self._sink)
        # warm-up runs must not leak into the step's gradients or the routers' load statistics
        if flat is not None:
            for b, s0 in zip(flat.grad_buffers(), saved):
                b.copy_(s0)
        for b, s0 in zip(routers, saved_r):
            b.copy_(s0)
        return g

    # ------------------------------------------------------------------ the schedule's stage function
    def __call__(self, mb: int, *inputs):
        slot = mb % self.slots
        self._load(slot, mb)
        if self.graphs[slot] is None:
            self.graphs[slot] = self._build(slot, inputs)
        out = self.graphs[slot](*inputs)
        if self.stage.is_last:
            self.module.log("ce_sum", self.ce[slot].clone())
            # the schedule keeps every micro-batch's loss until the end of the step, and the static output is
            # overwritten by the slot's next replay: hand out a copy (still attached to the replay node)
            return out[0].clone()
        return out if len(out) > 1 else out[0]
