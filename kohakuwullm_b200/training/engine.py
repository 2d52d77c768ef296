"""``TrainEngine``: one optimizer step over packed micro-batches with token-exact accumulation.

The step is free of host synchronisation:

1. the trained-token count of the step is taken from the HOST copy of the labels, summed over the
   data-parallel group on the device, and kept as a device scalar ``inv_tokens``;
2. every micro-batch is copied host->device (pinned, non-blocking), run forward with
   ``reduction="sum"`` and backward with unit scale, so ``main_grad`` accumulates plain sums;
3. gradient buffers are summed across ranks, the global norm is taken on the device, and the clipping
   coefficient times ``inv_tokens`` enters the fused AdamW kernel as its ``grad_scale``;
4. MXFP8 weight copies are re-quantised and router biases updated.

Loss and gradients are therefore identical (up to summation order) for any split of the same tokens
into micro-batches and ranks. Reference semantics: src/kohakuwullm/training/loop/trainer.py:172-240.
"""

from __future__ import annotations

import ctypes
import os
from typing import Sequence

import torch
import torch.distributed as dist
from torch import nn

from kohakuwullm_b200.data.packing import PackedBatch
from kohakuwullm_b200.ops import gemm as gemm_ops
from kohakuwullm_b200.ops import native
from kohakuwullm_b200.parallel.ddp import GradSync
from kohakuwullm_b200.parallel.flat import FlatParameters
from kohakuwullm_b200.training.optim.fused_adamw import FlatAdamW
from kohakuwullm_b200.training.optim.lowbit import cast_parameters_
from kohakuwullm_b200.utils import nvtx


class GraphedMicroStep:
    """Forward + backward of one packed micro-batch captured in a CUDA graph.

    A 546M-parameter step is several thousand small launches per micro-batch; replaying them from a
    graph removes the host from the critical path. Shapes are fixed by ``(tokens, max_docs)``:
    ``cu_seqlens`` is padded with zero-length documents up to ``max_docs`` (they produce no attention
    tiles), so packs with any number of documents replay the same graph. A micro-batch with FEWER tokens
    than the graph holds is completed by one fully masked filler document (label -100 everywhere, its
    own positions), the same padding ``collate_packed(pad_to_multiple=...)`` produces, so that
    document-aligned splits of varying size share a few graphs instead of capturing one each. Inputs are
    copied straight from (pinned) host memory into the graph's static buffers.
    """

    def __init__(self, engine: "TrainEngine", tokens: int, max_docs: int):
        dev = engine.device
        self.engine, self.tokens, self.max_docs = engine, tokens, max_docs
        self.tok = torch.zeros(tokens, dtype=torch.long, device=dev)
        self.lab = torch.full((tokens,), -100, dtype=torch.long, device=dev)
        self.pos = torch.zeros(tokens, dtype=torch.long, device=dev)
        self._arange = torch.arange(tokens, dtype=torch.long, device=dev)
        self.cu = torch.full((max_docs + 1,), tokens, dtype=torch.int32, device=dev)
        self.cu[0] = 0
        self.ce = torch.zeros((), dtype=torch.float32, device=dev)
        self.total = torch.zeros((), dtype=torch.float32, device=dev)
        self.extra: dict[str, torch.Tensor] = {}
        self.graph: torch.cuda.CUDAGraph | None = None

    def _info(self):
        from kohakuwullm_b200.models.seqinfo import SeqInfo

        return SeqInfo(self.cu, self.pos, self.tokens, self.max_docs, None)

    def load(self, mb: PackedBatch) -> None:
        n_docs = mb.seq_info.num_seqs
        T = mb.num_tokens
        pad = self.tokens - T
        if pad < 0 or n_docs + (1 if pad else 0) > self.max_docs:
            raise ValueError("micro-batch does not fit this graph")
        self.tok[:T].copy_(mb.tokens, non_blocking=True)
        self.lab[:T].copy_(mb.labels, non_blocking=True)
        self.pos[:T].copy_(mb.seq_info.position_ids, non_blocking=True)
        self.cu[: n_docs + 1].copy_(mb.seq_info.cu_seqlens, non_blocking=True)
        if n_docs < self.max_docs:
            # the filler document [T, tokens) followed by empty documents
            self.cu[n_docs + 1:].fill_(self.tokens)
        if pad:
            self.lab[T:].fill_(-100)
            self.pos[T:].copy_(self._arange[:pad])

    def _run(self) -> None:
        eng = self.engine
        loss, logs = eng.model.loss(self.tok, self.lab, self._info(), reduction="sum",
                                    router_scale=eng._router_scale)
        eng._backward(loss)
        self.ce.copy_(logs["ce"])
        self.total.copy_(loss.detach())
        for k in ("z_loss", "router_loss"):
            if k in logs:
                if k not in self.extra:
                    self.extra[k] = torch.zeros((), dtype=torch.float32, device=eng.device)
                self.extra[k].copy_(logs[k])

    def capture(self, warmup: int = 2) -> None:
        eng = self.engine
        side = torch.cuda.Stream(device=eng.device)
        side.wait_stream(torch.cuda.current_stream())
        saved = [b.clone() for b in eng.flat.grad_buffers()]
        with torch.cuda.stream(side):
            for _ in range(warmup):
                self._run()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        lib = native.lib()
        before = lib.kwu_launch_count()
        with torch.cuda.graph(self.graph):
            self._run()
        self.native_launches = int(lib.kwu_launch_count() - before)  # kernels of this library per replay
        # warm-up and capture runs must not leak into the real gradients / router statistics
        for b, s0 in zip(eng.flat.grad_buffers(), saved):
            b.copy_(s0)

    def replay(self) -> None:
        self.graph.replay()
        self.engine.replayed_native_launches += self.native_launches


class TrainEngine:
    def __init__(self, model: nn.Module, *, lr: float = 3e-4, betas=(0.9, 0.95), eps: float = 1e-8,
                 weight_decay: float = 0.1, max_grad_norm: float = 1.0,
                 param_dtype: torch.dtype | None = None, group=None, grad_sync: str = "nccl",
                 device: torch.device | str | None = None, lr_schedule=None,
                 cuda_graphs: bool | None = None, graph_max_docs: int | None = None,
                 graph_token_bucket: int = 512, graph_cache_size: int = 8,
                 expert_parallel: bool | str = False, ep_capacity_factor: float = 2.0,
                 ep_on_overflow: str = "raise", optimizer: str = "fused_adamw", optimizer_kwargs: dict | None = None,
                 grad_compress: str | None = None):
        """``grad_compress``: ``"bf16"`` / ``"fp16"`` sends the NCCL gradient buckets in that dtype (ignored by the
        fused peer-memory step, which reduces fp32).
        ``expert_parallel``: split every MoE layer's experts over the ranks of ``group`` (tokens travel
        to the owning rank over peer memory); all other parameters stay data-parallel replicas.
        ``"reference"`` keeps the sharding but moves tokens with plain collectives (test oracle).
        ``graph_token_bucket``: captured micro-step graphs hold a multiple of this many tokens; a micro-batch
        is padded up to the next multiple with a masked filler document. ``graph_cache_size``: at most this
        many graphs are kept (least recently used goes first); each pins one forward + backward pool.
        ``optimizer``: ``"fused_adamw"`` is the flat one-launch AdamW (the only one the fused gradient step can
        carry); any other registered name (``muon``, ``adamw16``, ``stochastic_adamw``, ``adamw8bit``, ``adamw``,
        ...) is built by ``build_optimizer`` with the same grouping rules and stepped from the reduced, clipped
        gradients (NCCL gradient sync)."""
        self.model = model
        if device is not None:
            model.to(device)
        self.device = next(model.parameters()).device
        if param_dtype is not None and param_dtype != torch.float32:
            cast_parameters_(model, param_dtype)
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.generic_optimizer = optimizer != "fused_adamw"
        self.fused_sync = (grad_sync == "fused" and self.world > 1 and self.device.type == "cuda"
                           and not self.generic_optimizer)
        self.ep = None
        self.ep_sharded = bool(expert_parallel) and self.world > 1
        if expert_parallel and self.world > 1:
            from kohakuwullm_b200.parallel.ep import ExpertParallel, shard_experts

            if self.device.type == "cuda" and native.available() and expert_parallel != "reference":
                self.ep = ExpertParallel(group, capacity_factor=ep_capacity_factor, on_overflow=ep_on_overflow)
            shard_experts(model, self.ep, group if group is not None else dist.group.WORLD)
        if self.fused_sync:
            from kohakuwullm_b200.parallel.fused_ddp import FusedGradSync
            from kohakuwullm_b200.parallel.symm import SymmetricPool

            pool = SymmetricPool(group)
            self.flat = FlatParameters(model, allocator=pool.empty)
            self.sync = FusedGradSync(self.flat, pool, group)
            shard = (self.rank, self.world)
        else:
            self.flat = FlatParameters(model)
            self.sync = GradSync(self.flat, group, compress=grad_compress)
            shard = None
        if self.generic_optimizer:
            from kohakuwullm_b200.training.optim.build import build_optimizer

            kw = dict(optimizer_kwargs or {})
            if optimizer not in ("sgd", "muon"):
                kw.setdefault("eps", eps)
            self.optimizer = build_optimizer(model, optimizer, lr=lr, weight_decay=weight_decay, betas=betas, **kw)
            for g in self.optimizer.param_groups:
                g.setdefault("initial_lr", g["lr"])
            self._base_lr = lr
        else:
            self.optimizer = FlatAdamW(self.flat, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, shard=shard)
        self.max_grad_norm = max_grad_norm
        self.lr_schedule = lr_schedule
        self.global_step = 0
        dev = self.device
        self._sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        self._coef = torch.ones(1, dtype=torch.float32, device=dev)
        self._norm = torch.zeros(1, dtype=torch.float32, device=dev)
        self._partial = None
        self.has_mxfp8 = hasattr(model, "refresh_mxfp8") and getattr(getattr(model, "config", None), "mxfp8", False)
        self.has_router = hasattr(model, "update_router_bias")
        self.last_router_stats: dict = {}
        self.cuda_graphs = (self.device.type == "cuda" and native.available()) if cuda_graphs is None else cuda_graphs
        self.graph_max_docs = graph_max_docs
        self.graph_token_bucket = max(int(graph_token_bucket), 1)
        self.graph_cache_size = max(int(graph_cache_size), 1)
        self._graphs: dict[tuple[int, int], GraphedMicroStep] = {}   # insertion order = recency (LRU first)
        self.replayed_native_launches = 0
        # weight gradients on a side stream: measured neutral on the dense step (every kernel of the chain
        # already fills the GPU), so off unless asked for
        self.wgrad_overlap = os.environ.get("KWU_WGRAD_OVERLAP", "0") == "1"
        self._router_scale = torch.ones(1, dtype=torch.float32, device=dev)

    def _graph_for(self, mb: PackedBatch) -> GraphedMicroStep | None:
        """Graph matching this micro-batch's token count (captured on first use), or None."""
        if not self.cuda_graphs or not getattr(mb.seq_info, "packed", True):
            return None        # padded (rows, S) batches run eagerly
        b = self.graph_token_bucket
        T = (mb.num_tokens + b - 1) // b * b
        max_docs = self.graph_max_docs or max(8, T // 32)
        if mb.seq_info.num_seqs + (1 if T != mb.num_tokens else 0) > max_docs:
            return None
        key = (T, max_docs)
        g = self._graphs.pop(key, None)
        if g is None:
            while len(self._graphs) >= self.graph_cache_size:
                old = self._graphs.pop(next(iter(self._graphs)))
                old.graph = None   # releases the graph and its private memory pool
            g = GraphedMicroStep(self, T, max_docs)
            g.load(mb)
            router_state = self._snapshot_router()
            g.capture()
            self._restore_router(router_state)
        self._graphs[key] = g      # most recently used last
        return g

    def _same_micro_batch_count(self, micro_batches: Sequence[PackedBatch]) -> list[PackedBatch]:
        """Under expert parallelism every MoE layer of every micro-batch is a collective exchange, so all ranks
        have to run the same number of micro-batches. A document-aligned split can give one rank fewer pieces than
        another (few long documents); the ranks agree on the largest count and the others append fully masked
        filler micro-batches (no loss, no gradient, but they take part in the exchanges)."""
        from kohakuwullm_b200.models.seqinfo import SeqInfo

        n = torch.tensor([len(micro_batches)], dtype=torch.int32, device=self.device)
        dist.all_reduce(n, op=dist.ReduceOp.MAX, group=self.group)
        missing = int(n) - len(micro_batches)
        out = list(micro_batches)
        for _ in range(missing):
            out.append(PackedBatch(torch.zeros(16, dtype=torch.long), torch.full((16,), -100, dtype=torch.long),
                                   SeqInfo.from_lengths([16]), 0))
        return out

    @torch.no_grad()
    def _generic_step(self) -> None:
        """Step an optimizer that reads ``p.grad``: the flat fp32 gradient buffers are scaled in place by the
        token-count / clipping coefficient, handed over as ``.grad`` (in the parameter's dtype for 16-bit
        parameters), and cleared afterwards."""
        for buf in self.flat.grad_buffers():
            buf.mul_(self._coef)
        params = [p for p in self.model.parameters() if p.requires_grad and hasattr(p, "main_grad")]
        for p in params:
            g = p.main_grad
            p.grad = g if g.dtype == p.dtype else g.to(p.dtype)
        self.optimizer.step()
        for p in params:
            p.grad = None
        self.flat.zero_grad()

    def _backward(self, loss: torch.Tensor) -> None:
        """Backward of one micro-batch with the weight-gradient products on a side stream (they only have to be
        done before the optimizer reads ``main_grad``, so they run in the shadow of the activation-gradient
        chain); the side stream is joined before this returns."""
        overlap = self.wgrad_overlap and self.device.type == "cuda"
        gemm_ops.set_wgrad_overlap(overlap)
        try:
            loss.backward()
        finally:
            gemm_ops.set_wgrad_overlap(False)
            gemm_ops.join_wgrad()

    def native_launch_total(self) -> int:
        """Kernels of the native library launched so far: direct launches plus graph replays."""
        return int(native.lib().kwu_launch_count()) + self.replayed_native_launches

    def _snapshot_router(self):
        return [b.clone() for n, b in self.model.named_buffers() if n.endswith("load_accum")]

    def _restore_router(self, saved):
        bufs = [b for n, b in self.model.named_buffers() if n.endswith("load_accum")]
        for b, s0 in zip(bufs, saved):
            b.copy_(s0)

    # ------------------------------------------------------------------
    def _grad_norm_and_coef(self, inv_tokens: torch.Tensor) -> None:
        """Global gradient norm and the optimizer's gradient scale, on the device. Replicated buffers hold
        the same reduced sums on every rank; expert-parallel buffers differ per rank, so their squared
        norms are summed over the group first."""
        local = [self.flat.groups[k].main_grad for k in self.flat.local_keys()]
        shared = [self.flat.groups[k].main_grad for k in self.flat.replicated_keys()]
        if self.device.type == "cuda" and native.available():
            L = native.require()
            if self._partial is None:
                self._partial = torch.empty(L.kwu_sumsq_blocks(), dtype=torch.float32, device=self.device)

            def add(bufs, first):
                for i, b in enumerate(bufs):
                    rc = L.kwu_sumsq_flat(native.ptr(b), ctypes.c_longlong(b.numel()), native.ptr(self._partial),
                                          native.ptr(self._sumsq), ctypes.c_int(int(not (first and i == 0))),
                                          native.stream_ptr())
                    native.check(rc, "sumsq_flat")

            if local:
                add(local, True)
                if self.world > 1:
                    dist.all_reduce(self._sumsq, group=self.group)
            add(shared, not local)
            rc = L.kwu_clip_coef(native.ptr(self._sumsq), native.ptr(inv_tokens),
                                 ctypes.c_float(self.max_grad_norm or 0.0), native.ptr(self._coef),
                                 native.ptr(self._norm), native.stream_ptr())
            native.check(rc, "clip_coef")
        else:
            sq = sum((b.double() ** 2).sum() for b in shared) if shared else torch.zeros((), dtype=torch.float64)
            if local:
                sq_local = sum((b.double() ** 2).sum() for b in local)
                if self.world > 1:
                    dist.all_reduce(sq_local, group=self.group)
                sq = sq + sq_local
            sq = sq.float()
            norm = sq.sqrt() * inv_tokens
            self._norm.copy_(norm.reshape(1))
            coef = inv_tokens.clone().reshape(1)
            if self.max_grad_norm:
                coef = coef * torch.clamp(self.max_grad_norm / (norm + 1e-6), max=1.0)
            self._coef.copy_(coef.reshape(1))

    def step(self, micro_batches: Sequence[PackedBatch]) -> dict[str, torch.Tensor]:
        model = self.model
        model.train()
        dev = self.device
        if dev.type == "cuda":
            # a kernel of an earlier step whose bounded wait ran out (a peer that never arrived, an expert
            # buffer that overflowed) surfaces here as an exception, without a host synchronisation
            native.poll_status()
        if self.ep_sharded:
            micro_batches = self._same_micro_batch_count(micro_batches)
        local_tokens = sum(mb.trained_tokens() for mb in micro_batches)
        tok = torch.tensor([float(local_tokens)], dtype=torch.float32).to(dev, non_blocking=True)
        self.sync.all_reduce_scalar(tok)
        inv_tokens = 1.0 / tok.clamp(min=1.0)
        # router auxiliary terms are per-micro-batch means: weight them like one rank's share of tokens
        self._router_scale.copy_(tok / (self.world * max(len(micro_batches), 1)))
        ce_total = torch.zeros((), dtype=torch.float32, device=dev)
        loss_total = torch.zeros((), dtype=torch.float32, device=dev)
        extra: dict[str, torch.Tensor] = {}
        for i, mb in enumerate(micro_batches):
            graph = self._graph_for(mb)
            if graph is not None:
                with nvtx.range(f"micro_step_{i}/graph"):
                    graph.load(mb)
                    graph.replay()
                ce_total = ce_total + graph.ce
                loss_total = loss_total + graph.total
                for k, v in graph.extra.items():
                    extra[k] = extra.get(k, 0) + v
                continue
            with nvtx.range(f"micro_step_{i}/eager"):
                mb = mb.to(dev, non_blocking=True)
                loss, logs = model.loss(mb.tokens, mb.labels, mb.seq_info, reduction="sum",
                                        router_scale=self._router_scale)
                self._backward(loss)
            ce_total = ce_total + logs["ce"]
            loss_total = loss_total + loss.detach().float()
            for k in ("z_loss", "router_loss"):
                if k in logs:
                    extra[k] = extra.get(k, 0) + logs[k]
        if self.lr_schedule is not None:
            now = self.lr_schedule(self.global_step)
            if self.generic_optimizer:      # every group keeps its ratio to the base rate (Muon, embedding, muP groups)
                for g in self.optimizer.param_groups:
                    g["lr"] = g["initial_lr"] * (now / self._base_lr)
            else:
                self.optimizer.param_groups[0]["lr"] = now
        if self.fused_sync:
            # one fused pass: reduce-scatter + scaling + clipping + sharded AdamW + all-gather
            with nvtx.range("grad_sync+optimizer/fused"):
                self.sync.step(self.optimizer, inv_tokens.reshape(1), self.max_grad_norm)
            self._norm = self.sync.norm
            if self.has_mxfp8:
                with nvtx.range("mxfp8_refresh"):
                    model.refresh_mxfp8()
        elif local_tokens > 0 or self.world > 1:
            with nvtx.range("grad_sync"):
                self.sync.reduce()
            with nvtx.range("clip+optimizer"):
                self._grad_norm_and_coef(inv_tokens)
                if self.generic_optimizer:
                    self._generic_step()
                else:
                    self.optimizer.step(grad_scale=self._coef, zero_grad=True)
            if self.has_mxfp8:
                with nvtx.range("mxfp8_refresh"):
                    model.refresh_mxfp8()
        else:
            self.flat.zero_grad()  # an all-masked step updates nothing
        if self.has_router:
            self.last_router_stats = model.update_router_bias()
        self.global_step += 1
        sums = torch.stack([loss_total.reshape(()), ce_total.reshape(())])
        if self.world > 1:
            sums = self.sync.all_reduce_scalar(sums.clone())
        # "loss" is the optimised objective (cross-entropy + z-loss + router terms) per trained token
        out = {"loss": (sums[0] * inv_tokens).reshape(()), "ce": (sums[1] * inv_tokens).reshape(()),
               "grad_norm": self._norm.reshape(()).clone(), "tokens": tok.reshape(())}
        for k, v in extra.items():
            out[k] = v * inv_tokens.reshape(())
        if self.ep is not None:
            # pairs this rank's tokens lost to a full receive buffer during the step (0 in a healthy run)
            out["ep_dropped_pairs"] = self.ep.dropped_pairs(reset=True)
        return out
