"""Expert parallelism: the experts of every MoE layer are split over the ranks of one NVSwitch domain,
tokens travel to the expert's owner and back through peer-mapped memory (``csrc/moe_ep.cu``).

``ExpertParallel`` owns the symmetric workspace shared by all layers (count table, flags, one receive
buffer and one output buffer of ``cap`` rows) and the device-resident epoch counters. One layer's
forward is::

    plan = ep.plan(idx, counts)                       # counts exchange + offsets, all on the device
    rows = ep.dispatch(x, plan)                       # peer stores -> barrier -> private expert-sorted rows
    ...grouped GEMM / SwiGLU / grouped GEMM on the LOCAL experts (ops.moe._GroupedLinear)...
    y    = ep.combine(y_rows, weight, plan, T)        # output buffer -> barrier -> peer-load gather-sum

and backward runs the mirror image (gate-scaled output gradients are pushed to the owners, input
gradients are pulled back). Nothing synchronises with the host, every wait in the kernels is bounded, and
the same launch sequence replays from a CUDA graph.

``cap`` is ``capacity_factor x T x k`` rows (rounded up, plus padding): with perfectly balanced routing
a rank receives ``T x k`` rows. If a step routes more rows than that to one rank the kernels drop the
excess pairs, set the overflow code in the status word, and the next status check raises.

``shard_experts`` converts a model built with full expert tensors into its expert-parallel form (local
slices, flagged ``ep_local`` so that the data-parallel gradient reduction skips them);
``gather_expert_state`` undoes it for checkpoints. CPU / single-rank fallback: ``reference_ep_forward``
(all-gather based, differentiable) is what the gloo tests compare against.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch
import torch.distributed as dist
from torch import nn

from kohakuwullm_b200.ops import native

c_int, c_ll = ctypes.c_int, ctypes.c_longlong
FLAG_COUNTS, FLAG_ARRIVED, FLAG_OUTPUT = 0, 1, 2


@dataclass
class EPPlan:
    offsets: torch.Tensor     # (El+1,) int32 padded offsets of the local experts
    totals: torch.Tensor      # (El,) int32 real rows per local expert
    tiles: torch.Tensor       # (max_tiles, 4) int32
    send_base: torch.Tensor   # (E,) int32
    cursors: torch.Tensor     # (E,) int32
    pos_of: torch.Tensor      # (T*k,) int32 row of every pair inside the owner's buffers, -1 = dropped
    idx: torch.Tensor         # (T*k,) int32 expert of every pair
    max_rows: int             # == cap
    top_k: int
    num_experts: int          # LOCAL expert count: what the grouped GEMMs iterate over
    row_ptrs: torch.Tensor | None = None   # (cap,) int64 scatter map of the received rows (filled by dispatch)


class ExpertParallel:
    def __init__(self, group=None, capacity_factor: float = 2.0, wait_limit_cycles: int = 0,
                 scatter_epilogue: bool | None = None, on_overflow: str = "raise"):
        """``on_overflow``: what a receive buffer that is too small does. ``"raise"``: the overflow code goes
        into the status word and the next status check ends the run. ``"count"``: the excess (token, expert)
        pairs are dropped (they contribute zero, like a capacity-limited router) and the run goes on. Either
        way every rank counts the pairs it could not place; ``dropped_pairs()`` reads the count.

        ``scatter_epilogue``: let the expert GEMM epilogues store result rows straight into the source ranks'
        per-pair buffers (no return kernel) instead of the default pull path (owner writes a peer-visible
        buffer, sources gather with coalesced peer loads). Measured on 2 B200s, MoE 991M with skewed routers:
        pull 263.0k tokens/s, scatter 231.4k: the epilogue's 64-byte row segments use the link worse than the
        pull kernel's 512-byte row reads, so pull is the default; ``KWU_EP_SCATTER=1`` switches."""
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if self.world > 8:
            raise ValueError("expert parallelism over peer memory supports up to 8 ranks (one NVSwitch domain)")
        if on_overflow not in ("raise", "count"):
            raise ValueError(f"on_overflow must be 'raise' or 'count', not {on_overflow!r}")
        self.on_overflow = on_overflow
        self.capacity_factor = capacity_factor
        self.limit = wait_limit_cycles
        if scatter_epilogue is None:
            import os

            scatter_epilogue = os.environ.get("KWU_EP_SCATTER", "0") not in ("", "0")
        self.scatter_epilogue = bool(scatter_epilogue)
        self._ws = None
        self._shape = None

    # ------------------------------------------------------------------ workspace
    def _workspace(self, n_pairs: int, D: int, E: int, device):
        L = native.require()
        El = E // self.world
        cap = int(self.capacity_factor * n_pairs) + El * 127
        cap = -(-cap // 128) * 128
        if self._ws is not None:
            have_cap, have_D, have_E = self._shape
            if (D, E) != (have_D, have_E) or cap > have_cap or n_pairs > self._ws["n_pairs"]:
                raise ValueError(f"expert-parallel workspace was sized for {self._shape}, got {(cap, D, E)}: all "
                                 "MoE layers of one engine must share dim and E, and no micro-batch may be "
                                 "larger than the first one")
            return self._ws
        from kohakuwullm_b200.parallel.symm import SymmetricPool

        pool = SymmetricPool(self.group)
        table = pool.empty(L.kwu_ep_table_ints(c_int(self.world), c_int(E)), torch.int32, device)
        flags = pool.empty(L.kwu_ep_flag_ints(), torch.int32, device)
        xrecv = pool.empty(cap * D, torch.bfloat16, device)
        yout = pool.empty(cap * D, torch.bfloat16, device)
        meta = pool.empty(cap, torch.int32, device)
        ypairs = pool.empty(n_pairs * D, torch.bfloat16, device)
        table.zero_()
        flags.zero_()
        ypairs.zero_()
        pool.rendezvous_all()
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)
        tabs = tuple(pool.find(t).ptr_table() for t in (table, flags, xrecv, yout, meta, ypairs))
        epochs = torch.zeros(4, dtype=torch.int32, device=device)
        self._ws = dict(pool=pool, table=table, flags=flags, xrecv=xrecv.view(cap, D), yout=yout.view(cap, D),
                        meta=meta, ypairs=ypairs.view(n_pairs, D), n_pairs=n_pairs,
                        pair_ids=torch.arange(n_pairs, dtype=torch.int32, device=device),
                        tabs=tabs, epochs=epochs, cap=cap, El=El,
                        dropped=torch.zeros(1, dtype=torch.int32, device=device))
        self._shape = (cap, D, E)
        return self._ws

    def dropped_pairs(self, reset: bool = True) -> torch.Tensor:
        """Device scalar: (token, expert) pairs of THIS rank that found no room at their owner since the last
        reset, all layers together (the backward reuses the forward's placement). No host sync."""
        if self._ws is None:
            return torch.zeros((), dtype=torch.int32)
        count = self._ws["dropped"].clone().reshape(())
        if reset:
            self._ws["dropped"].zero_()
        return count

    def _barrier(self, ws, kind: int) -> None:
        L = native.require()
        rc = L.kwu_ep_barrier(*ws["tabs"], native.ptr(ws["epochs"]), c_int(kind), c_int(self.rank), c_int(self.world),
                              c_ll(self.limit), native.stream_ptr(), native.ptr(native.status_word()))
        native.check(rc, "ep_barrier")

    # ------------------------------------------------------------------ plan
    @torch.no_grad()
    def plan(self, idx: torch.Tensor, counts: torch.Tensor, D: int) -> EPPlan:
        L = native.require()
        T, k = idx.shape
        E = counts.numel()
        dev = idx.device
        ws = self._workspace(T * k, D, E, dev)
        El, cap = ws["El"], ws["cap"]
        max_tiles = cap // 128
        i32 = dict(dtype=torch.int32, device=dev)
        offsets, totals = torch.empty(El + 1, **i32), torch.empty(El, **i32)
        tiles = torch.empty(max_tiles, 4, **i32)
        send_base, cursors = torch.empty(E, **i32), torch.empty(E, **i32)
        pos_of = torch.empty(T * k, **i32)
        idx32 = idx.to(torch.int32).contiguous().view(-1)
        rc = L.kwu_ep_plan(*ws["tabs"], native.ptr(counts.to(torch.int32)), native.ptr(ws["epochs"]), c_int(self.rank),
                           c_int(self.world), c_int(E), c_int(cap), native.ptr(offsets), native.ptr(totals),
                           native.ptr(tiles), c_int(max_tiles), native.ptr(send_base), native.ptr(cursors),
                           c_ll(self.limit), c_int(1 if self.on_overflow == "raise" else 0), native.stream_ptr(),
                           native.ptr(native.status_word()))
        native.check(rc, "ep_plan")
        return EPPlan(offsets, totals, tiles, send_base, cursors, pos_of, idx32, cap, k, El)

    # ------------------------------------------------------------------ data movement (autograd)
    def dispatch(self, x: torch.Tensor, plan: EPPlan) -> torch.Tensor:
        return _EPDispatch.apply(x, self, plan)

    def combine(self, y_rows: torch.Tensor, weight: torch.Tensor, plan: EPPlan, T: int) -> torch.Tensor:
        return _EPCombine.apply(y_rows, weight, self, plan, T)

    # raw steps shared by forward and backward --------------------------------------------------
    def _push_rows(self, x, plan):
        """rows of x -> owners' receive buffers (first use of the plan assigns the positions)."""
        L = native.require()
        ws = self._ws
        rc = L.kwu_ep_dispatch(*ws["tabs"], c_int(self.world), native.ptr(x), c_int(x.stride(0)), native.ptr(plan.idx),
                               c_int(plan.idx.numel()), c_int(plan.top_k), native.ptr(plan.send_base),
                               native.ptr(plan.cursors), native.ptr(plan.pos_of), c_int(x.shape[1]), c_int(ws["El"]),
                               c_int(ws["cap"]), c_int(self.rank), native.ptr(ws["dropped"]), native.stream_ptr())
        native.check(rc, "ep_dispatch")

    def _take_received(self, plan, D, build_scatter_map: bool = False):
        """barrier, then receive buffer -> private rows with zeroed padding. ``build_scatter_map``: also turn
        the row tags into the scatter map the expert GEMMs use (``plan.row_ptrs``)."""
        L = native.require()
        ws = self._ws
        self._barrier(ws, FLAG_ARRIVED)
        rows = torch.empty(ws["cap"], D, dtype=torch.bfloat16, device=ws["xrecv"].device)
        if build_scatter_map:
            plan.row_ptrs = torch.empty(ws["cap"], dtype=torch.int64, device=rows.device)
        rc = L.kwu_ep_copy_rows(*ws["tabs"], c_int(self.world), c_int(self.rank), native.ptr(ws["xrecv"]),
                                native.ptr(rows), native.ptr(plan.offsets), native.ptr(plan.totals), c_int(ws["El"]),
                                c_int(D), c_int(1), native.ptr(plan.row_ptrs if build_scatter_map else None),
                                native.stream_ptr())
        native.check(rc, "ep_copy_rows")
        return rows

    def output_rows(self) -> torch.Tensor:
        """The peer-visible (cap, D) output buffer. Passed as the nominal output of a GEMM whose epilogue
        scatters its rows to the sources (``row_ptrs``), it tells ``_publish_rows`` that nothing is left to copy."""
        return self._ws["yout"]

    def _publish_rows(self, rows, plan):
        """Make the owners' results visible to the sources. Rows that a GEMM epilogue already scattered into the
        sources' per-pair buffers (``rows`` is then the nominal output buffer) only need the barrier; private
        rows are first copied into the peer-visible output buffer (pull path)."""
        L = native.require()
        ws = self._ws
        in_place = rows.data_ptr() == ws["yout"].data_ptr()
        scattered = in_place and self.scatter_epilogue
        if not in_place:
            rc = L.kwu_ep_copy_rows(*ws["tabs"], c_int(self.world), c_int(self.rank), native.ptr(rows),
                                    native.ptr(ws["yout"]), native.ptr(plan.offsets), native.ptr(plan.totals),
                                    c_int(ws["El"]), c_int(rows.shape[1]), c_int(0), native.ptr(None),
                                    native.stream_ptr())
            native.check(rc, "ep_copy_rows")
        self._barrier(ws, FLAG_OUTPUT)
        return scattered

    def _sum_pairs(self, plan, w, T, D, keep: bool):
        """Local tail of the scattered path: out[t] = sum_slot w[t,slot] * ypairs[t*k + slot]."""
        L = native.require()
        ws = self._ws
        n = plan.idx.numel()
        out = torch.empty(T, D, dtype=torch.bfloat16, device=ws["ypairs"].device)
        rc = L.kwu_moe_combine(native.ptr(ws["ypairs"]), native.ptr(ws["pair_ids"]), native.ptr(w), native.ptr(out),
                               c_int(D), c_int(T), c_int(plan.top_k), c_int(D), native.stream_ptr())
        native.check(rc, "moe_combine")
        kept = ws["ypairs"][:n].clone() if keep else None
        return out, kept

    def _pull(self, plan, w, T, D, keep: bool):
        L = native.require()
        ws = self._ws
        dev = ws["yout"].device
        out = torch.empty(T, D, dtype=torch.bfloat16, device=dev)
        kept = torch.empty(plan.idx.numel(), D, dtype=torch.bfloat16, device=dev) if keep else None
        rc = L.kwu_ep_combine(*ws["tabs"], c_int(self.world), native.ptr(plan.pos_of), native.ptr(plan.idx),
                              native.ptr(w), native.ptr(out), c_int(D), native.ptr(kept), c_int(T), c_int(plan.top_k),
                              c_int(D), c_int(ws["El"]), native.stream_ptr())
        native.check(rc, "ep_combine")
        return out, kept


class _EPDispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, ep: ExpertParallel, plan: EPPlan):
        x = x.contiguous()
        ep._push_rows(x, plan)
        rows = ep._take_received(plan, x.shape[1], build_scatter_map=True)
        ctx.ep, ctx.plan, ctx.T = ep, plan, x.shape[0]
        return rows

    @staticmethod
    def backward(ctx, drows):
        ep, plan = ctx.ep, ctx.plan
        drows = drows.contiguous()
        if ep._publish_rows(drows, plan):
            dx, _ = ep._sum_pairs(plan, None, ctx.T, drows.shape[1], keep=False)
        else:
            dx, _ = ep._pull(plan, None, ctx.T, drows.shape[1], keep=False)
        return dx, None, None


class _EPCombine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y_rows, weight, ep: ExpertParallel, plan: EPPlan, T):
        y_rows = y_rows.contiguous()
        w = weight.reshape(-1).float().contiguous()
        if ep._publish_rows(y_rows, plan):
            out, kept = ep._sum_pairs(plan, w, T, y_rows.shape[1], keep=True)
        else:
            out, kept = ep._pull(plan, w, T, y_rows.shape[1], keep=True)
        ctx.save_for_backward(kept, w)
        ctx.ep, ctx.plan, ctx.wshape, ctx.wdtype = ep, plan, weight.shape, weight.dtype
        return out

    @staticmethod
    def backward(ctx, dout):
        L = native.require()
        kept, w = ctx.saved_tensors
        ep, plan = ctx.ep, ctx.plan
        ws = ep._ws
        dout = dout.contiguous()
        D = dout.shape[1]
        dw = torch.empty_like(w)
        rc = L.kwu_ep_combine_bwd(*ws["tabs"], c_int(ep.world), native.ptr(dout), c_int(dout.stride(0)),
                                  native.ptr(kept), native.ptr(plan.pos_of), native.ptr(plan.idx), native.ptr(w),
                                  native.ptr(dw), c_int(plan.idx.numel()), c_int(plan.top_k), c_int(D),
                                  c_int(ws["El"]), native.stream_ptr())
        native.check(rc, "ep_combine_bwd")
        d_rows = ep._take_received(plan, D)
        return d_rows, dw.view(ctx.wshape).to(ctx.wdtype), None, None, None


def ep_routed_experts(ep: ExpertParallel, x, idx, weight, counts, w_in_local, w_out_local, q_in=None, q_out=None):
    """Expert-parallel routed MLP on the native path. ``w_in_local`` (El, 2H, dim), ``w_out_local`` (El, dim, H);
    ``q_in`` / ``q_out``: their MXFP8 copies (block-scaled fp8 expert GEMMs)."""
    from kohakuwullm_b200.ops.elementwise import swiglu
    from kohakuwullm_b200.ops.moe import grouped_linear

    T, D = x.shape
    plan = ep.plan(idx, counts, D)
    rows = ep.dispatch(x, plan)
    # `stage` is the peer-visible output buffer: the second GEMM (forward) and the first GEMM's dgrad (backward)
    # write it directly. With ``scatter_epilogue`` their epilogues instead store every row straight into the
    # SOURCE rank's per-pair buffer through the scatter map, and the return all-to-all rides on the GEMM's own
    # stores, tile by tile.
    stage = ep.output_rows()
    ptrs = plan.row_ptrs if ep.scatter_epilogue else None   # None: pull path, the GEMMs write `stage` itself
    h = grouped_linear(rows, w_in_local, plan, q_in, dgrad_out=stage, dgrad_row_ptrs=ptrs)
    a = swiglu(h, emit_mx=q_out is not None, emit_mx_grad=q_in is not None)
    y_rows = grouped_linear(a, w_out_local, plan, q_out, out=stage, out_row_ptrs=ptrs)
    return ep.combine(y_rows, weight, plan, T)


# ---------------------------------------------------------------------------------------- reference
class _AllGatherCat(torch.autograd.Function):
    """Concatenate every rank's tensor along dim 0 (equal shapes); backward returns this rank's slice of
    the summed gradient."""

    @staticmethod
    def forward(ctx, t, group):
        world = dist.get_world_size(group)
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t.contiguous(), group=group)
        ctx.group, ctx.n = group, t.shape[0]
        return torch.cat(parts, 0)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        r = dist.get_rank(ctx.group)
        return g[r * ctx.n:(r + 1) * ctx.n], None


def reference_ep_forward(x, idx, weight, w_in_local, w_out_local, group=None):
    """Collective-based oracle (any backend): gather all ranks' tokens and routing, let each rank apply
    its LOCAL experts to every token routed to them, and sum the partial outputs across ranks. Ranks may
    hold different numbers of tokens (shorter ones are padded with unrouted rows)."""
    group = group if group is not None else dist.group.WORLD
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    El = w_in_local.shape[0]
    T = x.shape[0]
    sizes = [torch.zeros(1, dtype=torch.int64, device=x.device) for _ in range(world)]
    dist.all_gather(sizes, torch.tensor([T], dtype=torch.int64, device=x.device), group=group)
    Tmax = int(max(int(s) for s in sizes))
    pad = Tmax - T
    if pad:
        x = torch.cat([x, x.new_zeros(pad, x.shape[1])])
        weight = torch.cat([weight, weight.new_zeros(pad, weight.shape[1])])
        idx = torch.cat([idx, idx.new_full((pad, idx.shape[1]), -1)])
    xa = _AllGatherCat.apply(x, group)
    wa = _AllGatherCat.apply(weight, group)
    ia = _AllGatherCat.apply(idx.to(torch.int64), group)
    y = torch.zeros(xa.shape, dtype=torch.float32, device=x.device)
    for le in range(El):
        mask = ia == rank * El + le                                  # (W*Tmax, k)
        tok = mask.any(-1).nonzero(as_tuple=True)[0]
        if tok.numel() == 0:
            continue
        h = torch.nn.functional.linear(xa[tok], w_in_local[le].to(x.dtype))
        g, v = h.float().chunk(2, dim=-1)
        a = (torch.nn.functional.silu(g) * v).to(x.dtype)
        o = torch.nn.functional.linear(a, w_out_local[le].to(x.dtype)).float()
        gate = (wa[tok].float() * mask[tok].float()).sum(-1, keepdim=True)
        y = y.index_add(0, tok, o * gate)
    y = _ReduceScatterRows.apply(y, group, Tmax)
    return y[:T].to(x.dtype)


class _ReduceScatterRows(torch.autograd.Function):
    """Sum (W*T, D) over ranks and keep this rank's T rows; backward all-gathers the row gradients."""

    @staticmethod
    def forward(ctx, y, group, T):
        y = y.contiguous()
        dist.all_reduce(y, group=group)
        r = dist.get_rank(group)
        ctx.group = group
        return y[r * T:(r + 1) * T].clone()

    @staticmethod
    def backward(ctx, g):
        world = dist.get_world_size(ctx.group)
        parts = [torch.empty_like(g) for _ in range(world)]
        dist.all_gather(parts, g.contiguous(), group=ctx.group)
        return torch.cat(parts, 0), None, None


# ---------------------------------------------------------------------------------------- model surgery
def shard_experts(model: nn.Module, ep: ExpertParallel | None = None, group=None) -> int:
    """Replace every MoE layer's stacked expert tensors by this rank's slice (experts
    ``[rank*El, (rank+1)*El)``), mark them ``ep_local`` and attach the expert-parallel context. Returns
    the number of converted layers. The router stays replicated and keeps all E experts."""
    from kohakuwullm_b200.models.components.moe import MoEMLP

    group = group if group is not None else (ep.group if ep is not None else dist.group.WORLD)
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    n = 0
    for mod in model.modules():
        if not isinstance(mod, MoEMLP) or getattr(mod, "ep_world", 1) > 1:
            continue
        E = mod.num_experts
        if E % world:
            raise ValueError(f"{E} experts do not split over {world} ranks")
        El = E // world
        for name in ("w_in", "w_out"):
            full = getattr(mod, name)
            local = nn.Parameter(full.data[rank * El:(rank + 1) * El].clone(), requires_grad=full.requires_grad)
            local.ep_local = True
            setattr(mod, name, local)
        mod.ep, mod.ep_group, mod.ep_world, mod.ep_rank = ep, group, world, rank
        n += 1
    return n


@torch.no_grad()
def gather_expert_state(state: dict, model: nn.Module, group=None) -> dict:
    """Full-model state dict from an expert-parallel one: every ``ep_local`` tensor is all-gathered along
    the expert dimension (call on all ranks)."""
    out = dict(state)
    for name, p in model.named_parameters():
        if getattr(p, "ep_local", False) and name in out:
            g = group if group is not None else dist.group.WORLD
            parts = [torch.empty_like(p.data) for _ in range(dist.get_world_size(g))]
            dist.all_gather(parts, p.data.contiguous(), group=g)
            out[name] = torch.cat(parts, 0)
    return out


@torch.no_grad()
def scatter_expert_state(state: dict, model: nn.Module, group=None) -> dict:
    """The inverse of ``gather_expert_state``: from a full-model state dict keep, for every ``ep_local``
    parameter, this rank's slice of the expert dimension (so a checkpoint written by any layout loads
    into an expert-parallel model of any group size that divides the expert count)."""
    g = group if group is not None else dist.group.WORLD
    world, rank = dist.get_world_size(g), dist.get_rank(g)
    out = dict(state)
    for name, p in model.named_parameters():
        if getattr(p, "ep_local", False) and name in out:
            full = out[name]
            if full.shape[0] == p.shape[0]:
                continue                      # already a local slice
            if full.shape[0] != p.shape[0] * world:
                raise ValueError(f"{name}: {full.shape[0]} experts do not split into {world} x {p.shape[0]}")
            out[name] = full[rank * p.shape[0]:(rank + 1) * p.shape[0]].clone()
    return out
