"""Routed-expert evaluation: router top-k, counting-sort dispatch, grouped expert GEMMs, combine.

``routed_experts_reference`` is the per-expert PyTorch loop (CPU path and test oracle; one host read of
the expert offsets). ``routed_experts`` is the native, host-sync-free path:

1. ``plan`` — from the router's per-expert ``counts`` build 128-row-aligned expert offsets, the tile table
   of the grouped GEMMs and the placement of every (token, slot) pair (``csrc/moe.cu``);
2. gather the token rows into expert order (padding rows are zero);
3. ``h = rows @ w_in[e]^T`` — grouped tcgen05 GEMM, SwiGLU, ``y = a @ w_out[e]^T`` — grouped GEMM;
4. combine: per-token gather-sum weighted by the gate (deterministic, no atomics on the output).

Backward mirrors it: combine-bwd -> grouped dgrad / grouped wgrad (fp32, straight into ``main_grad``
when the trainer provides it) -> SwiGLU-bwd -> gather-bwd (a per-token gather-sum again).
Buffer sizes are host-known upper bounds (``pairs + E*127`` rows), so nothing waits on the device.
Reference: src/kohakuwullm/kernels/moe/moe_dispatch.py:14-130, grouped_gemm.py:22-362, router.py:76-280.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from kohakuwullm_b200.ops import native
from kohakuwullm_b200.ops.elementwise import swiglu

c_int, c_float = ctypes.c_int, ctypes.c_float
SCORE_IDS = {"sigmoid": 0, "softmax": 1, "sqrtsoftplus": 2}


def routed_experts_reference(x, idx, weight, w_in, w_out):
    """x (T,dim); idx (T,k) expert ids; weight (T,k); w_in (E,2H,dim); w_out (E,dim,H)."""
    T, dim = x.shape
    k = idx.shape[1]
    E = w_in.shape[0]
    flat_expert = idx.reshape(-1).long()
    order = torch.argsort(flat_expert, stable=True)          # pair index sorted by expert
    token_of = order // k
    counts = torch.bincount(flat_expert, minlength=E)
    bounds = torch.cumsum(counts, 0).tolist()
    rows = x[token_of]
    out_rows = torch.empty(rows.shape[0], dim, dtype=x.dtype, device=x.device)
    start = 0
    for e in range(E):
        end = bounds[e]
        if end > start:
            h = torch.nn.functional.linear(rows[start:end], w_in[e].to(x.dtype))
            g, v = h.float().chunk(2, dim=-1)
            a = (torch.nn.functional.silu(g) * v).to(x.dtype)
            out_rows[start:end] = torch.nn.functional.linear(a, w_out[e].to(x.dtype))
        start = end
    gate = weight.reshape(-1)[order].to(torch.float32)
    y = torch.zeros(T, dim, dtype=torch.float32, device=x.device)
    y.index_add_(0, token_of, out_rows.float() * gate[:, None])
    return y.to(x.dtype)


def native_supported(x, w_in) -> bool:
    return (native.available() and x.is_cuda and x.dtype == torch.bfloat16 and w_in.dtype == torch.bfloat16
            and x.shape[-1] % 64 == 0 and w_in.shape[1] % 128 == 0 and w_in.shape[0] <= 128)


# ------------------------------------------------------------------------------------ router
class _RouterTopK(torch.autograd.Function):
    """Gate logits on the tensor cores (fp32 gate matrix as a bf16 hi/lo pair), then one kernel for score,
    biased top-k, gate weights and the load histogram. Backward: one kernel turns the gate-weight gradient into
    logit gradients (normalisation, scaling, score function; dense auxiliary-loss logit gradients are added);
    ``dx = dl W`` and ``dW += dl^T x`` run on the tensor-core GEMM with bf16 operands and fp32 accumulation,
    the latter straight into ``main_grad`` when the trainer provides it. The all-fp32 SIMT tile kernels
    (``kwu_moe_router_fwd`` with ``x``, ``kwu_moe_router_bwd`` with ``dx`` / ``dW``) remain in the library."""

    @staticmethod
    def forward(ctx, x, W, bias, load_accum, top_k, score, norm_topk, scaling):
        from kohakuwullm_b200.ops.gemm import matmul

        L = native.require()
        T, D = x.shape
        E = W.shape[0]
        logits = torch.empty(T, E, dtype=torch.float32, device=x.device)
        idx = torch.empty(T, top_k, dtype=torch.int32, device=x.device)
        weight = torch.empty(T, top_k, dtype=torch.float32, device=x.device)
        counts = torch.zeros(E, dtype=torch.int32, device=x.device)
        tensor_core = D % 8 == 0 and x.stride(1) == 1
        if tensor_core:
            # gate logits on the tensor cores with the fp32 gate matrix split into a bf16 head and a bf16
            # remainder: x W_hi^T + x W_lo^T, fp32 accumulation, keeps ~16 mantissa bits of W
            w_hi = W.detach().to(torch.bfloat16)
            w_lo = (W.detach() - w_hi.float()).to(torch.bfloat16)
            xc = x if x.is_contiguous() else x.contiguous()
            matmul(xc, w_hi, out=logits)
            matmul(xc, w_lo, out=logits, accumulate=True)
        rc = L.kwu_moe_router_fwd(native.ptr(None if tensor_core else x), c_int(x.stride(0)), native.ptr(W),
                                  native.ptr(bias), native.ptr(logits), native.ptr(idx), native.ptr(weight),
                                  native.ptr(counts), native.ptr(load_accum), c_int(T), c_int(D), c_int(E), c_int(top_k),
                                  c_int(SCORE_IDS[score]), c_int(int(norm_topk)), c_float(scaling), native.stream_ptr())
        native.check(rc, "moe_router_fwd")
        ctx.save_for_backward(x, W, logits, idx)
        ctx.cfg = (score, norm_topk, scaling)
        ctx.weight_param = W
        ctx.mark_non_differentiable(idx, counts)
        return idx, weight, counts, logits

    @staticmethod
    def backward(ctx, _didx, dweight, _dcounts, dlogits_in):
        from kohakuwullm_b200.ops.gemm import matmul

        L = native.require()
        x, W, logits, idx = ctx.saved_tensors
        score, norm_topk, scaling = ctx.cfg
        T, D = x.shape
        E = W.shape[0]
        k = idx.shape[1]
        dl = torch.empty(T, E, dtype=torch.float32, device=x.device)
        dl16 = torch.empty(T, E, dtype=torch.bfloat16, device=x.device)
        dw_in = dweight.float().contiguous() if dweight is not None else torch.zeros(T, k, dtype=torch.float32, device=x.device)
        dl_in = dlogits_in.float().contiguous() if dlogits_in is not None else None
        need_dx, need_dW = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        # logit gradient (fp32 and a bf16 copy); the two gate-matrix products then run on the tensor cores
        rc = L.kwu_moe_router_bwd(native.ptr(logits), native.ptr(idx), native.ptr(dw_in), native.ptr(dl_in), native.ptr(dl),
                                  native.ptr(dl16), native.ptr(None), c_int(0), native.ptr(W), native.ptr(None), c_int(0),
                                  native.ptr(None), c_int(T), c_int(D), c_int(E), c_int(k), c_int(SCORE_IDS[score]),
                                  c_int(int(norm_topk)), c_float(scaling), native.stream_ptr())
        native.check(rc, "moe_router_bwd")
        xc = x if x.is_contiguous() else x.contiguous()
        dx = matmul(dl16, W.detach().to(torch.bfloat16), b_mn=True, out_dtype=x.dtype) if need_dx else None
        dW = None
        if need_dW:
            main_grad = getattr(ctx.weight_param, "main_grad", None)
            into_main = main_grad is not None and main_grad.dtype == torch.float32 and main_grad.is_contiguous()
            target = main_grad if into_main else torch.zeros(E, D, dtype=torch.float32, device=x.device)
            matmul(dl16, xc, a_mn=True, b_mn=True, out=target, accumulate=True)    # dW += dl^T x, fp32
            if not into_main:
                dW = target.to(W.dtype)
        return dx, dW, None, None, None, None, None, None


def router_topk(x, W, bias, load_accum, top_k, score="sigmoid", norm_topk=True, scaling=1.0):
    """Native router. Returns ``(idx int32 (T,k), weight fp32 (T,k), counts int32 (E,), logits fp32 (T,E))``."""
    return _RouterTopK.apply(x, W, bias, load_accum, top_k, score, norm_topk, float(scaling))


def router_supported(x, W, num_groups: int) -> bool:
    return (native.available() and x.is_cuda and x.dtype == torch.bfloat16 and W.dtype == torch.float32
            and W.shape[0] <= 128 and W.shape[0] % 8 == 0 and num_groups <= 1)


# ------------------------------------------------------------------------------------ dispatch plan
@dataclass
class DispatchPlan:
    offsets: torch.Tensor    # (E+1,) int32, 128-aligned expert row offsets; offsets[E] = rows in use
    tiles: torch.Tensor      # (max_tiles, 4) int32: (m0, expert, valid, 0)
    pos_of: torch.Tensor     # (T*k,) int32 row of every (token, slot) pair
    pair_of: torch.Tensor    # (max_rows,) int32 pair of every row, -1 for padding
    max_rows: int
    top_k: int
    num_experts: int


def make_plan(idx: torch.Tensor, counts: torch.Tensor, num_experts: int) -> DispatchPlan:
    L = native.require()
    T, k = idx.shape
    n_pairs = T * k
    max_rows = L.kwu_moe_max_rows(c_int(n_pairs), c_int(num_experts))
    max_tiles = max_rows // 128
    dev = idx.device
    offsets = torch.empty(num_experts + 1, dtype=torch.int32, device=dev)
    cursors = torch.empty(num_experts, dtype=torch.int32, device=dev)
    tiles = torch.empty(max_tiles, 4, dtype=torch.int32, device=dev)
    pos_of = torch.empty(n_pairs, dtype=torch.int32, device=dev)
    pair_of = torch.empty(max_rows, dtype=torch.int32, device=dev)
    rc = L.kwu_moe_plan_and_place(native.ptr(counts), native.ptr(idx), c_int(n_pairs), c_int(num_experts),
                                  native.ptr(offsets), native.ptr(cursors), native.ptr(tiles), c_int(max_tiles),
                                  native.ptr(pos_of), native.ptr(pair_of), c_int(max_rows), native.stream_ptr())
    native.check(rc, "moe_plan_and_place")
    return DispatchPlan(offsets, tiles, pos_of, pair_of, max_rows, k, num_experts)


class _Gather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, plan: DispatchPlan, emit_mx=False):
        """``emit_mx``: also write the MXFP8 copy of the gathered rows for the MXFP8 expert GEMM that follows."""
        from kohakuwullm_b200.ops import mxfp8 as mx

        L = native.require()
        T, D = x.shape
        rows = torch.empty(plan.max_rows, D, dtype=x.dtype, device=x.device)
        q = sf = None
        if emit_mx and mx.can_emit(plan.max_rows, D):
            q, sf = mx.alloc_quantized(plan.max_rows, D, x.device)
        rc = L.kwu_moe_gather(native.ptr(x), c_int(x.stride(0)), native.ptr(plan.pair_of), c_int(plan.top_k),
                              native.ptr(rows), c_int(D), c_int(plan.max_rows), native.ptr(plan.offsets),
                              c_int(plan.num_experts), native.ptr(q), native.ptr(sf), native.stream_ptr())
        native.check(rc, "moe_gather")
        if q is not None:
            mx.stash_quantized(rows, q, sf)
        ctx.plan, ctx.T = plan, T
        return rows

    @staticmethod
    def backward(ctx, drows):
        L = native.require()
        plan = ctx.plan
        D = drows.shape[1]
        dx = torch.empty(ctx.T, D, dtype=drows.dtype, device=drows.device)
        rc = L.kwu_moe_combine(native.ptr(drows.contiguous()), native.ptr(plan.pos_of), native.ptr(None), native.ptr(dx),
                               c_int(D), c_int(ctx.T), c_int(plan.top_k), c_int(D), native.stream_ptr())
        native.check(rc, "moe_gather_bwd")
        return dx, None, None


class _GroupedLinear(torch.autograd.Function):
    """``out[rows of expert e] = rows @ W[e]^T`` with W (E, N, K)."""

    @staticmethod
    def forward(ctx, rows, W, plan: DispatchPlan, out=None, dgrad_out=None, out_row_ptrs=None, dgrad_row_ptrs=None):
        """``out`` / ``dgrad_out``: caller-owned (max_rows, N) / (max_rows, K) buffers for the product and for
        the input gradient. ``out_row_ptrs`` / ``dgrad_row_ptrs``: (max_rows,) int64 scatter maps; the kernel's
        epilogue then stores row r at that byte address (0: dropped) instead of into the buffer, which may be
        another GPU's peer-mapped memory (expert parallelism returns rows to their source ranks this way)."""
        L = native.require()
        E, N, K = W.shape
        if out is None:
            out = torch.empty(plan.max_rows, N, dtype=rows.dtype, device=rows.device)
        ctx.dgrad_out, ctx.dgrad_row_ptrs = dgrad_out, dgrad_row_ptrs
        rc = L.kwu_gemm_bf16_grouped_rows(native.ptr(rows), native.ptr(W), native.ptr(out), c_int(plan.max_rows), c_int(N),
                                          c_int(K), c_int(rows.stride(0)), c_int(K), c_int(N), c_int(0), c_int(E),
                                          native.ptr(plan.tiles), c_int(plan.tiles.shape[0]), c_int(0),
                                          native.ptr(out_row_ptrs), native.stream_ptr(),
                                          native.ptr(native.status_word()))
        native.check(rc, "grouped_gemm_fwd")
        ctx.save_for_backward(rows, W)
        ctx.plan = plan
        return out

    @staticmethod
    def backward(ctx, dout):
        L = native.require()
        rows, W = ctx.saved_tensors
        plan = ctx.plan
        E, N, K = W.shape
        dout = dout.contiguous()
        drows = dW = None
        if ctx.needs_input_grad[0]:
            drows = ctx.dgrad_out if ctx.dgrad_out is not None else \
                torch.empty(plan.max_rows, K, dtype=rows.dtype, device=rows.device)
            # dx = dy W_e : B = W viewed as (E*N, K) stored [contraction N rows][K cols] per expert
            rc = L.kwu_gemm_bf16_grouped_rows(native.ptr(dout), native.ptr(W), native.ptr(drows), c_int(plan.max_rows),
                                              c_int(K), c_int(N), c_int(dout.stride(0)), c_int(K), c_int(K), c_int(1),
                                              c_int(E), native.ptr(plan.tiles), c_int(plan.tiles.shape[0]), c_int(0),
                                              native.ptr(ctx.dgrad_row_ptrs), native.stream_ptr(),
                                              native.ptr(native.status_word()))
            native.check(rc, "grouped_gemm_dgrad")
        if ctx.needs_input_grad[1]:
            main_grad = getattr(W, "main_grad", None)
            target = main_grad if main_grad is not None else torch.zeros(E, N, K, dtype=torch.float32, device=W.device)
            rc = L.kwu_gemm_bf16_grouped_wgrad(native.ptr(dout), native.ptr(rows), native.ptr(target), c_int(plan.max_rows),
                                               c_int(N), c_int(K), c_int(dout.stride(0)), c_int(rows.stride(0)), c_int(E),
                                               native.ptr(plan.offsets), c_int(1), c_int(1), native.stream_ptr(),
                                               native.ptr(native.status_word()))
            native.check(rc, "grouped_gemm_wgrad")
            if main_grad is None:
                dW = target.to(W.dtype)
        return drows, dW, None, None, None, None, None


class _Combine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, rows, weight, plan: DispatchPlan, T, emit_mx_grad=False):
        L = native.require()
        D = rows.shape[1]
        out = torch.empty(T, D, dtype=rows.dtype, device=rows.device)
        w = weight.reshape(-1).float().contiguous()
        rc = L.kwu_moe_combine(native.ptr(rows), native.ptr(plan.pos_of), native.ptr(w), native.ptr(out), c_int(D),
                               c_int(T), c_int(plan.top_k), c_int(D), native.stream_ptr())
        native.check(rc, "moe_combine")
        ctx.save_for_backward(rows, w)
        ctx.plan, ctx.wshape, ctx.wdtype = plan, weight.shape, weight.dtype
        ctx.emit_mx_grad = emit_mx_grad
        return out

    @staticmethod
    def backward(ctx, dout):
        L = native.require()
        rows, w = ctx.saved_tensors
        plan = ctx.plan
        D = rows.shape[1]
        dout = dout.contiguous()
        from kohakuwullm_b200.ops import mxfp8 as mx

        drows = torch.empty_like(rows)
        dw = torch.zeros_like(w)
        q = sf = None
        if ctx.emit_mx_grad and mx.can_emit(rows.shape[0], D):
            q, sf = mx.alloc_quantized(rows.shape[0], D, rows.device)
        rc = L.kwu_moe_combine_bwd(native.ptr(rows), native.ptr(dout), c_int(dout.stride(0)), native.ptr(plan.pair_of),
                                   native.ptr(w), native.ptr(drows), native.ptr(dw), c_int(plan.top_k), c_int(D),
                                   native.ptr(plan.offsets), c_int(plan.num_experts), native.ptr(q), native.ptr(sf),
                                   native.stream_ptr())
        native.check(rc, "moe_combine_bwd")
        if q is not None:
            mx.stash_quantized(drows, q, sf)
        return drows, dw.view(ctx.wshape).to(ctx.wdtype), None, None, None


def grouped_linear(rows, W, plan, qweight=None, out=None, dgrad_out=None, out_row_ptrs=None, dgrad_row_ptrs=None):
    """Expert-grouped linear: bf16 tcgen05 GEMM, or the MXFP8 recipe when ``qweight`` (a
    ``GroupedQuantizedWeight`` of ``W``) is given. ``out`` / ``dgrad_out``: optional caller-owned buffers for
    the product and for the input gradient; ``out_row_ptrs`` / ``dgrad_row_ptrs``: optional scatter maps for
    their rows (see ``_GroupedLinear.forward``)."""
    if qweight is not None:
        from kohakuwullm_b200.ops.mxfp8 import _MXFP8GroupedLinear

        return _MXFP8GroupedLinear.apply(rows, W, qweight, plan, out, dgrad_out, out_row_ptrs, dgrad_row_ptrs)
    return _GroupedLinear.apply(rows, W, plan, out, dgrad_out, out_row_ptrs, dgrad_row_ptrs)


def routed_experts(x, idx, weight, counts, w_in, w_out, q_in=None, q_out=None):
    """Native routed-expert MLP. ``idx`` (T,k) int32, ``weight`` (T,k), ``counts`` (E,) int32 from the router.
    ``q_in`` / ``q_out``: MXFP8 copies of the expert weights (both GEMMs then run block-scaled fp8)."""
    T = x.shape[0]
    plan = make_plan(idx.to(torch.int32).contiguous(), counts.to(torch.int32), w_in.shape[0])
    # with MXFP8 experts every producer writes the fp8 copy its consumer needs in the same pass
    rows = _Gather.apply(x.contiguous(), plan, q_in is not None)
    h = grouped_linear(rows, w_in, plan, q_in)
    a = swiglu(h, emit_mx=q_out is not None, emit_mx_grad=q_in is not None)
    y_rows = grouped_linear(a, w_out, plan, q_out)
    return _Combine.apply(y_rows, weight, plan, T, q_out is not None)
