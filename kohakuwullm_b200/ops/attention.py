"""Packed variable-length causal / sliding-window attention with attention sinks.

Inputs are packed: ``q`` (T,Hq,D), ``k``/``v`` (T,Hkv,D), ``cu_seqlens`` (N+1,) int32. A query
attends to keys of its own document only, never to later positions, and (with ``window=w``) only
to the ``w`` most recent positions including itself. Attention sinks are extra softmax columns
with a learned logit and a zero value: with ``sink_lse[h] = logsumexp(sinks[h, :])`` the result
equals ``softmax-attention * sigmoid(lse - sink_lse)`` (one sink per head is the reference's
``out * sigmoid(lse - sink)``, src/kohakuwullm/models/components/attention.py:91-100).

``varlen_attention`` runs the tcgen05 flash kernels (``csrc/flash_fwd.cu`` / ``flash_bwd.cu``)
for bf16 CUDA tensors with head_dim 64 and the fp32 PyTorch reference everywhere else.
Reference kernels: src/kohakuwullm/kernels/attention/flash_attn_fwd.py:35-154,
flash_attn_bwd.py:16-348.
"""

from __future__ import annotations

import ctypes
import math
import os

import torch

from kohakuwullm_b200.ops import native

c_int, c_float = ctypes.c_int, ctypes.c_float


def _doc_ids(cu_seqlens: torch.Tensor, total: int) -> torch.Tensor:
    idx = torch.arange(total, device=cu_seqlens.device)
    return torch.searchsorted(cu_seqlens[1:].to(torch.long).contiguous(), idx, right=True)


def attention_mask(cu_seqlens: torch.Tensor, total: int, window: int | None) -> torch.Tensor:
    """(T,T) bool mask, true where query i may attend key j."""
    doc = _doc_ids(cu_seqlens, total)
    i = torch.arange(total, device=cu_seqlens.device)
    allowed = (doc[:, None] == doc[None, :]) & (i[None, :] <= i[:, None])
    if window is not None:
        allowed &= (i[:, None] - i[None, :]) < window
    return allowed


def varlen_attention_reference(q, k, v, cu_seqlens, window=None, sink_lse=None, scale=None,
                               return_lse=False):
    """fp32 oracle. Works document by document so memory stays O(max_len^2)."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    group = Hq // Hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    bounds = cu_seqlens.tolist()
    outs, lses = [], []
    for s, e in zip(bounds[:-1], bounds[1:]):
        L = e - s
        qf = q[s:e].float().transpose(0, 1)                              # (Hq, L, D)
        kf = k[s:e].float().transpose(0, 1).repeat_interleave(group, 0)  # (Hq, L, D)
        vf = v[s:e].float().transpose(0, 1).repeat_interleave(group, 0)
        scores = torch.matmul(qf, kf.transpose(1, 2)) * scale           # (Hq, L, L)
        i = torch.arange(L, device=q.device)
        ok = i[None, :] <= i[:, None]
        if window is not None:
            ok &= (i[:, None] - i[None, :]) < window
        scores = scores.masked_fill(~ok, float("-inf"))
        lse = torch.logsumexp(scores, dim=-1)                             # (Hq, L)
        if sink_lse is not None:
            lse = torch.logaddexp(lse, sink_lse.float()[:, None])
        p = torch.exp(scores - lse[..., None])
        outs.append(torch.matmul(p, vf).transpose(0, 1))                  # (L, Hq, D)
        lses.append(lse)
    out = torch.cat(outs, 0).to(q.dtype) if outs else q.new_zeros(q.shape)
    if return_lse:
        return out, torch.cat(lses, 1)
    return out


# --------------------------------------------------------------------------------- native path
def attention_plan(cu_seqlens: torch.Tensor, total_tokens: int, tile: int = 128) -> torch.Tensor:
    """Device-side work lists: one int4 ``(q0, doc_start, doc_end, valid)`` per 128-row tile, twice.

    Rows ``[0, n)`` hold the tiles sorted by how many keys a query tile sees (heaviest first: the order in
    which the forward and dQ kernels hand them to their persistent CTAs), rows ``[n, 2n)`` the same tiles
    sorted by how many queries see a key tile (the dK / dV kernel). ``n = ceil(T/tile) + num_docs`` is a
    host-known upper bound on the number of tiles (unused entries are marked invalid and sort last), so
    building and using the lists needs no host synchronisation and is graph-capturable.
    """
    L = native.require()
    ndocs = cu_seqlens.numel() - 1
    max_tiles = (total_tokens + tile - 1) // tile + ndocs
    plan = torch.empty(2 * max_tiles, 4, dtype=torch.int32, device=cu_seqlens.device)
    rc = L.kwu_attn_plan(native.ptr(cu_seqlens), c_int(ndocs), c_int(tile), native.ptr(plan),
                         c_int(max_tiles), native.stream_ptr())
    native.check(rc, "attn_plan")
    return plan


class _FlashVarlen(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens, plan, window, sink_lse, scale):
        L = native.require()
        T, Hq, D = q.shape
        Hkv = k.shape[1]
        out = torch.empty(T, Hq, D, dtype=q.dtype, device=q.device)
        lse = torch.empty(Hq, T, dtype=torch.float32, device=q.device)
        rc = L.kwu_flash_fwd(
            native.ptr(q), c_int(q.stride(0)), native.ptr(k), c_int(k.stride(0)), native.ptr(v),
            c_int(v.stride(0)), native.ptr(out), native.ptr(lse), native.ptr(plan),
            c_int(plan.shape[0] // 2), c_int(T), c_int(Hq), c_int(Hkv), c_int(window or 0),
            native.ptr(sink_lse), c_float(scale), native.stream_ptr(), native.ptr(native.status_word()),
        )
        native.check(rc, "flash_fwd")
        ctx.save_for_backward(q, k, v, out, lse, plan, sink_lse, cu_seqlens)
        ctx.window, ctx.scale = window, scale
        ctx.mark_non_differentiable(lse)
        return out, lse

    @staticmethod
    def backward(ctx, dout, _dlse):
        L = native.require()
        q, k, v, out, lse, plan, sink_lse, cu_seqlens = ctx.saved_tensors
        T, Hq, D = q.shape
        Hkv = k.shape[1]
        dout = dout.contiguous()
        dq = torch.empty(T, Hq, D, dtype=q.dtype, device=q.device)
        dk = torch.empty(T, Hkv, D, dtype=q.dtype, device=q.device)
        dv = torch.empty(T, Hkv, D, dtype=q.dtype, device=q.device)
        delta = torch.empty(Hq, T, dtype=torch.float32, device=q.device)
        n_scratch = L.kwu_flash_bwd_scratch_floats(c_int(T), c_int(Hq), c_int(Hkv))
        scratch = torch.empty(n_scratch, dtype=torch.float32, device=q.device) if n_scratch else None
        rc = L.kwu_flash_bwd(
            native.ptr(q), c_int(q.stride(0)), native.ptr(k), c_int(k.stride(0)), native.ptr(v),
            c_int(v.stride(0)), native.ptr(out), native.ptr(dout), native.ptr(lse), native.ptr(delta),
            native.ptr(dq), native.ptr(dk), c_int(dk.stride(0)), native.ptr(dv), c_int(dv.stride(0)),
            native.ptr(scratch), native.ptr(plan),
            c_int(plan.shape[0] // 2), c_int(T), c_int(Hq), c_int(Hkv), c_int(ctx.window or 0),
            c_float(ctx.scale), native.stream_ptr(), native.ptr(native.status_word()),
        )
        native.check(rc, "flash_bwd")
        dsink = None
        if sink_lse is not None and ctx.needs_input_grad[6]:
            # sink columns carry a zero value, so dS_sink = -p_sink * delta summed over queries
            dsink = -(torch.exp(sink_lse.float()[:, None] - lse) * delta).sum(1).to(sink_lse.dtype)
        return dq, dk, dv, None, None, None, dsink, None


def native_supported(q, k, v) -> bool:
    return (
        native.available() and q.is_cuda and q.dtype == torch.bfloat16 and k.dtype == q.dtype
        and v.dtype == q.dtype and q.shape[-1] == 64 and q.stride(-1) == 1 and k.stride(-1) == 1
        and v.stride(-1) == 1 and q.stride(1) == 64 and k.stride(1) == 64 and v.stride(1) == 64
    )


def _block_attention(qb, kf, vf, q0: int, window, sink, scale: float):
    """Rows [q0, q0 + len(qb)) of ONE document against its keys [lo, q0 + len(qb)): (out, lse) in fp32."""
    Lq = qb.shape[1]
    hi = q0 + Lq
    lo = max(0, q0 - window + 1) if window is not None else 0
    scores = torch.matmul(qb, kf[:, lo:hi].transpose(1, 2)) * scale            # (Hq, Lq, hi - lo)
    qi = torch.arange(q0, hi, device=qb.device)[:, None]
    kj = torch.arange(lo, hi, device=qb.device)[None, :]
    ok = kj <= qi
    if window is not None:
        ok &= (qi - kj) < window
    scores = scores.masked_fill(~ok, float("-inf"))
    lse = torch.logsumexp(scores, dim=-1)
    if sink is not None:
        lse = torch.logaddexp(lse, sink[:, None])
    return torch.matmul(torch.exp(scores - lse[..., None]), vf[:, lo:hi]), lse


def varlen_attention_blockwise(q, k, v, cu_seqlens, window=None, sink_lse=None, scale=None, return_lse=False,
                               block: int = 1024):
    """PyTorch path for head sizes the native kernels do not cover (they are written for 64): the same
    semantics as the oracle above, but a document is processed ``block`` query rows at a time, each block under
    activation recomputation, so the peak is (heads x block x keys) instead of (heads x L x L) in forward AND
    backward, and a sliding window also bounds the keys a block touches."""
    from torch.utils.checkpoint import checkpoint

    T, Hq, D = q.shape
    group = Hq // k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    sink = sink_lse.float() if sink_lse is not None else None
    bounds = cu_seqlens.tolist()
    outs, lses = [], []
    for s, e in zip(bounds[:-1], bounds[1:]):
        qf = q[s:e].float().transpose(0, 1)
        kf = k[s:e].float().transpose(0, 1).repeat_interleave(group, 0)
        vf = v[s:e].float().transpose(0, 1).repeat_interleave(group, 0)
        for q0 in range(0, e - s, block):
            qb = qf[:, q0:q0 + block]
            if torch.is_grad_enabled() and (qb.requires_grad or kf.requires_grad or vf.requires_grad):
                o, l = checkpoint(_block_attention, qb, kf, vf, q0, window, sink, float(scale), use_reentrant=False)
            else:
                o, l = _block_attention(qb, kf, vf, q0, window, sink, float(scale))
            outs.append(o.transpose(0, 1))
            lses.append(l)
    out = torch.cat(outs, 0).to(q.dtype) if outs else q.new_zeros(q.shape)
    return (out, torch.cat(lses, 1)) if return_lse else out


def varlen_attention(q, k, v, cu_seqlens, max_seqlen=None, window=None, sink_lse=None, scale=None,
                     plan=None, return_lse=False):
    """Packed causal attention; see the module docstring for the semantics."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if native_supported(q, k, v):
        if plan is None:
            plan = attention_plan(cu_seqlens, q.shape[0])
        if sink_lse is not None:
            sink_lse = sink_lse.float()
        out, lse = _FlashVarlen.apply(q, k, v, cu_seqlens, plan, window, sink_lse, float(scale))
        return (out, lse) if return_lse else out
    return varlen_attention_blockwise(q, k, v, cu_seqlens, window, sink_lse, scale, return_lse)


# --------------------------------------------------------------------------------- fused core
# KWU_FUSED_QK=0 restores one norm+rope launch per tensor and the separate quantise passes (A/B timing only)
FUSED_QK = os.environ.get("KWU_FUSED_QK", "1") != "0"


class _AttentionCore(torch.autograd.Function):
    """QK-norm + RoPE + flash attention over a fused ``qkv`` projection output, as ONE autograd node.

    Forward reads q / k / v as strided slices of ``qkv`` (no split copies). Backward writes the three
    gradient slices straight into one ``dqkv`` buffer: dv by the flash backward kernel, dq / dk by the
    norm+rope backward kernel, so autograd never materialises zero-padded slice gradients.
    """

    @staticmethod
    def forward(ctx, qkv, q_norm, k_norm, cos, sin, cu_seqlens, plan, sink_lse, Hq, Hkv, window, scale,
                eps, do_norm, emit_mx_grad=False, emit_mx_out=False):
        from kohakuwullm_b200.ops.elementwise import c_float as cf, c_int as ci

        L = native.require()
        T = qkv.shape[0]
        D = 64
        ld = qkv.stride(0)
        q_src = qkv[:, : Hq * D]
        k_src = qkv[:, Hq * D:(Hq + Hkv) * D]
        v = qkv[:, (Hq + Hkv) * D:].view(T, Hkv, D)
        q = torch.empty(T, Hq, D, dtype=qkv.dtype, device=qkv.device)
        k = torch.empty(T, Hkv, D, dtype=qkv.dtype, device=qkv.device)
        rot_half = 0 if cos is None else cos.shape[-1]
        fused_qk = FUSED_QK and rot_half in (0, 32) and ld % 8 == 0 and qkv.data_ptr() % 16 == 0
        emit_mx_out = emit_mx_out and FUSED_QK
        if fused_qk:
            # q and k heads in one launch (they are adjacent in the projection output)
            rc = L.kwu_qknorm_rope_fwd_qk(native.ptr(qkv), ci(ld), native.ptr(q), native.ptr(k), native.ptr(q_norm),
                                          native.ptr(k_norm), native.ptr(cos), native.ptr(sin), ci(T), ci(Hq), ci(Hkv),
                                          ci(rot_half), cf(eps), ci(int(do_norm)), native.stream_ptr())
            native.check(rc, "qknorm_rope_fwd_qk")
        else:
            for src, dst, w, H in ((q_src, q, q_norm, Hq), (k_src, k, k_norm, Hkv)):
                rc = L.kwu_qknorm_rope_fwd(native.ptr(src), ci(ld), native.ptr(dst), ci(H * D), native.ptr(w),
                                           native.ptr(cos), native.ptr(sin), ci(T), ci(H), ci(D), ci(rot_half),
                                           cf(eps), ci(int(do_norm)), native.stream_ptr())
                native.check(rc, "qknorm_rope_fwd")
        out = torch.empty(T, Hq, D, dtype=qkv.dtype, device=qkv.device)
        lse = torch.empty(Hq, T, dtype=torch.float32, device=qkv.device)
        o8 = osf = None
        if emit_mx_out:
            from kohakuwullm_b200.ops import mxfp8 as mx

            if mx.can_emit(T, Hq * D):
                # the epilogue also writes the e4m3 + scale copy of the output for an MXFP8 output projection
                o8, osf = mx.alloc_quantized(T, Hq * D, qkv.device)
        if o8 is not None:
            rc = L.kwu_flash_fwd_mx(native.ptr(q), ci(Hq * D), native.ptr(k), ci(Hkv * D), native.ptr(v), ci(ld),
                                    native.ptr(out), native.ptr(lse), native.ptr(plan), ci(plan.shape[0] // 2), ci(T),
                                    ci(Hq), ci(Hkv), ci(window or 0), native.ptr(sink_lse), cf(scale),
                                    native.ptr(o8), native.ptr(osf), native.stream_ptr(),
                                    native.ptr(native.status_word()))
            mx.stash_quantized(out.view(T, Hq * D), o8, osf)
        else:
            rc = L.kwu_flash_fwd(native.ptr(q), ci(Hq * D), native.ptr(k), ci(Hkv * D), native.ptr(v), ci(ld),
                                 native.ptr(out), native.ptr(lse), native.ptr(plan), ci(plan.shape[0] // 2), ci(T),
                                 ci(Hq), ci(Hkv), ci(window or 0), native.ptr(sink_lse), cf(scale),
                                 native.stream_ptr(), native.ptr(native.status_word()))
        native.check(rc, "flash_fwd")
        ctx.save_for_backward(qkv, q, k, out, lse, plan, sink_lse, q_norm, k_norm, cos, sin)
        ctx.cfg = (Hq, Hkv, window, scale, eps, do_norm)
        ctx.fused_qk, ctx.emit_mx_grad = fused_qk, bool(emit_mx_grad)
        ctx.norm_params = (q_norm, k_norm)   # Parameter objects: their ``main_grad`` takes the gradients directly
        return out

    @staticmethod
    def backward(ctx, dout):
        from kohakuwullm_b200.ops.elementwise import c_float as cf, c_int as ci

        L = native.require()
        qkv, q, k, out, lse, plan, sink_lse, q_norm, k_norm, cos, sin = ctx.saved_tensors
        Hq, Hkv, window, scale, eps, do_norm = ctx.cfg
        T, D = qkv.shape[0], 64
        ld = qkv.stride(0)
        dout = dout.contiguous()
        dqkv = torch.empty_like(qkv)
        dld = dqkv.stride(0)
        dq = torch.empty(T, Hq, D, dtype=qkv.dtype, device=qkv.device)
        dk = torch.empty(T, Hkv, D, dtype=qkv.dtype, device=qkv.device)
        dv = dqkv[:, (Hq + Hkv) * D:]
        v = qkv[:, (Hq + Hkv) * D:]
        delta = torch.empty(Hq, T, dtype=torch.float32, device=qkv.device)
        n_scratch = L.kwu_flash_bwd_scratch_floats(ci(T), ci(Hq), ci(Hkv))
        scratch = torch.empty(n_scratch, dtype=torch.float32, device=qkv.device) if n_scratch else None
        rc = L.kwu_flash_bwd(native.ptr(q), ci(Hq * D), native.ptr(k), ci(Hkv * D), native.ptr(v), ci(ld),
                             native.ptr(out), native.ptr(dout), native.ptr(lse), native.ptr(delta),
                             native.ptr(dq), native.ptr(dk), ci(Hkv * D), native.ptr(dv), ci(dld),
                             native.ptr(scratch), native.ptr(plan), ci(plan.shape[0] // 2), ci(T), ci(Hq), ci(Hkv),
                             ci(window or 0), cf(scale), native.stream_ptr(), native.ptr(native.status_word()))
        native.check(rc, "flash_bwd")
        rot_half = 0 if cos is None else cos.shape[-1]
        dws = []
        targets = []
        for w, wp in ((q_norm, ctx.norm_params[0]), (k_norm, ctx.norm_params[1])):
            mg = getattr(wp, "main_grad", None)
            into_main = w is not None and mg is not None and mg.dtype == torch.float32 and mg.is_contiguous()
            dw = (mg if into_main else torch.zeros(D, dtype=torch.float32, device=qkv.device)) if w is not None else None
            targets.append((w, dw, into_main))
        if ctx.fused_qk:
            from kohakuwullm_b200.ops import mxfp8 as mx

            q8 = sf = None
            if ctx.emit_mx_grad and mx.can_emit(T, dqkv.shape[1]) and dqkv.is_contiguous():
                # the fp8 copy of the whole gradient row (q, k and the v slice the attention backward wrote)
                # for the dgrad of an MXFP8 qkv projection
                q8, sf = mx.alloc_quantized(T, dqkv.shape[1], qkv.device)
            rc = L.kwu_qknorm_rope_bwd_qk(native.ptr(qkv), ci(ld), native.ptr(dq), native.ptr(dk), native.ptr(dqkv),
                                          ci(dld), native.ptr(q_norm), native.ptr(k_norm), native.ptr(targets[0][1]),
                                          native.ptr(targets[1][1]), native.ptr(cos), native.ptr(sin), ci(T), ci(Hq),
                                          ci(Hkv), ci(rot_half), cf(eps), ci(int(do_norm)), native.ptr(q8),
                                          ci(dqkv.shape[1]), native.ptr(sf), native.stream_ptr())
            native.check(rc, "qknorm_rope_bwd_qk")
            if q8 is not None:
                mx.stash_quantized(dqkv, q8, sf)
        else:
            for (src, g, dst, H), (w, dw, _) in zip(((qkv[:, : Hq * D], dq, dqkv[:, : Hq * D], Hq),
                                                     (qkv[:, Hq * D:(Hq + Hkv) * D], dk, dqkv[:, Hq * D:(Hq + Hkv) * D], Hkv)),
                                                    targets):
                rc = L.kwu_qknorm_rope_bwd(native.ptr(src), ci(ld), native.ptr(g), ci(H * D), native.ptr(dst), ci(dld),
                                           native.ptr(w), native.ptr(dw), native.ptr(cos), native.ptr(sin), ci(T),
                                           ci(H), ci(D), ci(rot_half), cf(eps), ci(int(do_norm)), native.stream_ptr())
                native.check(rc, "qknorm_rope_bwd")
        dws = [None if into_main else dw for _, dw, into_main in targets]
        dsink = None
        if sink_lse is not None and ctx.needs_input_grad[7]:
            dsink = -(torch.exp(sink_lse.float()[:, None] - lse) * delta).sum(1).to(sink_lse.dtype)
        return (dqkv, dws[0], dws[1], None, None, None, None, dsink, None, None, None, None, None, None, None, None)


def attention_core_supported(qkv, head_dim, q_norm, k_norm, cos) -> bool:
    return (native.available() and qkv.is_cuda and qkv.dtype == torch.bfloat16 and head_dim == 64
            and qkv.stride(1) == 1 and (q_norm is None or q_norm.dtype == torch.float32)
            and (cos is None or (cos.dtype == torch.float32 and cos.shape[-1] in (8, 16, 32))))


def attention_core(qkv, q_norm, k_norm, cos, sin, cu_seqlens, plan, sink_lse, Hq, Hkv, window, scale, eps,
                   do_norm, emit_mx_grad=False, emit_mx_out=False):
    """``emit_mx_grad``: the backward also writes the MXFP8 copy of ``d(qkv)`` for an MXFP8 projection's dgrad.
    ``emit_mx_out``: the forward also writes the MXFP8 copy of the output for an MXFP8 output projection."""
    if plan is None:
        plan = attention_plan(cu_seqlens, qkv.shape[0])
    if sink_lse is not None:
        sink_lse = sink_lse.float()
    return _AttentionCore.apply(qkv, q_norm, k_norm, cos, sin, cu_seqlens, plan, sink_lse, Hq, Hkv, window,
                                float(scale), float(eps), bool(do_norm), bool(emit_mx_grad), bool(emit_mx_out))


# ------------------------------------------------------------------------------------ decode
def decode_supported(q, k_cache) -> bool:
    return (native.available() and q.is_cuda and q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
            and q.shape[-1] == 64 and q.shape[-2] % k_cache.shape[-2] == 0 and q.shape[-2] // k_cache.shape[-2] <= 8)


_decode_scratch: dict = {}


@torch.no_grad()
def decode_attention(q, k_cache, v_cache, kv_len: int, window: int | None = None, scale: float | None = None,
                     sink: torch.Tensor | None = None, return_lse: bool = False):
    """One new token per row against a KV cache: q (B,H,64); caches (B,L_max,Hkv,64); the query sits at
    position ``kv_len - 1`` and attends keys ``[max(0, kv_len - window), kv_len)``. ``sink`` (H,S) fp32 learned
    sink logits join the softmax denominator. Split-KV kernel in ``csrc/decode_attn.cu``."""
    L = native.require()
    B, H, D = q.shape
    Hkv = k_cache.shape[2]
    scale = scale if scale is not None else D ** -0.5
    out = torch.empty(B, H, D, dtype=q.dtype, device=q.device)
    lse = torch.empty(B, H, dtype=torch.float32, device=q.device)
    need = int(L.kwu_decode_scratch_floats(ctypes.c_int(B), ctypes.c_int(H), ctypes.c_int(k_cache.shape[1])))
    key = (q.device, need)
    scratch = _decode_scratch.get(key)
    if scratch is None:
        scratch = _decode_scratch[key] = torch.empty(need, dtype=torch.float32, device=q.device)
    sink_f = sink.detach().float().contiguous() if sink is not None else None
    ll = ctypes.c_longlong
    rc = L.kwu_decode_attention(
        native.ptr(q), ll(q.stride(0)), ll(q.stride(1)),
        native.ptr(k_cache), ll(k_cache.stride(0)), ll(k_cache.stride(1)), ll(k_cache.stride(2)),
        native.ptr(v_cache), ll(v_cache.stride(0)), ll(v_cache.stride(1)), ll(v_cache.stride(2)),
        native.ptr(out), ll(out.stride(0)), ll(out.stride(1)), native.ptr(lse), native.ptr(scratch),
        ctypes.c_int(B), ctypes.c_int(H), ctypes.c_int(Hkv), ctypes.c_int(int(kv_len)), ctypes.c_int(int(window or 0)),
        ctypes.c_float(scale), native.ptr(sink_f), ctypes.c_int(0 if sink_f is None else sink_f.shape[1]),
        native.stream_ptr())
    native.check(rc, "decode_attention")
    return (out, lse) if return_lse else out


# ------------------------------------------------------------------------------------ MXFP8 operands
def quantize_heads_reference(x: torch.Tensor, smooth: bool = False) -> torch.Tensor:
    """(T,H,64) -> the values an MXFP8 (e4m3, one UE8M0 scale per 32 channels) copy of x holds, as x.dtype.
    ``smooth`` subtracts the per-(head, channel) mean over the T tokens first."""
    from kohakuwullm_b200.ops.mxfp8 import dequantize, quantize_reference

    T, H, D = x.shape
    xf = x.float()
    if smooth:
        xf = xf - xf.mean(0, keepdim=True)
    q, e = quantize_reference(xf.reshape(T * H, D))
    return dequantize(q, e).view(T, H, D).to(x.dtype)


class _QuantizeHeads(torch.autograd.Function):
    """Per-head MXFP8 quantisation of an attention operand, returned as the exactly representable bf16
    values (``csrc/mxfp8.cu``: ``mxfp8_quant_heads``). Backward is straight-through; with ``smooth`` the
    gradient's own token mean is removed, as the mean subtraction requires."""

    @staticmethod
    def forward(ctx, x, smooth):
        L = native.require()
        T, H, D = x.shape
        if x.stride(2) != 1 or x.stride(1) != D:
            x = x.contiguous()
        mu = None
        if smooth:
            mu = torch.empty(H, D, dtype=torch.float32, device=x.device)
            rc = L.kwu_mxfp8_column_mean(native.ptr(x), ctypes.c_longlong(x.stride(0)), ctypes.c_int(T), ctypes.c_int(H),
                                         native.ptr(mu), native.stream_ptr())
            native.check(rc, "mxfp8_column_mean")
        out = torch.empty(T, H, D, dtype=x.dtype, device=x.device)
        rc = L.kwu_mxfp8_quant_heads(native.ptr(x), ctypes.c_longlong(x.stride(0)), native.ptr(mu), native.ptr(None),
                                     native.ptr(None), native.ptr(out), ctypes.c_int(T), ctypes.c_int(H),
                                     native.stream_ptr())
        native.check(rc, "mxfp8_quant_heads")
        ctx.smooth = smooth
        return out

    @staticmethod
    def backward(ctx, dy):
        if not ctx.smooth:
            return dy, None
        L = native.require()
        dy = dy.contiguous()
        T, H, D = dy.shape
        mu = torch.empty(H, D, dtype=torch.float32, device=dy.device)
        rc = L.kwu_mxfp8_column_mean(native.ptr(dy), ctypes.c_longlong(dy.stride(0)), ctypes.c_int(T), ctypes.c_int(H),
                                     native.ptr(mu), native.stream_ptr())
        native.check(rc, "mxfp8_column_mean")
        return (dy.float() - mu[None]).to(dy.dtype), None


def quantize_heads(x: torch.Tensor, smooth: bool = False) -> torch.Tensor:
    """MXFP8 round trip of a (T,H,64) attention operand (native on bf16 CUDA input, PyTorch elsewhere).
    Gradients pass straight through the rounding; with ``smooth`` they flow through the mean subtraction."""
    if native.available() and x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] == 64:
        return _QuantizeHeads.apply(x, smooth)
    base = x - x.float().mean(0, keepdim=True).to(x.dtype) if smooth else x
    return base + (quantize_heads_reference(x, smooth) - base).detach()
