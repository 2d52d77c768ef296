"""RMSNorm, SwiGLU and the fused per-head QK-norm + rotary embedding.

Each op has two implementations with identical semantics:

* ``*_reference`` — plain PyTorch in fp32, runs anywhere, and is the oracle of the GPU tests;
* the native sm_100a kernel (``csrc/elementwise.cu``), used for bf16 CUDA tensors.

Counterparts in the reference: src/kohakuwullm/kernels/elementwise/rmsnorm.py:20-128,
swiglu.py:49-119, src/kohakuwullm/kernels/attention/rope.py:27-89.
"""

from __future__ import annotations

import ctypes

import torch

from kohakuwullm_b200.ops import native

c_int, c_float = ctypes.c_int, ctypes.c_float


def _native_ok(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16


# ----------------------------------------------------------------------------- RMSNorm
def rmsnorm_reference(x, weight=None, eps=1e-6, one_plus=False, residual=None):
    h = x if residual is None else (x.float() + residual.float()).to(x.dtype)
    hf = h.float()
    y = hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps)
    if weight is not None:
        y = y * ((1.0 + weight.float()) if one_plus else weight.float())
    y = y.to(x.dtype)
    return y if residual is None else (y, h)


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, residual, eps, one_plus, emit_mx=False, emit_mx_grad=False):
        L = native.require()
        cols = x.shape[-1]
        x2 = x.reshape(-1, cols)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        h = None
        r2 = None
        if residual is not None:
            r2 = residual.reshape(-1, cols)
            if not r2.is_contiguous():
                r2 = r2.contiguous()
            h = torch.empty_like(x2)
        from kohakuwullm_b200.ops import mxfp8 as mx

        if emit_mx and mx.can_emit(rows, cols):
            q, sf = mx.alloc_quantized(rows, cols, x.device)
            rc = L.kwu_rmsnorm_fwd_mx(
                native.ptr(x2), native.ptr(r2), native.ptr(weight), native.ptr(y), native.ptr(h),
                native.ptr(rstd), c_int(rows), c_int(cols), c_float(eps), c_int(int(one_plus)),
                native.ptr(q), c_int(cols), native.ptr(sf), native.stream_ptr())
            mx.stash_quantized(y, q, sf)
        else:
            rc = L.kwu_rmsnorm_fwd(
                native.ptr(x2), native.ptr(r2), native.ptr(weight), native.ptr(y), native.ptr(h),
                native.ptr(rstd), c_int(rows), c_int(cols), c_float(eps), c_int(int(one_plus)),
                native.stream_ptr(),
            )
        native.check(rc, "rmsnorm_fwd")
        ctx.emit_mx_grad = emit_mx_grad
        ctx.weight_param = weight   # the Parameter object: its ``main_grad`` takes the weight gradient directly
        ctx.save_for_backward(h if h is not None else x2, weight, rstd)
        ctx.one_plus = one_plus
        ctx.has_res = residual is not None
        ctx.shape = x.shape
        if residual is not None:
            return y.view(x.shape), h.view(x.shape)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy, dh=None):
        L = native.require()
        xin, weight, rstd = ctx.saved_tensors
        rows, cols = xin.shape
        dy2 = dy.reshape(rows, cols)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dres = None
        if ctx.has_res and dh is not None:
            dres = dh.reshape(rows, cols)
            if not dres.is_contiguous():
                dres = dres.contiguous()
        dx = torch.empty_like(xin)
        dw = partial = None
        acc = 0
        main_grad = getattr(ctx.weight_param, "main_grad", None)
        if weight is not None and ctx.needs_input_grad[1]:
            nblocks = L.kwu_rmsnorm_bwd_blocks(c_int(rows))
            partial = torch.empty(nblocks, cols, dtype=torch.float32, device=xin.device)
            if main_grad is not None and main_grad.dtype == torch.float32 and main_grad.is_contiguous():
                dw, acc = main_grad, 1      # summed straight into the trainer's fp32 gradient buffer
            else:
                dw = torch.empty(cols, dtype=torch.float32, device=xin.device)
        from kohakuwullm_b200.ops import mxfp8 as mx

        if ctx.emit_mx_grad and mx.can_emit(rows, cols) and cols <= 2048:
            q, sf = mx.alloc_quantized(rows, cols, xin.device)
            rc = L.kwu_rmsnorm_bwd_mx(
                native.ptr(xin), native.ptr(weight), native.ptr(rstd), native.ptr(dy2), native.ptr(dres),
                native.ptr(dx), native.ptr(dw), native.ptr(partial), c_int(rows), c_int(cols),
                c_int(int(ctx.one_plus)), c_int(acc), native.ptr(q), c_int(cols), native.ptr(sf), native.stream_ptr())
            mx.stash_quantized(dx, q, sf)
        else:
            rc = L.kwu_rmsnorm_bwd(
                native.ptr(xin), native.ptr(weight), native.ptr(rstd), native.ptr(dy2), native.ptr(dres),
                native.ptr(dx), native.ptr(dw), native.ptr(partial), c_int(rows), c_int(cols),
                c_int(int(ctx.one_plus)), c_int(acc), native.stream_ptr(),
            )
        native.check(rc, "rmsnorm_bwd")
        dxv = dx.view(ctx.shape)
        if acc:
            dw = None
        elif dw is not None:
            dw = dw.to(weight.dtype)
        return dxv, dw, (dxv if ctx.has_res else None), None, None, None, None


def rmsnorm(x, weight=None, eps=1e-6, one_plus=False, residual=None, emit_mx=False, emit_mx_grad=False):
    """RMSNorm over the last dimension.

    With ``residual`` the sum ``h = x + residual`` is formed inside the kernel and the call
    returns ``(norm(h), h)``: the residual add and the pre-norm of a decoder block in one pass.
    """
    if _native_ok(x) and x.shape[-1] % 8 == 0 and (weight is None or weight.dtype == torch.float32):
        return _RMSNorm.apply(x, weight, residual, eps, one_plus, emit_mx, emit_mx_grad)
    return rmsnorm_reference(x, weight, eps, one_plus, residual)


# ----------------------------------------------------------------------------- SwiGLU
def swiglu_reference(h):
    g, v = h.float().chunk(2, dim=-1)
    return (torch.nn.functional.silu(g) * v).to(h.dtype)


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, emit_mx=False, emit_mx_grad=False):
        L = native.require()
        H2 = h.shape[-1]
        h2 = h.reshape(-1, H2)
        if h2.stride(1) != 1:
            h2 = h2.contiguous()
        rows, H = h2.shape[0], H2 // 2
        out = torch.empty(rows, H, dtype=h.dtype, device=h.device)
        from kohakuwullm_b200.ops import mxfp8 as mx

        if emit_mx and mx.can_emit(rows, H):
            q, sf = mx.alloc_quantized(rows, H, h.device)
            rc = L.kwu_swiglu_fwd_mx(native.ptr(h2), c_int(h2.stride(0)), native.ptr(out), c_int(H),
                                     c_int(rows), c_int(H), native.ptr(q), c_int(H), native.ptr(sf), native.stream_ptr())
            mx.stash_quantized(out, q, sf)
        else:
            rc = L.kwu_swiglu_fwd(native.ptr(h2), c_int(h2.stride(0)), native.ptr(out), c_int(H),
                                  c_int(rows), c_int(H), native.stream_ptr())
        native.check(rc, "swiglu_fwd")
        ctx.emit_mx_grad = emit_mx_grad
        ctx.save_for_backward(h2)
        ctx.shape = h.shape
        return out.view(*h.shape[:-1], H)

    @staticmethod
    def backward(ctx, dout):
        L = native.require()
        (h2,) = ctx.saved_tensors
        rows, H2 = h2.shape
        H = H2 // 2
        d2 = dout.reshape(rows, H)
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        din = torch.empty(rows, H2, dtype=h2.dtype, device=h2.device)
        from kohakuwullm_b200.ops import mxfp8 as mx

        if ctx.emit_mx_grad and mx.can_emit(rows, H2) and H % 32 == 0:
            q, sf = mx.alloc_quantized(rows, H2, h2.device)
            rc = L.kwu_swiglu_bwd_mx(native.ptr(h2), c_int(h2.stride(0)), native.ptr(d2), c_int(H),
                                     native.ptr(din), c_int(H2), c_int(rows), c_int(H), native.ptr(q), c_int(H2),
                                     native.ptr(sf), native.stream_ptr())
            mx.stash_quantized(din, q, sf)
        else:
            rc = L.kwu_swiglu_bwd(native.ptr(h2), c_int(h2.stride(0)), native.ptr(d2), c_int(H),
                                  native.ptr(din), c_int(H2), c_int(rows), c_int(H), native.stream_ptr())
        native.check(rc, "swiglu_bwd")
        return din.view(ctx.shape), None, None


def swiglu(h, emit_mx=False, emit_mx_grad=False):
    """``silu(h[..., :H]) * h[..., H:]`` for a fused gate|value projection output. ``emit_mx`` /
    ``emit_mx_grad``: also write the MXFP8 copy of the output / of the input gradient for the MXFP8 linear
    that consumes it (see ``ops.mxfp8.stash_quantized``)."""
    if _native_ok(h) and (h.shape[-1] // 2) % 8 == 0:
        return _SwiGLU.apply(h, emit_mx, emit_mx_grad)
    return swiglu_reference(h)


# ----------------------------------------------------------------------------- QK-norm + RoPE
def rotate_half_reference(x, cos, sin):
    """x (T,H,D); cos/sin (T, rot/2) fp32. Rotates the first ``rot`` channels, rotate-half style."""
    rot_half = cos.shape[-1]
    xf = x.float()
    a, b, tail = xf[..., :rot_half], xf[..., rot_half:2 * rot_half], xf[..., 2 * rot_half:]
    c, s = cos[:, None, :].float(), sin[:, None, :].float()
    return torch.cat([a * c - b * s, b * c + a * s, tail], dim=-1).to(x.dtype)


def qknorm_rope_reference(x, weight, cos, sin, eps=1e-6, do_norm=True):
    """x (T,H,D) -> rope(rmsnorm_over_D(x)); the normalised value is rounded to x.dtype first."""
    if do_norm:
        xf = x.float()
        xn = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
        if weight is not None:
            xn = xn * weight.float()
        x = xn.to(x.dtype)
    if cos is None:
        return x
    return rotate_half_reference(x, cos, sin)


class _QKNormRope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, cos, sin, eps, do_norm):
        # x: (T, H, 64) view with unit stride on the last dim and heads contiguous (stride 64)
        L = native.require()
        T, H, D = x.shape
        out = torch.empty(T, H, D, dtype=x.dtype, device=x.device)
        rot_half = 0 if cos is None else cos.shape[-1]
        rc = L.kwu_qknorm_rope_fwd(
            native.ptr(x), c_int(x.stride(0)), native.ptr(out), c_int(H * D), native.ptr(weight),
            native.ptr(cos), native.ptr(sin), c_int(T), c_int(H), c_int(D), c_int(rot_half),
            c_float(eps), c_int(int(do_norm)), native.stream_ptr(),
        )
        native.check(rc, "qknorm_rope_fwd")
        ctx.save_for_backward(x, weight, cos, sin)
        ctx.eps, ctx.do_norm = eps, do_norm
        ctx.weight_param = weight
        return out

    @staticmethod
    def backward(ctx, dout):
        L = native.require()
        x, weight, cos, sin = ctx.saved_tensors
        T, H, D = x.shape
        if dout.stride(2) != 1 or dout.stride(1) != D:
            dout = dout.contiguous()
        dx = torch.empty(T, H, D, dtype=x.dtype, device=x.device)
        dw = None
        main_grad = getattr(ctx.weight_param, "main_grad", None)
        into_main = main_grad is not None and main_grad.dtype == torch.float32 and main_grad.is_contiguous()
        if weight is not None and ctx.needs_input_grad[1]:
            # the kernel accumulates with atomics, so the trainer's fp32 buffer can take the sum directly
            dw = main_grad if into_main else torch.zeros(D, dtype=torch.float32, device=x.device)
        rot_half = 0 if cos is None else cos.shape[-1]
        rc = L.kwu_qknorm_rope_bwd(
            native.ptr(x), c_int(x.stride(0)), native.ptr(dout), c_int(dout.stride(0)), native.ptr(dx),
            c_int(H * D), native.ptr(weight), native.ptr(dw), native.ptr(cos), native.ptr(sin),
            c_int(T), c_int(H), c_int(D), c_int(rot_half), c_float(ctx.eps), c_int(int(ctx.do_norm)),
            native.stream_ptr(),
        )
        native.check(rc, "qknorm_rope_bwd")
        if dw is not None:
            dw = None if into_main else dw.to(weight.dtype)
        return dx, dw, None, None, None, None


def qknorm_rope(x, weight, cos, sin, eps=1e-6, do_norm=True):
    """Per-head RMSNorm over ``head_dim`` followed by rotary embedding, in one kernel.

    ``x`` is (T, H, D), typically a strided view into the fused qkv projection output; ``cos`` /
    ``sin`` are per-token (T, rot/2) fp32 tables (``None`` disables the rotation).
    """
    ok = (
        _native_ok(x) and x.dim() == 3 and x.shape[-1] == 64 and x.stride(2) == 1 and x.stride(1) == 64
        and (weight is None or weight.dtype == torch.float32)
        and (cos is None or (cos.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous()
                             and cos.shape[-1] in (8, 16, 32)))
    )
    if ok:
        return _QKNormRope.apply(x, weight, cos, sin, eps, do_norm)
    return qknorm_rope_reference(x, weight, cos, sin, eps, do_norm)


# ----------------------------------------------------------------------------- embedding
class _Embedding(torch.autograd.Function):
    """Row gather with an optional scale; the backward adds the token gradients straight into the weight's
    fp32 ``main_grad`` (vector reductions), or into a fresh fp32 buffer when there is none."""

    @staticmethod
    def forward(ctx, tokens, weight, scale):
        L = native.require()
        flat = tokens.reshape(-1).contiguous()
        V, D = weight.shape
        out = torch.empty(flat.numel(), D, dtype=weight.dtype, device=weight.device)
        rc = L.kwu_embedding_fwd(native.ptr(flat), native.ptr(weight), native.ptr(out), c_int(flat.numel()), c_int(D),
                                 c_int(V), c_float(scale), native.stream_ptr())
        native.check(rc, "embedding_fwd")
        ctx.save_for_backward(flat)
        ctx.weight_param, ctx.scale, ctx.shape = weight, scale, (V, D)
        return out.view(*tokens.shape, D)

    @staticmethod
    def backward(ctx, dout):
        L = native.require()
        (flat,) = ctx.saved_tensors
        V, D = ctx.shape
        w = ctx.weight_param
        main_grad = getattr(w, "main_grad", None)
        use_main = main_grad is not None and main_grad.dtype == torch.float32 and main_grad.is_contiguous()
        target = main_grad if use_main else torch.zeros(V, D, dtype=torch.float32, device=dout.device)
        d2 = dout.reshape(-1, D).contiguous()
        rc = L.kwu_embedding_bwd(native.ptr(flat), native.ptr(d2), native.ptr(target), c_int(flat.numel()), c_int(D),
                                 c_int(V), c_float(ctx.scale), native.stream_ptr())
        native.check(rc, "embedding_bwd")
        return None, (None if use_main else target.to(w.dtype)), None


def embedding(tokens: torch.Tensor, weight: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """``weight[tokens] * scale``; native gather / scatter-add on bf16 CUDA weights, PyTorch elsewhere."""
    if native.available() and weight.is_cuda and weight.dtype == torch.bfloat16 and weight.shape[1] % 8 == 0 \
            and tokens.dtype == torch.long:
        return _Embedding.apply(tokens, weight, float(scale))
    x = torch.nn.functional.embedding(tokens, weight)
    return x * scale if scale != 1.0 else x
