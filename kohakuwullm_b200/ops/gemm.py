"""bf16 matrix products on the tcgen05 GEMM kernel, and the ``linear`` autograd function.

``matmul(a, b, a_mn, b_mn)`` computes ``C[M,N] (+)= alpha * op(A) op(B)`` where each operand is
either K-major (contraction index contiguous) or MN-major (output index contiguous). The three
products of a linear layer map onto it without any transpose pass:

====================  =======================  ====================
product               A                        B
====================  =======================  ====================
``y = x @ W.T``       ``x`` (T,K)  K-major     ``W`` (N,K) K-major
``dx = dy @ W``       ``dy`` (T,N) K-major     ``W`` (N,K) MN-major
``dW = dy.T @ x``     ``dy`` (T,N) MN-major    ``x`` (T,K) MN-major
====================  =======================  ====================

On CPU (and for dtypes other than bf16) the same functions run plain ``torch.matmul`` so the
whole framework can be exercised without a GPU; that path is also the numerical oracle of the
GPU tests. Replaces the cuBLAS calls behind ``nn.Linear`` in the reference
(src/kohakuwullm/models/components/attention.py:77-89).
"""

from __future__ import annotations

import ctypes
import os

import torch

from kohakuwullm_b200.ops import native


# ------------------------------------------------------------------------------------ weight-gradient overlap
# In the backward pass the chain of activation gradients (dgrad GEMM -> elementwise backward -> attention
# backward -> ...) is the critical path; a layer's weight gradient only has to be finished before the optimizer
# reads ``main_grad``. With the overlap switched on, every weight-gradient product that accumulates into
# ``main_grad`` is launched on a side stream right behind the point where its operands exist, and runs in the
# shadow of the kernels that follow on the main stream: it fills the SMs a latency-bound attention backward, a
# memory-bound norm kernel or the last partial wave of a GEMM leave idle. The caller (the training engine)
# switches it on around a backward pass and joins the side stream afterwards; under CUDA-graph capture the
# fork and the join are captured as parallel branches of the graph.
_wgrad_overlap = {"on": False, "streams": {}, "dirty": False}


def set_wgrad_overlap(on: bool) -> None:
    _wgrad_overlap["on"] = bool(on)


def wgrad_overlap_enabled() -> bool:
    return _wgrad_overlap["on"]


def launch_wgrad(fn, *operands: torch.Tensor) -> None:
    """Run ``fn()`` (a weight-gradient product reading ``operands``) on the side stream when the overlap is on,
    else inline. The operands are marked as used by the side stream so that the caching allocator does not
    hand their memory out again before the product has read it."""
    if not _wgrad_overlap["on"] or not operands or not operands[0].is_cuda:
        fn()
        return
    dev = operands[0].device.index
    side = _wgrad_overlap["streams"].get(dev)
    if side is None:
        side = _wgrad_overlap["streams"][dev] = torch.cuda.Stream(device=operands[0].device)
    main = torch.cuda.current_stream(operands[0].device)
    side.wait_stream(main)
    with torch.cuda.stream(side):
        fn()
    for t in operands:
        t.record_stream(side)
    _wgrad_overlap["dirty"] = True


def join_wgrad() -> None:
    """Make the current stream wait for every weight-gradient product launched on a side stream."""
    if not _wgrad_overlap["dirty"]:
        return
    for dev, side in _wgrad_overlap["streams"].items():
        torch.cuda.current_stream(torch.device("cuda", dev)).wait_stream(side)
    _wgrad_overlap["dirty"] = False


def _use_native(*tensors: torch.Tensor) -> bool:
    return all(t.is_cuda and t.dtype == torch.bfloat16 for t in tensors)


def matmul(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    a_mn: bool = False,
    b_mn: bool = False,
    out: torch.Tensor | None = None,
    accumulate: bool = False,
    alpha: float = 1.0,
    out_dtype: torch.dtype | None = None,
    bn: int = 0,
    max_ctas: int = 0,
) -> torch.Tensor:
    """``out (+)= alpha * op(a) @ op(b)``.

    ``a`` is stored (M,K) when ``a_mn`` is false, (K,M) when true; ``b`` is stored (N,K) when
    ``b_mn`` is false, (K,N) when true. Both must be 2-D with unit inner stride.
    """
    if a_mn:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_mn:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    if K != Kb:
        raise ValueError(f"contraction mismatch: {tuple(a.shape)} (a_mn={a_mn}) vs {tuple(b.shape)} (b_mn={b_mn})")
    if out is None:
        if accumulate:
            raise ValueError("accumulate=True needs an output tensor")
        out = torch.empty(M, N, dtype=out_dtype or a.dtype, device=a.device)
    if out.shape != (M, N) or out.stride(1) != 1:
        raise ValueError(f"output must be ({M},{N}) with unit inner stride, got {tuple(out.shape)}")

    if not _use_native(a, b) or out.dtype not in (torch.bfloat16, torch.float32) or M == 0:
        am = a.t() if a_mn else a
        bm = b if b_mn else b.t()
        prod = torch.matmul(am.float(), bm.float()) * alpha
        if accumulate:
            out.add_(prod.to(out.dtype))
        else:
            out.copy_(prod.to(out.dtype))
        return out

    if a.stride(1) != 1 or b.stride(1) != 1:
        raise ValueError("native matmul needs unit inner strides")
    L = native.require()
    rc = L.kwu_gemm_bf16(
        native.ptr(a), native.ptr(b), native.ptr(out),
        ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K),
        ctypes.c_int(a.stride(0)), ctypes.c_int(b.stride(0)), ctypes.c_int(out.stride(0)),
        ctypes.c_int(int(a_mn)), ctypes.c_int(int(b_mn)),
        ctypes.c_int(int(out.dtype == torch.float32)), ctypes.c_int(int(accumulate)),
        ctypes.c_float(alpha), ctypes.c_int(bn), ctypes.c_int(max_ctas),
        native.stream_ptr(), native.ptr(native.status_word()),
    )
    native.check(rc, "gemm_bf16")
    return out


class _Linear(torch.autograd.Function):
    """``y = x @ W.T`` for 2-D ``x``; gradients through :func:`matmul`.

    When the weight carries a ``main_grad`` attribute (an fp32 tensor of the weight's shape owned
    by the trainer) the weight gradient is accumulated straight into it by the GEMM epilogue and
    autograd receives no weight gradient, which removes one write+read of every weight gradient
    per micro-batch.
    """

    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        return matmul(x, w)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = matmul(dy, w, b_mn=True)
        if ctx.needs_input_grad[1]:
            main_grad = getattr(w, "main_grad", None)
            if main_grad is not None:
                launch_wgrad(lambda: matmul(dy, x, a_mn=True, b_mn=True, out=main_grad, accumulate=True), dy, x)
                w.grad_in_main = True
            else:
                dw = matmul(dy, x, a_mn=True, b_mn=True, out_dtype=w.dtype)
        return dx, dw


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """Linear layer over the last dimension (any leading shape)."""
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if _use_native(x2, w):
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        y = _Linear.apply(x2, w)
    else:
        y = torch.nn.functional.linear(x2, w.to(x2.dtype))
    if bias is not None:
        y = y + bias.to(y.dtype)
    return y.reshape(*lead, w.shape[0])
