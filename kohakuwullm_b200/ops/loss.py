"""Linear + cross-entropy (+ z-loss) without ever writing the logits to memory.

``linear_cross_entropy(h, W, labels)`` returns per-token ``(ce, lse)`` in fp32, both
differentiable: ``ce[t] = lse[t] - logit[t, labels[t]]`` (zero on ignored rows) and
``lse[t] = logsumexp_v(h[t] . W[v])``. A z-loss is ``z_w * lse**2`` on top of the same pass, so
the second vocabulary GEMM that the reference pays for it (src/kohakuwullm/kernels/loss/zloss.py:21-70)
disappears.

Native path (bf16, CUDA):
  forward   one tcgen05 GEMM whose epilogue keeps, per row and 256-column tile, a running
            (max, sum-exp) and picks out the target logit; a tiny kernel folds the partials.
  backward  the same GEMM is re-run with an epilogue that turns the accumulator into
            ``dlogits = (g_ce + g_lse) * softmax - g_ce * onehot`` (bf16, in a reused scratch
            buffer, processed in row chunks), followed by the two products ``dh = dlogits W`` and
            ``dW += dlogits^T h``.
Everything else (CPU, fp32, fp16) runs the chunked PyTorch reference below, which is also the
test oracle. Reference implementation: src/kohakuwullm/kernels/loss/chunked_ce.py:94-293.
"""

from __future__ import annotations

import ctypes

import torch

from kohakuwullm_b200.ops import native
from kohakuwullm_b200.ops.gemm import launch_wgrad, matmul

c_int, c_float = ctypes.c_int, ctypes.c_float

IGNORE_INDEX = -100
_scratch: dict[tuple, torch.Tensor] = {}


def _scratch_buffer(key: str, shape: tuple[int, ...], dtype, device) -> torch.Tensor:
    """Reused scratch, grown on demand (one per device and purpose).

    While a CUDA graph is being captured the buffer is NOT taken from the shared cache: a graph replays with
    the addresses it was captured with, and the cached buffer is replaced when a larger request arrives
    later, which would leave the graph writing into freed memory. An allocation made during capture comes
    from the graph's private pool and lives as long as the graph does."""
    n = 1
    for s in shape:
        n *= s
    if torch.device(device).type == "cuda" and torch.cuda.is_current_stream_capturing():
        return torch.empty(n, dtype=dtype, device=device).view(*shape)
    k = (key, str(device), dtype)
    buf = _scratch.get(k)
    if buf is None or buf.numel() < n:
        buf = torch.empty(n, dtype=dtype, device=device)
        _scratch[k] = buf
    return buf[:n].view(*shape)


class _ChunkedReference(torch.autograd.Function):
    """Row-chunked fp32 evaluation; memory is O(chunk * vocab)."""

    @staticmethod
    def forward(ctx, h, w, labels, chunk, soft_cap):
        T = h.shape[0]
        ce = torch.zeros(T, dtype=torch.float32, device=h.device)
        lse = torch.empty(T, dtype=torch.float32, device=h.device)
        wf = w.float()
        for s in range(0, T, chunk):
            e = min(T, s + chunk)
            logits = h[s:e].float() @ wf.t()
            if soft_cap:
                logits = soft_cap * torch.tanh(logits / soft_cap)
            l = torch.logsumexp(logits, dim=-1)
            lse[s:e] = l
            lab = labels[s:e]
            valid = lab >= 0
            tgt = logits.gather(1, lab.clamp(min=0)[:, None]).squeeze(1)
            ce[s:e] = torch.where(valid, l - tgt, torch.zeros_like(l))
        ctx.save_for_backward(h, w, labels, lse)
        ctx.chunk, ctx.soft_cap = chunk, soft_cap
        return ce, lse

    @staticmethod
    def backward(ctx, g_ce, g_lse):
        h, w, labels, lse = ctx.saved_tensors
        T = h.shape[0]
        wf = w.float()
        dh = torch.empty_like(h, dtype=torch.float32)
        dw = torch.zeros_like(wf)
        for s in range(0, T, ctx.chunk):
            e = min(T, s + ctx.chunk)
            hf = h[s:e].float()
            raw = hf @ wf.t()
            logits = ctx.soft_cap * torch.tanh(raw / ctx.soft_cap) if ctx.soft_cap else raw
            p = torch.exp(logits - lse[s:e, None])
            lab = labels[s:e]
            valid = (lab >= 0).float()
            gce = g_ce[s:e].float() * valid
            d = p * (gce + g_lse[s:e].float())[:, None]
            d.scatter_add_(1, lab.clamp(min=0)[:, None], -gce[:, None])
            if ctx.soft_cap:
                d = d * (1.0 - (logits / ctx.soft_cap) ** 2)
            dh[s:e] = d @ wf
            dw += d.t() @ hf
        return dh.to(h.dtype), dw.to(w.dtype), None, None, None


class _FusedLinearCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, w, labels32, chunk):
        L = native.require()
        T, D = h.shape
        V = w.shape[0]
        tiles_n = L.kwu_ce_tiles_n(c_int(V))
        partial = _scratch_buffer("ce_partial", (tiles_n, T, 2), torch.float32, h.device)
        tgt = torch.zeros(T, dtype=torch.float32, device=h.device)
        lse = torch.empty(T, dtype=torch.float32, device=h.device)
        rc = L.kwu_gemm_lse(native.ptr(h), native.ptr(w), c_int(T), c_int(V), c_int(D),
                            c_int(h.stride(0)), c_int(w.stride(0)), native.ptr(labels32),
                            native.ptr(partial), native.ptr(tgt), c_float(1.0), native.stream_ptr(),
                            native.ptr(native.status_word()))
        native.check(rc, "gemm_lse")
        rc = L.kwu_ce_combine(native.ptr(partial), c_int(tiles_n), c_int(T), native.ptr(lse),
                              native.stream_ptr())
        native.check(rc, "ce_combine")
        ce = torch.where(labels32 >= 0, lse - tgt, torch.zeros_like(lse))
        ctx.save_for_backward(h, w, labels32, lse)
        ctx.chunk = chunk
        return ce, lse

    @staticmethod
    def backward(ctx, g_ce, g_lse):
        L = native.require()
        h, w, labels32, lse = ctx.saved_tensors
        T, D = h.shape
        V = w.shape[0]
        valid = (labels32 >= 0).float()
        coef_y = (g_ce.float() * valid).contiguous()
        coef_p = (coef_y + g_lse.float()).contiguous()
        dh = torch.empty_like(h)
        main_grad = getattr(w, "main_grad", None)
        dw = None
        if main_grad is None and ctx.needs_input_grad[1]:
            dw = torch.zeros(V, D, dtype=torch.float32, device=h.device)
        chunk = ctx.chunk
        for s in range(0, T, chunk):
            e = min(T, s + chunk)
            n = e - s
            dl = _scratch_buffer("ce_dlogits", (n, V), torch.bfloat16, h.device)
            rc = L.kwu_gemm_dlogits(native.ptr(h[s:e]), native.ptr(w), native.ptr(dl), c_int(n), c_int(V),
                                    c_int(D), c_int(h.stride(0)), c_int(w.stride(0)), c_int(V),
                                    native.ptr(labels32[s:e]), native.ptr(lse[s:e]), native.ptr(coef_p[s:e]),
                                    native.ptr(coef_y[s:e]), c_float(1.0), native.stream_ptr(),
                                    native.ptr(native.status_word()))
            native.check(rc, "gemm_dlogits")
            if ctx.needs_input_grad[0]:
                # contraction over the whole vocabulary with few output tiles: accumulate in fp32 so the
                # (tile, k-block) units can be dealt out evenly over the SMs, then round once
                dh32 = _scratch_buffer("ce_dh32", (n, D), torch.float32, h.device)
                dh32.zero_()
                matmul(dl, w, b_mn=True, out=dh32, accumulate=True)
                dh[s:e].copy_(dh32)
            if ctx.needs_input_grad[1]:
                target = main_grad if main_grad is not None else dw
                hs = h[s:e]
                if main_grad is not None and T <= chunk:
                    # one chunk: the scratch is not rewritten before the step joins the side stream, so the
                    # weight gradient may run beside the input-gradient product
                    launch_wgrad(lambda: matmul(dl, hs, a_mn=True, b_mn=True, out=target, accumulate=True), dl, hs)
                else:
                    matmul(dl, hs, a_mn=True, b_mn=True, out=target, accumulate=True)
        if main_grad is not None:
            w.grad_in_main = True
        elif dw is not None:
            dw = dw.to(w.dtype)
        return dh, dw, None, None


def linear_cross_entropy(h, w, labels, *, ignore_index=IGNORE_INDEX, chunk=8192, soft_cap=None):
    """Per-token ``(ce, lse)`` of ``softmax(h @ w.T)`` against ``labels`` (fp32, differentiable)."""
    if h.dim() != 2:
        h = h.reshape(-1, h.shape[-1])
        labels = labels.reshape(-1)
    lab = torch.where(labels == ignore_index, torch.full_like(labels, -1), labels)
    use_native = (native.available() and h.is_cuda and h.dtype == torch.bfloat16
                  and w.dtype == torch.bfloat16 and not soft_cap and h.shape[1] % 8 == 0)
    if use_native:
        if not h.is_contiguous():
            h = h.contiguous()
        return _FusedLinearCE.apply(h, w, lab.to(torch.int32).contiguous(), chunk)
    return _ChunkedReference.apply(h, w, lab.long(), min(chunk, 2048), soft_cap)


def linear_cross_entropy_reference(h, w, labels, ignore_index=IGNORE_INDEX, soft_cap=None):
    """Materialised-logit oracle for tests."""
    logits = h.float() @ w.float().t()
    if soft_cap:
        logits = soft_cap * torch.tanh(logits / soft_cap)
    lse = torch.logsumexp(logits, -1)
    valid = labels != ignore_index
    tgt = logits.gather(1, labels.clamp(min=0)[:, None]).squeeze(1)
    return torch.where(valid, lse - tgt, torch.zeros_like(lse)), lse
