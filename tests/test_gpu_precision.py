"""Kernels against FLOAT64 oracles, with bounds in units of the output type's rounding (relative RMS and ULP),
and attention at the document lengths the benchmarks run (4096 and 16384 tokens, window 1024, sinks, GQA 5:1).

An output rounded once from an fp32 accumulator has a mean error of a quarter ULP and, for bf16, a relative RMS
error of 1.65e-3 (both measured: 0.2504 ULP, 1.655e-3); the GEMM bounds sit 10-20 % above that, so a second
rounding anywhere in the kernel fails them. The attention bounds are about twice what the kernels measure on
a B200 (2.0-2.5e-3 for the output and the gradients at 4096 and 16384 tokens)."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel_rms(got, want):
    got, want = got.detach(), want.detach()
    return float((got.double() - want.double()).norm() / want.double().norm().clamp(min=1e-30))


@pytest.mark.parametrize("shape", [(512, 384, 256), (4096, 1280, 1280), (1000, 1792, 3584)])
def test_bf16_gemm_is_one_rounding_from_the_fp64_product(shape):
    from kohakuwullm_b200.bench.timing import ulp_error
    from kohakuwullm_b200.ops import native
    from kohakuwullm_b200.ops.gemm import matmul

    M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(1)
    a = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    b = torch.randn(N, K, device="cuda", generator=g).to(torch.bfloat16)
    want = a.double() @ b.double().t()
    out = matmul(a, b)
    out32 = torch.zeros(M, N, device="cuda", dtype=torch.float32)
    matmul(a, b, out=out32, accumulate=True)
    torch.cuda.synchronize()
    native.check_status()
    u = ulp_error(out, want)
    print(shape, u, _rel_rms(out, want), _rel_rms(out32, want))
    assert u["mean_ulp"] < 0.30, u                       # a single round-to-nearest: 0.25
    assert _rel_rms(out, want) < 1.8e-3, _rel_rms(out, want)
    assert _rel_rms(out32, want) < 3e-6, _rel_rms(out32, want)                # fp32 accumulation, no output rounding (measured 0.2-1.2e-6)


@pytest.mark.parametrize("shape,wide", [((512, 384, 256), False), ((4096, 1792, 1280), True), ((1000, 1280, 3584), True)])
def test_mxfp8_gemm_is_one_rounding_from_the_fp64_product_of_the_dequantised_operands(shape, wide):
    from kohakuwullm_b200.bench.timing import ulp_error
    from kohakuwullm_b200.ops import mxfp8 as mx
    from kohakuwullm_b200.ops import native

    M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(2)
    a = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    b = (torch.randn(N, K, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    aq, asf = mx.quantize(a)
    bq, bsf = mx.quantize(b)
    want = (mx.dequantize(aq.view(torch.float8_e4m3fn), mx.sf_to_natural(asf, M, K)).double()
            @ mx.dequantize(bq.view(torch.float8_e4m3fn), mx.sf_to_natural(bsf, N, K)).double().t())
    bn = mx.pick_tile_width(N, M) if wide else 128
    if bn != 128:
        bq = torch.empty(N, K, dtype=torch.uint8, device="cuda")
        bsf = mx.alloc_weight_sf(N, K, bn, "cuda")
        mx.quantize_weight(b, bq, bsf, bn)
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    mx.gemm(aq, asf, bq, bsf, out=out, bn=bn)
    torch.cuda.synchronize()
    native.check_status()
    u = ulp_error(out, want)
    print(shape, bn, u, _rel_rms(out, want))
    assert u["mean_ulp"] < 0.30, u
    assert _rel_rms(out, want) < 1.8e-3, _rel_rms(out, want)


def _attention_fp64(q, k, v, do, sink, window, scale):
    """One document, all heads of ONE kv group, float64, explicit backward (no autograd graph: at 16384 tokens
    every (L, L) matrix is 2 GiB)."""
    L, Hq, D = q.shape
    kd, vd = k[:, 0].double(), v[:, 0].double()
    pos = torch.arange(L, device=q.device)
    allowed = pos[None, :] <= pos[:, None]
    if window:
        allowed &= pos[None, :] > pos[:, None] - window
    out = torch.empty(L, Hq, D, dtype=torch.float64, device=q.device)
    dq = torch.empty_like(out)
    dk = torch.zeros(L, D, dtype=torch.float64, device=q.device)
    dv = torch.zeros_like(dk)
    dsink = torch.zeros(Hq, dtype=torch.float64, device=q.device)
    for h in range(Hq):
        qh, doh = q[:, h].double(), do[:, h].double()
        s = (qh @ kd.t()) * scale
        s.masked_fill_(~allowed, float("-inf"))
        m = s.max(dim=-1, keepdim=True).values
        if sink is not None:
            m = torch.maximum(m, sink[h].double().reshape(1, 1))
        p = torch.exp(s - m)
        den = p.sum(-1, keepdim=True)
        if sink is not None:
            ps = torch.exp(sink[h].double() - m)
            den = den + ps
        p /= den
        o = p @ vd
        out[:, h] = o
        delta = (o * doh).sum(-1, keepdim=True)
        dv += p.t() @ doh
        ds = p * ((doh @ vd.t()) - delta) * scale
        dq[:, h] = ds @ kd
        dk += ds.t() @ qh
        if sink is not None:
            dsink[h] = -((ps / den) * delta).sum()
        del s, p, ds
    return out, dq, dk, dv, dsink


@pytest.mark.parametrize("length,window,sinks", [(4096, None, False), (4096, 1024, True), (16384, None, False),
                                                 (16384, 1024, True)])
def test_flash_attention_at_benchmark_lengths_against_fp64(length, window, sinks):
    from kohakuwullm_b200.models.seqinfo import SeqInfo
    from kohakuwullm_b200.ops import native
    from kohakuwullm_b200.ops.attention import varlen_attention

    Hq, Hkv = 5, 1                                       # GQA 5:1, one kv group
    g = torch.Generator(device="cuda").manual_seed(3)
    info = SeqInfo.from_lengths([length], device="cuda")
    q = torch.randn(length, Hq, 64, device="cuda", generator=g).to(torch.bfloat16).requires_grad_()
    k = torch.randn(length, Hkv, 64, device="cuda", generator=g).to(torch.bfloat16).requires_grad_()
    v = torch.randn(length, Hkv, 64, device="cuda", generator=g).to(torch.bfloat16).requires_grad_()
    do = torch.randn(length, Hq, 64, device="cuda", generator=g).to(torch.bfloat16)
    sink = torch.randn(Hq, device="cuda", generator=g).requires_grad_() if sinks else None
    out = varlen_attention(q, k, v, info.cu_seqlens, window=window, sink_lse=sink)
    out.backward(do)
    torch.cuda.synchronize()
    native.check_status()
    with torch.no_grad():
        want = _attention_fp64(q.detach(), k.detach(), v.detach(), do, sink.detach() if sinks else None, window, 0.125)
    got = (out, q.grad, k.grad[:, 0], v.grad[:, 0]) + ((sink.grad,) if sinks else ())
    names = ("out", "dq", "dk", "dv", "dsink")
    bounds = {"out": 4e-3, "dq": 5e-3, "dk": 5e-3, "dv": 5e-3, "dsink": 6e-3}
    errs = {n: _rel_rms(a, b) for n, a, b in zip(names, got, want)}
    print(length, window, sinks, errs)
    for n, e in errs.items():
        assert e < bounds[n], errs
