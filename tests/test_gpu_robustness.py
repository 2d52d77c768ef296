"""Memory-safety substitutes for a sanitizer (which is not available on the GPU pool): poisoned padding that an
unmasked read would turn into NaN, canary rows around kernel outputs, and run-twice bit equality for the kernels
that claim to be deterministic."""

import pytest
import torch

pytestmark = pytest.mark.gpu

CANARY = 0x5A


def _guarded(rows, cols, dtype, guard=4):
    """A (rows, cols) view in the middle of a buffer whose ``guard`` rows before and after hold a canary pattern."""
    buf = torch.empty(rows + 2 * guard, cols, dtype=dtype, device="cuda")
    buf.view(torch.uint8).fill_(CANARY)
    return buf, buf[guard:guard + rows]


def _guards_intact(buf, rows, guard=4):
    raw = buf.view(torch.uint8)
    return bool((raw[:guard] == CANARY).all()) and bool((raw[guard + rows:] == CANARY).all())


@pytest.mark.parametrize("M,N,K", [(200, 328, 256), (77, 136, 128), (384, 512, 384)])
def test_poisoned_scale_padding_cannot_reach_valid_outputs(M, N, K):
    """Scale bytes of rows beyond the matrix edge (inside the last 128-row chunk) and a whole chunk behind the
    buffer's end are set to 0xFF (NaN in UE8M0): every stored output must stay finite and equal to the product of
    the dequantised operands, so no scale is read unmasked."""
    from kohakuwullm_b200.ops import mxfp8 as mx
    from kohakuwullm_b200.ops import native

    torch.manual_seed(M + N)
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    aq, asf = mx.quantize(a)
    bq, bsf = mx.quantize(b)
    clean = mx.gemm(aq, asf, bq, bsf)

    def poison(sf, rows):
        big = torch.full((sf.numel() + 512,), 0xFF, dtype=torch.uint8, device="cuda")   # a poisoned chunk behind the end
        big[: sf.numel()] = sf
        view = big[: sf.numel()]
        nk = K // 128
        chunks = view.view(-1, nk, 32, 4, 4)       # [row tile][k chunk][r % 32][r / 32][k block]
        last = (rows - 1) // 128
        for r in range(rows % 128 or 128, 128):
            if rows % 128:
                chunks[last, :, r % 32, r // 32, :] = 0xFF
        return view

    out = mx.gemm(aq, poison(asf, M), bq, poison(bsf, N))
    torch.cuda.synchronize()
    native.check_status()
    assert torch.isfinite(out.float()).all()
    assert torch.equal(out, clean)
    want = mx.dequantize(aq.view(torch.float8_e4m3fn), mx.sf_to_natural(asf, M, K)) @ \
        mx.dequantize(bq.view(torch.float8_e4m3fn), mx.sf_to_natural(bsf, N, K)).t()
    assert (out.float() - want).abs().max().item() <= 2e-2 * want.abs().max().item()


def test_canary_rows_around_kernel_outputs_stay_intact():
    """Quantiser, block-scaled GEMM, bf16 GEMM, RMSNorm and SwiGLU write exactly their output rows: guard rows in
    front of and behind every output keep their pattern, for row counts that are not multiples of any tile."""
    from kohakuwullm_b200.ops import mxfp8 as mx
    from kohakuwullm_b200.ops import native
    from kohakuwullm_b200.ops.gemm import matmul

    torch.manual_seed(0)
    M, N, K = 333, 392, 384
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    qbuf, q = _guarded(M, K, torch.uint8)
    sf_rows = mx.sf_bytes(M, K) // 512
    sbuf, sf = _guarded(sf_rows, 512, torch.uint8)
    mx.quantize(a, q, sf.view(-1))
    bq, bsf = mx.quantize(b)
    obuf, out = _guarded(M, N, torch.bfloat16)
    mx.gemm(q, sf.view(-1), bq, bsf, out=out)
    o2buf, out2 = _guarded(M, N, torch.bfloat16)
    matmul(a, b, out=out2)
    torch.cuda.synchronize()
    native.check_status()
    assert _guards_intact(qbuf, M) and _guards_intact(sbuf, sf_rows) and _guards_intact(obuf, M) and _guards_intact(o2buf, M)
    ref = a.float() @ b.float().t()
    assert (out2.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item()
    # elementwise producers through their public ops (outputs are allocated inside; check values at ragged sizes)
    from kohakuwullm_b200.ops.elementwise import rmsnorm, swiglu

    x = torch.randn(77, 1280, device="cuda").bfloat16()
    w = torch.rand(1280, device="cuda")
    y = rmsnorm(x, w, 1e-6)
    want = (x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6) * w).bfloat16()
    assert (y.float() - want.float()).abs().max().item() <= 2e-2
    h = torch.randn(77, 2 * 896, device="cuda").bfloat16()
    s = swiglu(h)
    want = (torch.nn.functional.silu(h[:, :896].float()) * h[:, 896:].float())
    assert (s.float() - want).abs().max().item() <= 2e-2 * want.abs().max().item()


def test_deterministic_kernels_give_the_same_bits_twice():
    """Kernels that reduce without atomics (attention backward with its group reduction, the MoE combine, the
    quantisers, both GEMM families with bf16 output) must be bit-reproducible run to run."""
    from kohakuwullm_b200.models.seqinfo import SeqInfo
    from kohakuwullm_b200.ops import mxfp8 as mx
    from kohakuwullm_b200.ops import native
    from kohakuwullm_b200.ops.attention import varlen_attention
    from kohakuwullm_b200.ops.gemm import matmul

    torch.manual_seed(1)
    info = SeqInfo.from_lengths([700, 324, 1024], device="cuda")
    T = info.total_tokens
    q0 = torch.randn(T, 20, 64, device="cuda").bfloat16()
    k0 = torch.randn(T, 4, 64, device="cuda").bfloat16()
    v0 = torch.randn(T, 4, 64, device="cuda").bfloat16()
    dout = torch.randn(T, 20, 64, device="cuda").bfloat16()

    def attention():
        q, k, v = (t.clone().requires_grad_() for t in (q0, k0, v0))
        out = varlen_attention(q, k, v, info.cu_seqlens, info.max_seqlen)
        out.backward(dout)
        return out.detach(), q.grad, k.grad, v.grad

    first, second = attention(), attention()
    for a, b in zip(first, second):
        assert torch.equal(a, b)
    a = torch.randn(512, 640, device="cuda").bfloat16()
    b = torch.randn(384, 640, device="cuda").bfloat16()
    assert torch.equal(matmul(a, b), matmul(a, b))
    aq, asf = mx.quantize(a)
    aq2, asf2 = mx.quantize(a)
    assert torch.equal(aq, aq2) and torch.equal(asf, asf2)
    bq, bsf = mx.quantize(b)
    assert torch.equal(mx.gemm(aq, asf, bq, bsf), mx.gemm(aq, asf, bq, bsf))
    # MoE combine: gather-sum in a fixed order
    from kohakuwullm_b200.ops import moe as moe_ops

    x = torch.randn(512, 256, device="cuda").bfloat16()
    w_in = (torch.randn(8, 512, 256, device="cuda") * 0.05).bfloat16()
    w_out = (torch.randn(8, 256, 256, device="cuda") * 0.05).bfloat16()
    idx = torch.randint(0, 8, (512, 2), device="cuda", dtype=torch.int32)
    weight = torch.rand(512, 2, device="cuda")
    counts = torch.bincount(idx.reshape(-1).long(), minlength=8).to(torch.int32)
    y1 = moe_ops.routed_experts(x, idx, weight, counts, w_in, w_out)
    y2 = moe_ops.routed_experts(x, idx, weight, counts, w_in, w_out)
    assert torch.equal(y1, y2)
    torch.cuda.synchronize()
    native.check_status()
