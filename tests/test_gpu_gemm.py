"""tcgen05 bf16 GEMM against an fp32 PyTorch product of the same bf16 operands."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _operands(M, N, K, a_mn, b_mn, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    a = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    b = torch.randn(N, K, device="cuda", generator=g).to(torch.bfloat16)
    ref = a.float() @ b.float().t()
    a_st = a.t().contiguous() if a_mn else a
    b_st = b.t().contiguous() if b_mn else b
    return a_st, b_st, ref


@pytest.mark.parametrize("bn", [128, 256])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("shape", [(256, 256, 128), (384, 640, 192), (200, 136, 72), (4096, 1280, 1280)])
def test_gemm_matches_fp32_reference(shape, a_mn, b_mn, bn):
    from kohakuwullm_b200.ops import native
    from kohakuwullm_b200.ops.gemm import matmul

    M, N, K = shape
    a, b, ref = _operands(M, N, K, a_mn, b_mn)
    out = matmul(a, b, a_mn=a_mn, b_mn=b_mn, bn=bn)
    torch.cuda.synchronize()
    native.check_status()
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 1e-2 * scale, f"max err {err} vs scale {scale}"


def test_gemm_fp32_accumulate_and_alpha():
    from kohakuwullm_b200.ops import native
    from kohakuwullm_b200.ops.gemm import matmul

    a, b, ref = _operands(512, 384, 256, True, True, seed=3)
    out = torch.ones(512, 384, device="cuda", dtype=torch.float32)
    matmul(a, b, a_mn=True, b_mn=True, out=out, accumulate=True, alpha=0.5)
    matmul(a, b, a_mn=True, b_mn=True, out=out, accumulate=True, alpha=0.5)
    torch.cuda.synchronize()
    native.check_status()
    torch.testing.assert_close(out, ref + 1.0, rtol=1e-4, atol=1e-3)


def test_linear_autograd_matches_torch():
    from kohakuwullm_b200.ops.gemm import linear

    torch.manual_seed(0)
    x = torch.randn(640, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = torch.randn(768, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    dy = torch.randn(640, 768, device="cuda", dtype=torch.bfloat16)
    y = linear(x, w)
    y.backward(dy)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = xr @ wr.t()
    yr.backward(dy.float())
    for got, want in ((y, yr), (x.grad, xr.grad), (w.grad, wr.grad)):
        err = (got.float() - want).abs().max().item()
        assert err <= 1e-2 * want.abs().max().item()


@pytest.mark.parametrize("M,N,K", [(1280, 1280, 4096), (7168, 1280, 4096), (1792, 1280, 8192), (384, 1000, 1024 + 64)])
def test_stream_k_weight_gradient_accumulates_exactly_once(M, N, K):
    """fp32 C += with a long contraction is scheduled stream-K: every CTA takes an equal run of (tile, k-block)
    units and adds its partial tiles into C with vector reductions; each unit must be counted exactly once."""
    from kohakuwullm_b200.ops import native
    from kohakuwullm_b200.ops.gemm import matmul

    a, b, ref = _operands(M, N, K, True, True, seed=5)
    out = torch.full((M, N), 2.0, device="cuda", dtype=torch.float32)
    matmul(a, b, a_mn=True, b_mn=True, out=out, accumulate=True)
    torch.cuda.synchronize()
    native.check_status()
    torch.testing.assert_close(out, ref + 2.0, rtol=1e-4, atol=2e-3 * (K / 4096) ** 0.5 + 1e-3)
