"""MXFP8: quantiser bit-exact against the PyTorch restatement, block-scaled GEMM against the fp32
product of the dequantised operands, linear layer against bf16."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,K", [(128, 128), (300, 256), (4096, 1280), (77, 3584)])
def test_quantize_bit_exact(M, K):
    from kohakuwullm_b200.ops import mxfp8 as mx

    torch.manual_seed(0)
    x = (torch.randn(M, K, device="cuda") * torch.logspace(-3, 2, K, device="cuda")).to(torch.bfloat16)
    x[0, :32] = 0  # an all-zero block
    q, sf = mx.quantize(x)
    q_ref, e_ref = mx.quantize_reference(x)
    assert torch.equal(mx.sf_to_natural(sf, M, K), e_ref)
    assert torch.equal(q.view(torch.float8_e4m3fn).float(), q_ref.float())
    # rows of the last 128-row tile beyond M carry the neutral exponent, never 0xFF
    pad = mx.sf_to_natural(sf, (M + 127) // 128 * 128, K)[M:]
    assert (pad == 127).all()


@pytest.mark.parametrize("R,C", [(128, 128), (1280, 1792), (3584, 1280)])
def test_quantize_transposed_matches_rowwise_of_transpose(R, C):
    from kohakuwullm_b200.ops import mxfp8 as mx

    torch.manual_seed(1)
    w = (torch.randn(R, C, device="cuda") * 0.05).to(torch.bfloat16)
    qt, sft = mx.quantize_transposed(w)
    q_ref, sf_ref = mx.quantize(w.t().contiguous())
    assert torch.equal(qt, q_ref)
    assert torch.equal(mx.sf_to_natural(sft, C, R), mx.sf_to_natural(sf_ref, C, R))


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (256, 384, 512), (4096, 1792, 1280), (1000, 1280, 3584)])
def test_block_scaled_gemm_matches_dequantised_product(M, N, K):
    from kohakuwullm_b200.ops import mxfp8 as mx, native

    torch.manual_seed(2)
    a = (torch.randn(M, K, device="cuda") * torch.logspace(-2, 1, K, device="cuda")).to(torch.bfloat16)
    b = (torch.randn(N, K, device="cuda") * 0.1).to(torch.bfloat16)
    aq, asf = mx.quantize(a)
    bq, bsf = mx.quantize(b)
    out = mx.gemm(aq, asf, bq, bsf, out_dtype=torch.float32)
    torch.cuda.synchronize()
    native.check_status()
    ref = (mx.dequantize(aq.view(torch.float8_e4m3fn), mx.sf_to_natural(asf, M, K))
           @ mx.dequantize(bq.view(torch.float8_e4m3fn), mx.sf_to_natural(bsf, N, K)).t())
    err = (out - ref).abs().max().item()
    assert err <= 2e-3 * ref.abs().max().item() + 1e-4, f"err {err} scale {ref.abs().max().item()}"


def test_mxfp8_linear_fwd_bwd_close_to_bf16():
    from kohakuwullm_b200.models.components.mlp import Linear
    from kohakuwullm_b200.ops import native

    torch.manual_seed(3)
    lin = Linear(1280, 1792).cuda()
    torch.nn.init.normal_(lin.weight, std=0.02)
    lin.weight.data = lin.weight.data.to(torch.bfloat16)
    x = torch.randn(512, 1280, device="cuda", dtype=torch.bfloat16)
    dy = torch.randn(512, 1792, device="cuda", dtype=torch.bfloat16)
    xa = x.clone().requires_grad_()
    ya = lin(xa)
    ya.backward(dy)
    ga, gw = xa.grad.clone(), lin.weight.grad.clone()
    lin.weight.grad = None
    lin.mxfp8 = True
    xb = x.clone().requires_grad_()
    yb = lin(xb)
    yb.backward(dy)
    torch.cuda.synchronize()
    native.check_status()
    for got, want, tol in ((yb, ya, 0.06), (xb.grad, ga, 0.06), (lin.weight.grad, gw, 0.02)):
        rel = (got.float() - want.float()).norm() / want.float().norm()
        assert rel < tol, f"relative error {rel}"
