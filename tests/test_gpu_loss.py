"""Fused linear cross-entropy (+lse for z-loss) against materialised fp32 logits."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,D,V,chunk", [(300, 256, 1000, 8192), (1024, 512, 4096, 512), (2048, 1280, 65536, 8192)])
def test_fused_linear_ce_fwd_bwd(T, D, V, chunk):
    from kohakuwullm_b200.ops import native
    from kohakuwullm_b200.ops.loss import linear_cross_entropy, linear_cross_entropy_reference

    torch.manual_seed(0)
    h = (torch.randn(T, D, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn(V, D, device="cuda") * 0.05).to(torch.bfloat16)
    labels = torch.randint(0, V, (T,), device="cuda")
    labels[::7] = -100
    zw = 1e-2

    ha, wa = h.clone().requires_grad_(), w.clone().requires_grad_()
    ce, lse = linear_cross_entropy(ha, wa, labels, chunk=chunk)
    loss = ce.sum() + zw * (lse ** 2).sum()
    loss.backward()
    torch.cuda.synchronize()
    native.check_status()

    hr, wr = h.float().requires_grad_(), w.float().requires_grad_()
    ce_r, lse_r = linear_cross_entropy_reference(hr, wr, labels)
    loss_r = ce_r.sum() + zw * (lse_r ** 2).sum()
    loss_r.backward()

    torch.testing.assert_close(lse, lse_r, rtol=1e-4, atol=2e-3)
    torch.testing.assert_close(ce, ce_r, rtol=1e-3, atol=5e-3)
    for got, want, name in ((ha.grad, hr.grad, "dh"), (wa.grad, wr.grad, "dw")):
        err = (got.float() - want).abs().max().item()
        scale = want.abs().max().item()
        assert err <= 3e-2 * scale, f"{name}: err {err} scale {scale}"
