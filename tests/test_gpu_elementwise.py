"""Native RMSNorm / SwiGLU / QK-norm+RoPE against their fp32 PyTorch references."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _close(got, want, tol=2e-2):
    err = (got.float() - want.float()).abs().max().item()
    scale = max(want.float().abs().max().item(), 1e-6)
    assert err <= tol * scale, f"max err {err} scale {scale}"


@pytest.mark.parametrize("rows,cols", [(37, 256), (4096, 1280), (513, 1536)])
@pytest.mark.parametrize("affine", [True, False])
@pytest.mark.parametrize("with_res", [False, True])
def test_rmsnorm_fwd_bwd(rows, cols, affine, with_res):
    from kohakuwullm_b200.ops.elementwise import rmsnorm, rmsnorm_reference

    torch.manual_seed(1)
    x = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16)
    res = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16) if with_res else None
    w = (torch.randn(cols, device="cuda") * 0.1 + 1.0) if affine else None
    dy = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16)
    dh = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16)

    def run(fn, xin, win, rin):
        xin = xin.clone().requires_grad_()
        win = win.clone().requires_grad_() if win is not None else None
        rin = rin.clone().requires_grad_() if rin is not None else None
        out = fn(xin, win, 1e-6, False, rin)
        if rin is not None:
            y, h = out
            torch.autograd.backward([y, h], [dy.to(y.dtype), dh.to(h.dtype)])
        else:
            y = out
            y.backward(dy.to(y.dtype))
        return y, xin.grad, (win.grad if win is not None else None), (rin.grad if rin is not None else None)

    y, dx, dw, dr = run(rmsnorm, x, w, res)
    yr, dxr, dwr, drr = run(rmsnorm_reference, x.float(), w, res.float() if res is not None else None)
    _close(y, yr)
    _close(dx, dxr, 3e-2)
    if affine:
        _close(dw, dwr, 3e-2)
    if with_res:
        _close(dr, drr, 3e-2)


@pytest.mark.parametrize("rows,H", [(33, 64), (4096, 3584)])
def test_swiglu_fwd_bwd(rows, H):
    from kohakuwullm_b200.ops.elementwise import swiglu, swiglu_reference

    torch.manual_seed(2)
    h = torch.randn(rows, 2 * H, device="cuda", dtype=torch.bfloat16)
    dy = torch.randn(rows, H, device="cuda", dtype=torch.bfloat16)
    a = h.clone().requires_grad_()
    y = swiglu(a)
    y.backward(dy)
    b = h.float().requires_grad_()
    yr = swiglu_reference(b)
    yr.backward(dy.float())
    _close(y, yr)
    _close(a.grad, b.grad)


@pytest.mark.parametrize("rot_half", [32, 16])
@pytest.mark.parametrize("affine", [False, True])
def test_qknorm_rope_fwd_bwd(rot_half, affine):
    from kohakuwullm_b200.ops.elementwise import qknorm_rope, qknorm_rope_reference

    torch.manual_seed(3)
    T, H, Hkv, D = 777, 6, 2, 64
    qkv = torch.randn(T, (H + 2 * Hkv) * D, device="cuda", dtype=torch.bfloat16)
    ang = torch.rand(T, rot_half, device="cuda") * 6.28
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    w = (torch.randn(D, device="cuda") * 0.1 + 1.0) if affine else None
    dq = torch.randn(T, H, D, device="cuda", dtype=torch.bfloat16)

    src = qkv.clone().requires_grad_()
    wn = w.clone().requires_grad_() if affine else None
    q = qknorm_rope(src[:, : H * D].view(T, H, D), wn, cos, sin)
    q.backward(dq)

    srcr = qkv.float().requires_grad_()
    wr = w.clone().requires_grad_() if affine else None
    qr = qknorm_rope_reference(srcr[:, : H * D].view(T, H, D), wr, cos, sin)
    qr.backward(dq.float())
    _close(q, qr)
    _close(src.grad[:, : H * D], srcr.grad[:, : H * D], 3e-2)
    if affine:
        _close(wn.grad, wr.grad, 3e-2)


def test_embedding_forward_backward_and_main_grad_accumulation():
    from kohakuwullm_b200.ops.elementwise import embedding

    torch.manual_seed(0)
    V, D, T = 1000, 256, 3000
    w = torch.randn(V, D, device="cuda").bfloat16().requires_grad_()
    tok = torch.randint(0, V, (T,), device="cuda")
    dy = torch.randn(T, D, device="cuda").bfloat16()
    y = embedding(tok, w, 2.0)
    ref = torch.nn.functional.embedding(tok, w.detach().float()) * 2.0
    torch.testing.assert_close(y.float(), ref, rtol=1e-2, atol=1e-2)
    y.backward(dy)
    gref = torch.zeros(V, D, device="cuda").index_add_(0, tok, dy.float() * 2.0)
    torch.testing.assert_close(w.grad.float(), gref, rtol=2e-2, atol=2e-2)
    # with a main_grad buffer the sum lands there (fp32, exact up to addition order) and .grad stays empty
    w2 = w.detach().clone().requires_grad_()
    w2.main_grad = torch.ones(V, D, device="cuda")
    embedding(tok, w2, 2.0).backward(dy)
    assert w2.grad is None
    torch.testing.assert_close(w2.main_grad, gref + 1.0, rtol=1e-5, atol=1e-4)


def test_norm_weight_gradients_accumulate_into_main_grad():
    from kohakuwullm_b200.ops.elementwise import qknorm_rope, rmsnorm

    torch.manual_seed(1)
    x = torch.randn(512, 384, device="cuda").bfloat16().requires_grad_()
    dy = torch.randn(512, 384, device="cuda").bfloat16()
    w = torch.rand(384, device="cuda").requires_grad_()
    rmsnorm(x, w).backward(dy)
    w2 = w.detach().clone().requires_grad_()
    w2.main_grad = torch.full((384,), 3.0, device="cuda")
    rmsnorm(x.detach().requires_grad_(), w2).backward(dy)
    assert w2.grad is None
    torch.testing.assert_close(w2.main_grad, w.grad + 3.0, rtol=1e-4, atol=1e-3)
    q = torch.randn(300, 4, 64, device="cuda").bfloat16().requires_grad_()
    dq = torch.randn(300, 4, 64, device="cuda").bfloat16()
    ang = torch.rand(300, 32, device="cuda") * 6.28
    qw = torch.rand(64, device="cuda").requires_grad_()
    qknorm_rope(q, qw, ang.cos(), ang.sin()).backward(dq)
    qw2 = qw.detach().clone().requires_grad_()
    qw2.main_grad = torch.full((64,), -1.0, device="cuda")
    qknorm_rope(q.detach().requires_grad_(), qw2, ang.cos(), ang.sin()).backward(dq)
    assert qw2.grad is None
    torch.testing.assert_close(qw2.main_grad, qw.grad - 1.0, rtol=1e-4, atol=1e-3)
