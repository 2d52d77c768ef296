"""The C++ CPU oracles (csrc/cpu/oracle.cpp) against the PyTorch references of the same rules: two
independent statements of every kernel family's arithmetic must agree before either is used to check a
CUDA kernel."""

import torch

from kohakuwullm_b200.ops import cpu_oracle as co


def test_rmsnorm_fwd_bwd():
    from kohakuwullm_b200.ops.elementwise import rmsnorm_reference

    torch.manual_seed(0)
    x = torch.randn(37, 96, requires_grad=True)
    w = torch.randn(96, requires_grad=True)
    dy = torch.randn(37, 96)
    for one_plus in (False, True):
        y = rmsnorm_reference(x, w, 1e-6, one_plus)
        gx, gw = torch.autograd.grad(y, (x, w), dy)
        torch.testing.assert_close(co.rmsnorm_fwd(x, w, 1e-6, one_plus), y.detach(), rtol=1e-5, atol=1e-5)
        dx, dw = co.rmsnorm_bwd(x, w, dy, 1e-6, one_plus)
        torch.testing.assert_close(dx, gx, rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(dw, gw, rtol=1e-4, atol=1e-4)


def test_swiglu_fwd_bwd():
    from kohakuwullm_b200.ops.elementwise import swiglu_reference

    torch.manual_seed(1)
    h = torch.randn(19, 64, requires_grad=True)
    d = torch.randn(19, 32)
    y = swiglu_reference(h)
    (gh,) = torch.autograd.grad(y, h, d)
    torch.testing.assert_close(co.swiglu_fwd(h), y.detach(), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(co.swiglu_bwd(h, d), gh, rtol=1e-4, atol=1e-5)


def test_rope_and_inverse():
    from kohakuwullm_b200.ops.elementwise import rotate_half_reference

    torch.manual_seed(2)
    x = torch.randn(11, 3, 64)
    ang = torch.rand(11, 16) * 6.28
    cos, sin = ang.cos(), ang.sin()
    y = co.rope(x, cos, sin)
    torch.testing.assert_close(y, rotate_half_reference(x, cos, sin).float(), rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(co.rope(y, cos, sin, inverse=True), x, rtol=1e-5, atol=1e-5)


def test_varlen_attention_window_and_sink():
    from kohakuwullm_b200.ops.attention import varlen_attention_reference

    torch.manual_seed(3)
    T, Hq, Hkv, D = 50, 4, 2, 16
    q, k, v = torch.randn(T, Hq, D), torch.randn(T, Hkv, D), torch.randn(T, Hkv, D)
    cu = torch.tensor([0, 17, 18, 50], dtype=torch.int32)
    sink = torch.randn(Hq)
    for window, s in ((None, None), (8, None), (8, sink)):
        ref, ref_lse = varlen_attention_reference(q, k, v, cu, window, s, return_lse=True)
        out, lse = co.attention_varlen(q, k, v, cu, window, s)
        torch.testing.assert_close(out, ref.float(), rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(lse, ref_lse.float(), rtol=1e-4, atol=1e-5)


def test_mxfp8_quantize_is_bit_exact_with_the_torch_rule():
    from kohakuwullm_b200.ops.mxfp8 import dequantize, quantize_reference

    torch.manual_seed(4)
    x = torch.randn(16, 128) * torch.logspace(-6, 4, 16)[:, None]
    x[0, :32] = 0.0                     # an all-zero block
    x[1, 5] = 448.0 * 2.0 ** 3          # an exact power-of-two multiple of the format maximum
    q, e8, deq = co.mxfp8_quantize(x)
    q_ref, e_ref = quantize_reference(x)
    assert torch.equal(e8, e_ref)
    assert torch.equal(q, q_ref.view(torch.uint8))
    torch.testing.assert_close(deq, dequantize(q_ref, e_ref), rtol=0, atol=0)
    # e4m3 conversion over every representable value and the midpoints between neighbours
    vals = torch.tensor([co.lib().kwo_e4m3_to_float(b) for b in range(0x7f)])
    mids = (vals[:-1] + vals[1:]) / 2
    probe = torch.cat([vals, mids, mids * 1.0001, mids * 0.9999])
    want = probe.to(torch.float8_e4m3fn).view(torch.uint8)
    got = torch.tensor([co.lib().kwo_e4m3_from_float(float(p)) for p in probe], dtype=torch.uint8)
    assert torch.equal(got, want)


def test_linear_ce():
    torch.manual_seed(5)
    x, W = torch.randn(23, 32), torch.randn(101, 32)
    labels = torch.randint(0, 101, (23,))
    labels[3] = -100
    logits = x @ W.t()
    ce_ref = torch.nn.functional.cross_entropy(logits, labels, reduction="none", ignore_index=-100)
    ce, lse = co.linear_ce(x, W, labels)
    torch.testing.assert_close(ce, ce_ref, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(lse, torch.logsumexp(logits, -1), rtol=1e-5, atol=1e-5)


def test_router_and_experts():
    from kohakuwullm_b200.models.components.moe import TopKRouter
    from kohakuwullm_b200.ops.moe import routed_experts_reference

    torch.manual_seed(6)
    T, D, E, k, H = 40, 32, 16, 3, 8
    x = torch.randn(T, D)
    for score in ("sigmoid", "softmax", "sqrtsoftplus"):
        r = TopKRouter(D, E, k, score=score, routed_scaling_factor=1.5)
        torch.nn.init.normal_(r.weight, std=0.5)
        r.expert_bias.normal_(0, 0.3)
        r.eval()
        idx_ref, w_ref, counts_ref = r.route(x)
        idx, w, counts = co.router_topk(x, r.weight, r.expert_bias, k, score, True, 1.5)
        assert torch.equal(idx.long(), idx_ref.long())
        torch.testing.assert_close(w, w_ref.float(), rtol=1e-5, atol=1e-6)
        assert torch.equal(counts.long(), counts_ref.long())
    w_in, w_out = torch.randn(E, 2 * H, D) * 0.2, torch.randn(E, D, H) * 0.2
    y_ref = routed_experts_reference(x, idx_ref, w_ref, w_in, w_out)
    torch.testing.assert_close(co.routed_experts(x, idx_ref, w_ref, w_in, w_out), y_ref.float(), rtol=1e-4, atol=1e-5)


def test_adamw_matches_torch():
    torch.manual_seed(7)
    p0, g = torch.randn(1000), torch.randn(1000)
    p = torch.nn.Parameter(p0.clone())
    opt = torch.optim.AdamW([p], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    pc, m, v = p0.clone(), torch.zeros(1000), torch.zeros(1000)
    for step in (1, 2, 3):
        p.grad = g * 0.5
        opt.step()
        co.adamw(pc, m, v, g, 0.5, 1e-2, 0.9, 0.95, 1e-8, 0.1, step)
    torch.testing.assert_close(pc, p.detach(), rtol=1e-5, atol=1e-6)


def test_stochastic_rounding_and_philox_draws():
    from kohakuwullm_b200.ops.optim import stochastic_round_reference as sr_round_reference

    torch.manual_seed(8)
    x = torch.randn(4096)
    bits = torch.randint(0, 1 << 16, (4096,))
    got = co.sr_round(x, bits)
    torch.testing.assert_close(got, sr_round_reference(x, bits).float(), rtol=0, atol=0)
    # unbiased: the mean over all 65536 draws of one value is the value itself
    one = torch.full((65536,), 1.2345678)
    mean = co.sr_round(one, torch.arange(65536)).double().mean().item()
    assert abs(mean - 1.2345678) < 1e-6
    # Philox draws: fixed vectors (counter 0 and a large index) stay stable and the eight draws of one
    # block come from one generator call
    d = [co.draw16(1234, i) for i in range(16)]
    assert len(set(d)) > 8 and all(0 <= v < 65536 for v in d)
    assert d != [co.draw16(1235, i) for i in range(16)]
