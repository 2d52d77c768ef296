"""Optimizer-side kernels on the GPU: stochastic rounding (bit-exact against the reference given the same
draws; Philox draws equal to the C++ oracle's), fused write-back, grouped write-back, 16-bit AdamW, flat
AdamW against the C++ oracle."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_sr_cast_bit_exact_with_given_draws_and_with_oracle_philox():
    from kohakuwullm_b200.ops import cpu_oracle as co
    from kohakuwullm_b200.ops.optim import sr_cast, stochastic_round_reference

    torch.manual_seed(0)
    x = torch.randn(5000, device="cuda") * 3
    draws64 = torch.randint(0, 1 << 16, (5000,))
    got = sr_cast(x, draws=draws64.to(torch.uint16).cuda())
    want = stochastic_round_reference(x.cpu(), draws64)
    assert torch.equal(got.cpu().view(torch.int16), want.view(torch.int16))
    # device Philox stream == C++ oracle stream
    seed, offset, n = 20090220, 12345, 257
    got = sr_cast(x[:n].contiguous(), seed=seed, offset=offset).cpu()
    bits = torch.tensor([co.draw16(seed, offset + i) for i in range(n)])
    want = co.sr_round(x[:n].cpu(), bits).to(torch.bfloat16)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))


def test_sr_update_and_grouped_writeback_agree():
    from kohakuwullm_b200.ops.optim import GroupedWriteback, sr_update_

    torch.manual_seed(1)
    shapes = [(300,), (17, 33), (1024,), (5, 7, 11)]
    ps = [torch.randn(s, device="cuda").bfloat16() for s in shapes]
    us = [torch.randn(s, device="cuda") for s in shapes]
    loop = [p.clone() for p in ps]
    offset = 0
    for p, u in zip(loop, us):
        sr_update_(p, u, 0.01, -0.5, seed=99, offset=offset)
        offset += p.numel()
    grouped = [p.clone() for p in ps]
    GroupedWriteback(grouped, us).step([0.01] * 4, [-0.5] * 4, seed=99)
    torch.cuda.synchronize()
    for a, b in zip(loop, grouped):
        assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    # stochastic rounding is unbiased: the mean of many roundings approaches the fp32 value
    p = torch.full((1 << 20,), 1.0, device="cuda").bfloat16()
    u = torch.full((1 << 20,), 0.00123, device="cuda")
    sr_update_(p, u, 0.0, 1.0, seed=5)
    assert abs(p.float().mean().item() - 1.00123) < 2e-5


def test_adamw16_matches_eager_twin():
    from kohakuwullm_b200.ops.optim import adamw16_step_

    torch.manual_seed(2)
    n = 10000
    p = torch.randn(n, device="cuda").bfloat16()
    m = torch.zeros(n, device="cuda").bfloat16()
    sv = torch.zeros(n, device="cuda").bfloat16()
    pc, mc, svc = p.cpu().clone(), m.cpu().clone(), sv.cpu().clone()
    for step in (1, 2, 3):
        g = torch.randn(n, device="cuda")
        kw = dict(lr=1e-2, betas=(0.9, 0.95), eps=1e-8, wd=0.1, step=step, grad_scale=0.5)
        adamw16_step_(p, m, sv, g, **kw)
        adamw16_step_(pc, mc, svc, g.cpu(), **kw)
    torch.testing.assert_close(p.cpu().float(), pc.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(m.cpu().float(), mc.float(), rtol=2e-2, atol=1e-3)


def test_flat_adamw_kernel_matches_cpp_oracle():
    from kohakuwullm_b200.ops import cpu_oracle as co
    from kohakuwullm_b200.parallel.flat import FlatParameters
    from kohakuwullm_b200.training.optim.fused_adamw import FlatAdamW

    torch.manual_seed(3)
    lin = torch.nn.Linear(64, 48, bias=False).cuda()
    flat = FlatParameters(lin)
    opt = FlatAdamW(flat, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    p = lin.weight.detach().cpu().reshape(-1).clone()
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    scale = torch.tensor([0.25], device="cuda")
    for step in (1, 2, 3):
        g = torch.randn(48, 64, device="cuda")
        lin.weight.main_grad.copy_(g)
        opt.step(grad_scale=scale)
        co.adamw(p, m, v, g.cpu().reshape(-1), 0.25, 1e-2, 0.9, 0.95, 1e-8, 0.1, step)
    torch.testing.assert_close(lin.weight.detach().cpu().reshape(-1), p, rtol=1e-5, atol=1e-6)
    assert float(lin.weight.main_grad.abs().sum()) == 0.0


def test_muon_batched_products_on_the_grouped_gemm_match_bmm():
    """The Newton-Schulz products of a batch of equal-shape matrices run as ONE grouped tcgen05 launch each; they
    must equal ``torch.bmm`` in fp32 to bf16 rounding, and the whole iteration must orthogonalise."""
    from kohakuwullm_b200.ops import native
    from kohakuwullm_b200.training.optim.muon import PHASES_GRAM, bmm_nt, newton_schulz_cubic

    torch.manual_seed(0)
    a = torch.randn(5, 256, 640, device="cuda").bfloat16()
    g = bmm_nt(a, a)                                   # X X^T, both operands K-major
    want = torch.bmm(a.float(), a.float().transpose(1, 2))
    assert (g.float() - want).abs().max().item() <= 2e-2 * want.abs().max().item()
    p = torch.randn(5, 256, 256, device="cuda").bfloat16()
    y = bmm_nt(p, a, b_mn=True)                        # P X, X MN-major
    want = torch.bmm(p.float(), a.float())
    assert (y.float() - want).abs().max().item() <= 2e-2 * want.abs().max().item()
    grads = torch.randn(6, 256, 768, device="cuda").bfloat16()
    u = newton_schulz_cubic(grads, torch.bfloat16, phases=PHASES_GRAM)
    ref = newton_schulz_cubic(grads.float().cpu(), torch.float32, phases=PHASES_GRAM)
    assert (u.float().cpu() - ref).abs().max().item() < 0.05
    sv = torch.linalg.svdvals(u.float())
    assert sv.min() > 0.3 and sv.max() < 1.3
    native.check_status()


@pytest.mark.parametrize("n", [1, 3, 1000, 4099, 1 << 20, (1 << 22) + 7])
def test_sumsq_flat_matches_float64_sum(n):
    """Sum of squares for global-norm clipping: ranges per block, tail elements, the accumulate flag; run twice,
    same bits (fixed reduction order)."""
    import ctypes

    from kohakuwullm_b200.ops import native

    L = native.require()
    g = torch.Generator(device="cuda").manual_seed(n)
    x = torch.randn(n, device="cuda", generator=g)
    partial = torch.empty(L.kwu_sumsq_blocks(), device="cuda")
    out = torch.full((1,), 5.0, device="cuda")

    def run(acc):
        native.check(L.kwu_sumsq_flat(native.ptr(x), ctypes.c_longlong(n), native.ptr(partial), native.ptr(out),
                                      ctypes.c_int(acc), native.stream_ptr()), "sumsq")
        return float(out)

    first = run(0)
    want = float(x.double().pow(2).sum())
    assert abs(first - want) <= 2e-6 * want + 1e-12
    assert run(0) == first
    assert abs(run(1) - 2 * want) <= 4e-6 * want + 1e-12
