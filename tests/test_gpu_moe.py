"""Native MoE path (router, dispatch, grouped GEMMs, combine) against the per-expert PyTorch loop."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("score", ["sigmoid", "softmax", "sqrtsoftplus"])
def test_router_matches_eager(score):
    from kohakuwullm_b200.models.components.moe import TopKRouter

    torch.manual_seed(0)
    r = TopKRouter(256, 64, 6, score=score).cuda()
    torch.nn.init.normal_(r.weight, std=0.5)
    r.expert_bias.normal_(0, 0.5)
    x = torch.randn(1000, 256, device="cuda", dtype=torch.bfloat16)
    r.train()
    idx, w, counts = r.route(x)                       # native
    load_native = r.load_accum.clone()
    r.load_accum.zero_()
    idx_e, w_e, counts_e = r.route(x.float())          # eager fp32 path on the same bf16 values
    assert torch.equal(counts.long(), counts_e.long())
    assert torch.equal(load_native, r.load_accum)
    assert torch.equal(idx.long().sort(-1).values, idx_e.sort(-1).values)
    torch.testing.assert_close(w.sort(-1).values, w_e.sort(-1).values, rtol=1e-4, atol=1e-5)


def test_moe_bias_steers_selection_not_weights():
    from kohakuwullm_b200.models.components.moe import TopKRouter

    torch.manual_seed(1)
    r = TopKRouter(128, 32, 4, norm_topk_prob=False).cuda()
    torch.nn.init.normal_(r.weight, std=0.5)
    x = torch.randn(256, 128, device="cuda", dtype=torch.bfloat16)
    idx0, w0, _ = r.route(x)
    r.expert_bias[5] = 100.0          # expert 5 is now always selected ...
    idx1, w1, _ = r.route(x)
    assert (idx1 == 5).any(-1).all()
    s = torch.sigmoid(x.float() @ r.weight.t())
    picked = w1[idx1 == 5]
    torch.testing.assert_close(picked, s[:, 5], rtol=1e-4, atol=1e-5)   # ... but weighted by its UNBIASED score


@pytest.mark.parametrize("T,dim,E,k,H", [(512, 256, 8, 2, 128), (4096, 1024, 64, 6, 384)])
def test_routed_experts_fwd_bwd(T, dim, E, k, H):
    from kohakuwullm_b200.ops import native
    from kohakuwullm_b200.ops.moe import routed_experts, routed_experts_reference

    torch.manual_seed(2)
    x = torch.randn(T, dim, device="cuda", dtype=torch.bfloat16)
    w_in = (torch.randn(E, 2 * H, dim, device="cuda") * 0.05).to(torch.bfloat16)
    w_out = (torch.randn(E, dim, H, device="cuda") * 0.05).to(torch.bfloat16)
    logits = torch.randn(T, E, device="cuda") + torch.randn(E, device="cuda") * 0.5   # skewed load
    idx = logits.topk(k, -1).indices.to(torch.int32)
    gate = torch.rand(T, k, device="cuda")
    counts = torch.bincount(idx.reshape(-1).long(), minlength=E).to(torch.int32)
    dy = torch.randn(T, dim, device="cuda", dtype=torch.bfloat16)

    a = [t.clone().requires_grad_() for t in (x, w_in, w_out, gate)]
    y = routed_experts(a[0], idx, a[3], counts, a[1], a[2])
    y.backward(dy)
    torch.cuda.synchronize()
    native.check_status()
    b = [t.float().clone().requires_grad_() for t in (x, w_in, w_out, gate)]
    yr = routed_experts_reference(b[0], idx.long(), b[3], b[1], b[2])
    yr.backward(dy.float())
    for got, want, name in ((y, yr, "y"), (a[0].grad, b[0].grad, "dx"), (a[1].grad, b[1].grad, "dw_in"),
                            (a[2].grad, b[2].grad, "dw_out"), (a[3].grad, b[3].grad, "dgate")):
        err = (got.float() - want).abs().max().item()
        scale = want.abs().max().item()
        assert err <= 4e-2 * scale, f"{name}: err {err} scale {scale}"


def test_moe_layer_end_to_end():
    from kohakuwullm_b200.models.components.moe import MoEMLP

    torch.manual_seed(3)
    m = MoEMLP(256, num_experts=16, top_k=2, num_shared=1, hidden=128).cuda()
    for n, p in m.named_parameters():
        if p.dim() >= 2:
            torch.nn.init.normal_(p, std=0.05)
            if "router" not in n:
                p.data = p.data.to(torch.bfloat16)
    x = torch.randn(600, 256, device="cuda", dtype=torch.bfloat16)
    y_native = m(x)
    m.expert_path = "eager"
    y_eager = m(x)
    err = (y_native.float() - y_eager.float()).abs().max().item()
    assert err <= 3e-2 * y_eager.float().abs().max().item()


def test_grouped_mxfp8_gemm_matches_dequantised_product():
    """Block-scaled grouped GEMM against fp32 products of the dequantised operands, expert by expert."""
    from kohakuwullm_b200.ops import moe as moe_ops
    from kohakuwullm_b200.ops import mxfp8

    torch.manual_seed(3)
    T, K, N, E, k = 2048, 512, 384, 8, 2
    x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
    W = (torch.randn(E, N, K, device="cuda") * 0.1).bfloat16()
    idx = torch.stack([torch.randperm(E, device="cuda")[:k] for _ in range(T)]).to(torch.int32)
    counts = torch.bincount(idx.reshape(-1).long(), minlength=E).to(torch.int32)
    plan = moe_ops.make_plan(idx, counts, E)
    rows = moe_ops._Gather.apply(x, plan)
    qw = mxfp8.GroupedQuantizedWeight(W)
    xq, xsf = mxfp8.quantize(rows)
    out = mxfp8.grouped_gemm(xq, xsf, qw.q, qw.sf, N, E, plan.tiles)
    torch.cuda.synchronize()
    off = plan.offsets.tolist()
    x_deq = mxfp8.dequantize(xq.view(torch.float8_e4m3fn)[: off[E]], mxfp8.sf_to_natural(xsf, plan.max_rows, K)[: off[E]])
    w_deq = mxfp8.dequantize(qw.q.view(torch.float8_e4m3fn), mxfp8.sf_to_natural(qw.sf, E * N, K)).view(E, N, K)
    for e in range(E):
        s, t = off[e], off[e] + int(counts[e])
        ref = x_deq[s:t] @ w_deq[e].t()
        torch.testing.assert_close(out[s:t].float(), ref, rtol=2e-2, atol=2e-2)
    # transposed copies: W[e]^T quantised along N, expert by expert
    wt_deq = mxfp8.dequantize(qw.qt.view(torch.float8_e4m3fn), torch.cat(
        [mxfp8.sf_to_natural(c, K, N) for c in qw.sft.view(E, -1)])).view(E, K, N)
    torch.testing.assert_close(wt_deq, W.float().transpose(1, 2), rtol=0.07, atol=1e-3)


def test_routed_experts_mxfp8_close_to_bf16():
    from kohakuwullm_b200.ops import moe as moe_ops
    from kohakuwullm_b200.ops import mxfp8

    torch.manual_seed(4)
    T, dim, E, k, H = 4096, 1024, 16, 4, 384
    x = torch.randn(T, dim, device="cuda", dtype=torch.bfloat16)
    w_in = (torch.randn(E, 2 * H, dim, device="cuda") * 0.03).bfloat16()
    w_out = (torch.randn(E, dim, H, device="cuda") * 0.03).bfloat16()
    logits = torch.randn(T, E, device="cuda")
    gate, idx = torch.softmax(logits, -1).topk(k, -1)
    idx = idx.to(torch.int32)
    counts = torch.bincount(idx.reshape(-1).long(), minlength=E).to(torch.int32)
    dy = torch.randn(T, dim, device="cuda", dtype=torch.bfloat16) * 0.1

    def run(q_in, q_out):
        xs, wi, wo, g = (t.clone().requires_grad_() for t in (x, w_in, w_out, gate))
        y = moe_ops.routed_experts(xs, idx, g, counts, wi, wo, q_in, q_out)
        y.backward(dy)
        return [t.float() for t in (y.detach(), xs.grad, g.grad, wi.grad, wo.grad)]

    ref = run(None, None)
    got = run(mxfp8.GroupedQuantizedWeight(w_in), mxfp8.GroupedQuantizedWeight(w_out))
    for name, a, b in zip(("y", "dx", "dgate", "dw_in", "dw_out"), got, ref):
        rel = ((a - b).norm() / b.norm().clamp(min=1e-9)).item()
        assert rel < 0.08, f"{name}: relative error {rel}"


@pytest.mark.parametrize("score", ["sigmoid", "softmax", "sqrtsoftplus"])
@pytest.mark.parametrize("norm_topk", [True, False])
def test_router_backward_matches_eager(score, norm_topk):
    """Gate-weight gradient -> logits -> (dx, dW) through the native backward kernels, against autograd over
    the eager fp32 router on the same bf16 values; the router z-loss exercises the dense logit-gradient input."""
    from kohakuwullm_b200.models.components.moe import TopKRouter

    torch.manual_seed(0)
    T, D, E, k = 777, 256, 64, 6
    r = TopKRouter(D, E, k, score=score, norm_topk_prob=norm_topk, routed_scaling_factor=1.7, z_loss_weight=1e-2).cuda()
    torch.nn.init.normal_(r.weight, std=0.3)
    r.train()
    x = torch.randn(T, D, device="cuda", dtype=torch.bfloat16)
    coef = torch.randn(T, k, device="cuda")

    def run(inp):
        r.weight.grad = None
        xs = inp.clone().requires_grad_()
        idx, w, _ = r.route(xs)
        order = idx.long().argsort(-1)                     # slot order may differ between the two paths
        loss = (w.gather(1, order) * coef).sum() + r.aux_loss * T
        loss.backward()
        return xs.grad.float(), r.weight.grad.float().clone()

    dx_n, dW_n = run(x)
    dx_e, dW_e = run(x.float())
    # the products run on the tensor cores with a bf16 copy of the logit gradient: bf16-level agreement
    torch.testing.assert_close(dW_n, dW_e, rtol=2e-2, atol=1e-2 * dW_e.abs().max().item())
    torch.testing.assert_close(dx_n, dx_e, rtol=2e-2, atol=2e-2 * dx_e.abs().max().item())
