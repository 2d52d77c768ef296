"""CPU paths of the ops: they are the oracles of the GPU tests, so they are pinned against
independent formulations here."""

import math

import torch

from kohakuwullm_b200.models.seqinfo import SeqInfo
from kohakuwullm_b200.ops.attention import attention_mask, varlen_attention, varlen_attention_reference
from kohakuwullm_b200.ops.elementwise import qknorm_rope, rmsnorm, swiglu
from kohakuwullm_b200.ops.gemm import linear, matmul
from kohakuwullm_b200.ops.loss import linear_cross_entropy, linear_cross_entropy_reference


def test_matmul_majors_on_cpu():
    a, b = torch.randn(5, 7), torch.randn(3, 7)
    ref = a @ b.t()
    torch.testing.assert_close(matmul(a, b), ref)
    torch.testing.assert_close(matmul(a.t().contiguous(), b, a_mn=True), ref)
    torch.testing.assert_close(matmul(a, b.t().contiguous(), b_mn=True), ref)
    out = torch.ones(5, 3)
    matmul(a, b, out=out, accumulate=True, alpha=2.0)
    torch.testing.assert_close(out, 1 + 2 * ref)
    torch.testing.assert_close(linear(a, b), ref)


def test_attention_reference_matches_dense_mask():
    torch.manual_seed(0)
    info = SeqInfo.from_lengths([5, 9, 3])
    T = info.total_tokens
    q, k, v = torch.randn(T, 4, 8), torch.randn(T, 2, 8), torch.randn(T, 2, 8)
    for window in (None, 4):
        out = varlen_attention(q, k, v, info.cu_seqlens, window=window)
        mask = attention_mask(info.cu_seqlens, T, window)
        kk, vv = k.repeat_interleave(2, 1), v.repeat_interleave(2, 1)
        s = torch.einsum("thd,shd->hts", q, kk) / math.sqrt(8)
        s = s.masked_fill(~mask[None], float("-inf"))
        ref = torch.einsum("hts,shd->thd", s.softmax(-1), vv)
        torch.testing.assert_close(out, ref, rtol=1e-4, atol=1e-5)


def test_attention_sink_is_sigmoid_gate():
    torch.manual_seed(1)
    info = SeqInfo.from_lengths([6, 4])
    T = info.total_tokens
    q, k, v = torch.randn(T, 2, 8), torch.randn(T, 2, 8), torch.randn(T, 2, 8)
    sink = torch.randn(2)
    plain, lse = varlen_attention_reference(q, k, v, info.cu_seqlens, return_lse=True)
    gated = varlen_attention_reference(q, k, v, info.cu_seqlens, sink_lse=sink)
    gate = torch.sigmoid(lse - sink[:, None]).t()[..., None]
    torch.testing.assert_close(gated, plain * gate, rtol=1e-4, atol=1e-5)


def test_chunked_ce_matches_materialised():
    torch.manual_seed(2)
    h = torch.randn(50, 16, requires_grad=True)
    w = torch.randn(40, 16, requires_grad=True)
    labels = torch.randint(0, 40, (50,))
    labels[::5] = -100
    ce, lse = linear_cross_entropy(h, w, labels, chunk=16)
    (ce.sum() + 0.1 * (lse ** 2).sum()).backward()
    g1, g2 = h.grad.clone(), w.grad.clone()
    h.grad = w.grad = None
    ce_r, lse_r = linear_cross_entropy_reference(h, w, labels)
    (ce_r.sum() + 0.1 * (lse_r ** 2).sum()).backward()
    torch.testing.assert_close(ce, ce_r)
    torch.testing.assert_close(g1, h.grad, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(g2, w.grad, rtol=1e-4, atol=1e-5)


def test_elementwise_cpu_paths():
    x = torch.randn(4, 16)
    y = rmsnorm(x, torch.ones(16))
    torch.testing.assert_close(y.pow(2).mean(-1), torch.ones(4), rtol=1e-3, atol=1e-3)
    y2, h = rmsnorm(x, None, residual=x)
    torch.testing.assert_close(h, 2 * x)
    g = torch.randn(3, 8)
    torch.testing.assert_close(swiglu(g), torch.nn.functional.silu(g[:, :4]) * g[:, 4:])
    q = torch.randn(5, 2, 64)
    ang = torch.rand(5, 32)
    out = qknorm_rope(q, None, ang.cos(), ang.sin())
    # rotation preserves the norm of the normalised vector
    torch.testing.assert_close(out.pow(2).mean(-1), torch.ones(5, 2), rtol=1e-3, atol=1e-3)


def test_quantize_heads_cpu_fallback_is_straight_through():
    import torch

    from kohakuwullm_b200.ops.attention import quantize_heads, quantize_heads_reference

    torch.manual_seed(0)
    x = torch.randn(50, 3, 64, requires_grad=True)
    y = quantize_heads(x)
    assert torch.equal(y.detach(), quantize_heads_reference(x.detach()))
    y.sum().backward()
    assert torch.equal(x.grad, torch.ones_like(x))
    k = torch.randn(50, 2, 64, requires_grad=True)
    ks = quantize_heads(k, smooth=True)
    (ks * torch.randn_like(ks)).sum().backward()
    assert k.grad.mean(0).abs().max() < 1e-6          # the mean subtraction removes the gradient's token mean
    # values are within one e4m3 step of the smoothed input
    err = (ks.detach() - (k.detach() - k.detach().mean(0, keepdim=True))).abs().max()
    assert err < 0.07 * k.detach().abs().max()


def test_mxfp8_wiring_sets_producer_flags():
    import torch

    from kohakuwullm_b200.models import LMBackbone, get_preset
    from kohakuwullm_b200.models.components.norm import RMSNorm

    cfg = get_preset("B200-smoke", vocab_size=512, mxfp8=True, mlp_hidden=768)
    model = LMBackbone(cfg)
    blocks = list(model.blocks)
    assert all(b.norm_attn.emit_mx and b.norm_mlp.emit_mx and b.norm_mlp.emit_mx_grad for b in blocks)
    assert not blocks[0].norm_attn.emit_mx_grad and all(b.norm_attn.emit_mx_grad for b in blocks[1:])
    assert model.final_norm.emit_mx_grad
    plain = LMBackbone(get_preset("B200-smoke", vocab_size=512, mxfp8=False, mlp_hidden=768))
    assert not any(m.emit_mx or m.emit_mx_grad for m in plain.modules() if isinstance(m, RMSNorm))
    # the CPU forward ignores the flags (no native kernels): same loss path as without them
    tok = torch.randint(0, 512, (64,))
    from kohakuwullm_b200.models.seqinfo import SeqInfo

    out = model(tok, SeqInfo.from_lengths([40, 24]))
    assert out.shape == (64, cfg.dim)


def test_mxfp8_swap_census_buckets_and_closing_sweep():
    """The conversion report accounts for every matmul-shaped parameter: converted work lands in ``fp8``, the
    vocabulary head and router gates in ``never``, a refused layer in ``skipped``, a declared-but-unconverted
    expert stack in ``unreached``, and a parameter nobody claims is listed by the closing sweep."""
    import torch
    from torch import nn

    from kohakuwullm_b200.models import LMBackbone, get_preset
    from kohakuwullm_b200.models.mxfp8_swap import swap_mxfp8

    torch.manual_seed(0)
    dense = LMBackbone(get_preset("B200-smoke", vocab_size=512, dim=256, depth=2, heads=4, kv_heads=2, mlp_hidden=384))
    rep = swap_mxfp8(dense)
    assert len(rep.modules) == 2 * 4 and not rep.blocking and not rep.unaccounted and not rep.unreached
    per_layer = 256 * (256 + 2 * 128) + 256 * 256 + 256 * 768 + 384 * 256
    assert rep.mac["fp8"] == 2 * per_layer and rep.mac["never"] == 512 * 256
    assert abs(sum(rep.share(b) for b in ("fp8", "skipped", "unreached", "never")) - 1.0) < 1e-9
    assert "mxfp8:" in str(rep) and "fp8" in str(rep)
    # a second pass finds the layers already converted and counts them the same way
    again = swap_mxfp8(dense)
    assert again.mac == rep.mac and len(again.modules) == len(rep.modules)
    # scope: everything outside it is 16-bit by choice
    dense2 = LMBackbone(get_preset("B200-smoke", vocab_size=512, dim=256, depth=2, heads=4, kv_heads=2, mlp_hidden=384))
    scoped = swap_mxfp8(dense2, scope=("attn",))
    assert all(".attn." in m for m in scoped.modules) and scoped.mac["never"] > 512 * 256
    # a refused layer (width not a multiple of 128) is 'skipped' and blocking
    odd = LMBackbone(get_preset("B200-smoke", vocab_size=512, dim=256, depth=1, heads=4, kv_heads=2, mlp_hidden=200))
    r3 = swap_mxfp8(odd)
    assert r3.blocking and r3.mac["skipped"] > 0
    # MoE: experts declared and converted at top_k per token; with convert_declared=False they are 'unreached'
    moe_cfg = dict(vocab_size=512, dim=128, depth=2, heads=2, kv_heads=1, mlp_hidden=256, moe_every=1, moe_first_dense=1,
                   moe_num_experts=4, moe_top_k=2, moe_num_shared=1, moe_hidden=128)
    moe = LMBackbone(get_preset("B200-smoke", **moe_cfg))
    r4 = swap_mxfp8(moe)
    assert any(d.endswith("w_in") for d in r4.declared) and not r4.unaccounted
    assert any("router" in b for b in r4.by_design)
    moe2 = LMBackbone(get_preset("B200-smoke", **moe_cfg))
    r5 = swap_mxfp8(moe2, convert_declared=False)
    assert r5.unreached and r5.mac["unreached"] == 2 * (2 * 128 * 128 + 128 * 128)
    # closing sweep: a bare matrix parameter that no rule knows about
    dense.blocks[0].extra_matrix = nn.Parameter(torch.zeros(64, 64))
    r6 = swap_mxfp8(dense)
    assert r6.unaccounted == ["blocks.0.extra_matrix(64, 64)"]


def test_blockwise_attention_fallback_matches_the_oracle_for_other_head_sizes():
    """Head sizes without a native kernel take a blockwise PyTorch path with recomputation: same outputs, lse and
    gradients as the full-matrix oracle, with windows and sinks, for blocks that do not divide the documents."""
    import torch

    from kohakuwullm_b200.models.seqinfo import SeqInfo
    from kohakuwullm_b200.ops.attention import varlen_attention, varlen_attention_blockwise, varlen_attention_reference

    torch.manual_seed(0)
    info = SeqInfo.from_lengths([70, 33, 129])
    T, Hq, Hkv, D = info.total_tokens, 4, 2, 128
    for window, sinks in ((None, False), (40, True)):
        q, k, v = (torch.randn(T, h, D, requires_grad=True) for h in (Hq, Hkv, Hkv))
        sink = torch.randn(Hq, requires_grad=True) if sinks else None
        ref, lse_r = varlen_attention_reference(q, k, v, info.cu_seqlens, window, sink, return_lse=True)
        g = torch.randn_like(ref)
        grads_r = torch.autograd.grad(ref, [q, k, v] + ([sink] if sinks else []), g)
        out, lse = varlen_attention_blockwise(q, k, v, info.cu_seqlens, window, sink, return_lse=True, block=48)
        grads = torch.autograd.grad(out, [q, k, v] + ([sink] if sinks else []), g)
        torch.testing.assert_close(out, ref, rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(lse, lse_r, rtol=1e-5, atol=1e-5)
        for a, b in zip(grads, grads_r):
            torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-5)
    assert torch.equal(varlen_attention(q, k, v, info.cu_seqlens, window=40, sink_lse=sink),
                       varlen_attention_blockwise(q, k, v, info.cu_seqlens, 40, sink))      # the public entry point uses it
