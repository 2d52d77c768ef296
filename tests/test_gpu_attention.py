"""tcgen05 flash attention (fwd + bwd) against the fp32 per-document reference."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _make(lengths, Hq, Hkv, seed=0, fused_qkv=False):
    from kohakuwullm_b200.models.seqinfo import SeqInfo

    g = torch.Generator(device="cuda").manual_seed(seed)
    info = SeqInfo.from_lengths(lengths, device="cuda")
    T = info.total_tokens
    if fused_qkv:
        qkv = torch.randn(T, (Hq + 2 * Hkv) * 64, device="cuda", generator=g).to(torch.bfloat16)
        q = qkv[:, : Hq * 64].view(T, Hq, 64)
        k = qkv[:, Hq * 64:(Hq + Hkv) * 64].view(T, Hkv, 64)
        v = qkv[:, (Hq + Hkv) * 64:].view(T, Hkv, 64)
    else:
        q = torch.randn(T, Hq, 64, device="cuda", generator=g).to(torch.bfloat16)
        k = torch.randn(T, Hkv, 64, device="cuda", generator=g).to(torch.bfloat16)
        v = torch.randn(T, Hkv, 64, device="cuda", generator=g).to(torch.bfloat16)
    do = torch.randn(T, Hq, 64, device="cuda", generator=g).to(torch.bfloat16)
    return info, q, k, v, do


CASES = [
    ([128], 1, 1, None, False),
    ([256], 2, 1, None, False),
    ([64, 200, 37, 515], 4, 2, None, False),
    ([300, 1000, 77], 5, 1, None, True),
    ([700, 33, 291], 4, 2, 128, False),
    ([1500, 548], 6, 2, 100, True),
    ([640], 2, 2, 1024, False),
]


@pytest.mark.parametrize("lengths,Hq,Hkv,window,sinks", CASES)
def test_flash_fwd_bwd_matches_reference(lengths, Hq, Hkv, window, sinks):
    from kohakuwullm_b200.ops import native
    from kohakuwullm_b200.ops.attention import varlen_attention, varlen_attention_reference

    info, q, k, v, do = _make(lengths, Hq, Hkv, fused_qkv=(len(lengths) == 3))
    sink = torch.randn(Hq, device="cuda") if sinks else None

    qa, ka, va = (t.detach().clone().requires_grad_() for t in (q, k, v))
    sa = sink.clone().requires_grad_() if sinks else None
    out, lse = varlen_attention(qa, ka, va, info.cu_seqlens, window=window, sink_lse=sa, return_lse=True)
    out.backward(do)
    torch.cuda.synchronize()
    native.check_status()

    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    sr = sink.clone().requires_grad_() if sinks else None
    ref, lse_r = varlen_attention_reference(qr, kr, vr, info.cu_seqlens, window=window, sink_lse=sr, return_lse=True)
    ref.backward(do.float())

    def close(got, want, tol, name):
        err = (got.float() - want.float()).abs().max().item()
        scale = max(want.float().abs().max().item(), 1e-6)
        assert err <= tol * scale, f"{name}: max err {err} scale {scale}"

    close(out, ref, 2e-2, "out")
    close(lse, lse_r, 1e-3, "lse")
    close(qa.grad, qr.grad, 3e-2, "dq")
    close(ka.grad, kr.grad, 3e-2, "dk")
    close(va.grad, vr.grad, 3e-2, "dv")
    if sinks:
        close(sa.grad, sr.grad, 3e-2, "dsink")


def test_attention_plan_lists_are_complete_and_sorted():
    from kohakuwullm_b200.models.seqinfo import SeqInfo
    from kohakuwullm_b200.ops.attention import attention_plan

    lengths = [300, 1000, 77, 64, 2655, 128, 1]
    info = SeqInfo.from_lengths(lengths, device="cuda")
    plan = attention_plan(info.cu_seqlens, info.total_tokens).cpu()
    n = plan.shape[0] // 2
    expect, start = set(), 0
    for ln in lengths:
        expect |= {(q0, start, start + ln) for q0 in range(start, start + ln, 128)}
        start += ln
    for half, cost in ((plan[:n], lambda r: min(r[0] + 128, r[2]) - r[1]), (plan[n:], lambda r: r[2] - r[0])):
        rows = half.tolist()
        valid = [r for r in rows if r[3] == 1]
        assert {tuple(r[:3]) for r in valid} == expect and len(valid) == len(expect)
        assert all(r[3] == 1 for r in rows[:len(valid)])          # unused entries come last
        costs = [cost(r) for r in valid]
        assert costs == sorted(costs, reverse=True)


def test_packed_attention_does_not_cross_documents():
    """Changing one document must leave every other document's output bit-identical."""
    from kohakuwullm_b200.ops.attention import varlen_attention

    info, q, k, v, _ = _make([200, 300, 150], 4, 2, seed=5)
    out1 = varlen_attention(q, k, v, info.cu_seqlens)
    k2, v2 = k.clone(), v.clone()
    k2[200:500] = torch.randn_like(k2[200:500])
    v2[200:500] = torch.randn_like(v2[200:500])
    out2 = varlen_attention(q, k2, v2, info.cu_seqlens)
    assert torch.equal(out1[:200], out2[:200])
    assert torch.equal(out1[500:], out2[500:])
    assert not torch.equal(out1[200:500], out2[200:500])


def test_attention_layer_fused_core_matches_unfused():
    """The fused QK-norm + RoPE + flash node must give the same output and gradients as the
    composition of the separate ops (which are tested against fp32 references above)."""
    from kohakuwullm_b200.models.components.attention import Attention, SDPAAttention
    from kohakuwullm_b200.models.components.posenc import RoPE
    from kohakuwullm_b200.models.seqinfo import SeqInfo

    torch.manual_seed(0)
    info = SeqInfo.from_lengths([300, 212], device="cuda")
    T = info.total_tokens
    kw = dict(dim=256, heads=4, kv_heads=2, head_dim=64, window=100, sink=True, num_sinks=2)
    a = Attention(**kw).cuda()
    b = SDPAAttention(**kw).cuda()
    for p in a.parameters():
        if p.dim() >= 2:
            torch.nn.init.normal_(p, std=0.05)
    b.load_state_dict(a.state_dict())
    for m in (a, b):
        for n, p in m.named_parameters():
            if p.dim() >= 2 and "sink" not in n:
                p.data = p.data.to(torch.bfloat16)
    rope = RoPE(64).cuda().prepare(info.position_ids)
    x = torch.randn(T, 256, device="cuda", dtype=torch.bfloat16)
    dy = torch.randn(T, 256, device="cuda", dtype=torch.bfloat16)
    outs = []
    for m in (a, b):
        xi = x.clone().requires_grad_()
        y = m(xi, info, rope)
        y.backward(dy)
        outs.append((y, xi.grad, m.qkv_proj.weight.grad, m.sink.grad, m.q_norm.grad))
    for got, want in zip(*outs):
        err = (got.float() - want.float()).abs().max().item()
        scale = max(want.float().abs().max().item(), 1e-6)
        assert err <= 4e-2 * scale, f"err {err} scale {scale}"


@pytest.mark.parametrize("B,H,Hkv,L,kv_len,window,n_sinks", [
    (2, 8, 2, 512, 300, None, 0),
    (3, 20, 4, 2048, 2048, 1024, 4),
    (1, 16, 16, 1024, 1, None, 1),
    (4, 24, 8, 4096, 3333, 1024, 0),
])
def test_decode_attention_matches_reference(B, H, Hkv, L, kv_len, window, n_sinks):
    from kohakuwullm_b200.ops.attention import decode_attention

    torch.manual_seed(kv_len)
    D = 64
    q = torch.randn(B, H, D, device="cuda", dtype=torch.bfloat16)
    kc = torch.randn(B, L, Hkv, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.randn(B, L, Hkv, D, device="cuda", dtype=torch.bfloat16)
    sink = torch.randn(H, n_sinks, device="cuda") if n_sinks else None
    out, lse = decode_attention(q, kc, vc, kv_len, window, None, sink, return_lse=True)
    lo = max(0, kv_len - window) if window else 0
    g = H // Hkv
    kf = kc[:, lo:kv_len].float().repeat_interleave(g, 2)            # (B, n, H, D)
    vf = vc[:, lo:kv_len].float().repeat_interleave(g, 2)
    s = torch.einsum("bhd,bnhd->bhn", q.float(), kf) * D ** -0.5
    ref_lse = torch.logsumexp(s, -1)
    if sink is not None:
        ref_lse = torch.logaddexp(ref_lse, torch.logsumexp(sink, -1)[None])
    p = torch.exp(s - ref_lse[..., None])
    ref = torch.einsum("bhn,bnhd->bhd", p, vf)
    torch.testing.assert_close(lse, ref_lse, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-2)


def test_cached_decode_step_matches_uncached_forward():
    """Prefill + one cached decode step (split-KV kernel, window and sinks on) against the full forward."""
    from kohakuwullm_b200.models import LMBackbone, get_preset
    from kohakuwullm_b200.models.cache import KVCache
    from kohakuwullm_b200.models.seqinfo import SeqInfo
    from kohakuwullm_b200.ops import native

    torch.manual_seed(0)
    cfg = get_preset("B200-smoke", vocab_size=512, sliding_window=16, global_layer_every=2, attn_sink=True,
                     attn_num_sinks=2)
    with torch.device("cuda"):
        model = LMBackbone(cfg).to(torch.bfloat16).eval()
    for blk in model.blocks:
        torch.nn.init.normal_(blk.attn.sink, std=1.0)
    tokens = torch.randint(0, 512, (3, 41), device="cuda")
    with torch.no_grad():
        full = model(tokens, SeqInfo.padded(3, 41, device="cuda"))
        cache = KVCache.from_config(cfg, 64, static=True)
        model(tokens[:, :40], cache.seq_info(tokens[:, :40]), cache=cache)
        before = native.lib().kwu_launch_count()
        last = model(tokens[:, 40:], cache.seq_info(tokens[:, 40:]), cache=cache)
        launched = native.lib().kwu_launch_count() - before
    assert launched >= 2 * cfg.depth, "the decode step did not go through the native decode kernels"
    torch.testing.assert_close(last[:, 0].float(), full[:, 40].float(), rtol=5e-2, atol=5e-2)


def test_mxfp8_head_quantisation_matches_reference_and_attention_runs():
    from kohakuwullm_b200.ops.attention import quantize_heads, quantize_heads_reference, varlen_attention

    torch.manual_seed(1)
    T, H, Hkv, D = 1000, 8, 2, 64
    q = (torch.randn(T, H, D, device="cuda") * 3).bfloat16().requires_grad_()
    k = (torch.randn(T, Hkv, D, device="cuda") + 2.0).bfloat16().requires_grad_()     # a visible channel mean
    v = torch.randn(T, Hkv, D, device="cuda").bfloat16()
    qq, kq = quantize_heads(q), quantize_heads(k, smooth=True)
    assert torch.equal(qq, quantize_heads_reference(q.detach()))
    # the mean is taken in fp32 over bf16 inputs by both; compare the smoothed copy loosely at block edges
    ref_k = quantize_heads_reference(k.detach(), smooth=True)
    assert (kq.float() - ref_k.float()).abs().max() <= 0.26 * ref_k.float().abs().max() / 8   # within one e4m3 step
    assert (kq != ref_k).float().mean() < 0.02
    cu = torch.tensor([0, 300, 1000], dtype=torch.int32, device="cuda")
    out = varlen_attention(qq, kq, v, cu, 700)
    ref = varlen_attention(q.detach(), k.detach(), v, cu, 700)
    rel = (out.float() - ref.float()).norm() / ref.float().norm()
    assert rel < 0.08, rel            # fp8 operands: a few percent, not garbage
    out.sum().backward()
    assert q.grad is not None and k.grad is not None
    assert k.grad.float().mean(0).abs().max() < 1e-2 * k.grad.float().abs().max() + 1e-3   # mean-free gradient


def test_mxfp8_attention_backend_trains():
    from kohakuwullm_b200.data.synthetic import make_packs
    from kohakuwullm_b200.models import LMBackbone, get_preset
    from kohakuwullm_b200.training.engine import TrainEngine

    torch.manual_seed(0)
    cfg = get_preset("B200-sliding-1B", depth=4, vocab_size=4096, dim=512, heads=8, kv_heads=4, mlp_hidden=1024,
                     attn="mxfp8", sliding_window=256)
    with torch.device("cuda"):
        model = LMBackbone(cfg)
    assert type(model.blocks[0].attn).__name__ == "MXFP8Attention"
    eng = TrainEngine(model, lr=1e-3, param_dtype=torch.bfloat16, cuda_graphs=False)
    packs = make_packs(2, 2048, 64, 1024, cfg.vocab_size, seed=3)
    losses = [float(eng.step(packs)["loss"]) for _ in range(6)]
    assert all(l == l for l in losses) and losses[-1] < losses[0]


@pytest.mark.parametrize("rotary", [True, False])
def test_fused_qk_norm_rope_matches_per_tensor_kernels_and_emits_fp8(rotary):
    """q and k heads handled by one launch give bit-identical outputs to the two per-tensor launches, forward and
    backward, and the MXFP8 copy of d(qkv) written by the backward equals quantising the stored gradient."""
    import ctypes

    from kohakuwullm_b200.ops import mxfp8 as mx
    from kohakuwullm_b200.ops import native

    torch.manual_seed(3)
    L = native.require()
    ci, cf = ctypes.c_int, ctypes.c_float
    T, Hq, Hkv, D = 384, 20, 4, 64
    cols = (Hq + 2 * Hkv) * D
    qkv = torch.randn(T, cols, device="cuda").bfloat16()
    wq = torch.rand(D, device="cuda") + 0.5
    wk = torch.rand(D, device="cuda") + 0.5
    ang = torch.rand(T, 32, device="cuda") * 6.28
    cos, sin = (ang.cos().contiguous(), ang.sin().contiguous()) if rotary else (None, None)
    rot = 32 if rotary else 0
    st = native.stream_ptr()
    # forward
    q1 = torch.empty(T, Hq, D, device="cuda", dtype=torch.bfloat16)
    k1 = torch.empty(T, Hkv, D, device="cuda", dtype=torch.bfloat16)
    q2, k2 = torch.empty_like(q1), torch.empty_like(k1)
    for src, dst, w, H in ((qkv[:, :Hq * D], q1, wq, Hq), (qkv[:, Hq * D:(Hq + Hkv) * D], k1, wk, Hkv)):
        native.check(L.kwu_qknorm_rope_fwd(native.ptr(src), ci(cols), native.ptr(dst), ci(H * D), native.ptr(w),
                                           native.ptr(cos), native.ptr(sin), ci(T), ci(H), ci(D), ci(rot), cf(1e-6),
                                           ci(1), st), "fwd")
    native.check(L.kwu_qknorm_rope_fwd_qk(native.ptr(qkv), ci(cols), native.ptr(q2), native.ptr(k2), native.ptr(wq),
                                          native.ptr(wk), native.ptr(cos), native.ptr(sin), ci(T), ci(Hq), ci(Hkv),
                                          ci(rot), cf(1e-6), ci(1), st), "fwd_qk")
    assert torch.equal(q1, q2) and torch.equal(k1, k2)
    # backward
    dq = torch.randn(T, Hq, D, device="cuda").bfloat16()
    dk = torch.randn(T, Hkv, D, device="cuda").bfloat16()
    dv = torch.randn(T, Hkv * D, device="cuda").bfloat16()
    d1 = torch.zeros(T, cols, device="cuda", dtype=torch.bfloat16)
    d1[:, (Hq + Hkv) * D:] = dv
    d2 = d1.clone()
    dw1 = [torch.zeros(D, device="cuda"), torch.zeros(D, device="cuda")]
    dw2 = [torch.zeros(D, device="cuda"), torch.zeros(D, device="cuda")]
    for src, g, dst, w, H, dw in ((qkv[:, :Hq * D], dq, d1[:, :Hq * D], wq, Hq, dw1[0]),
                                  (qkv[:, Hq * D:(Hq + Hkv) * D], dk, d1[:, Hq * D:(Hq + Hkv) * D], wk, Hkv, dw1[1])):
        native.check(L.kwu_qknorm_rope_bwd(native.ptr(src), ci(cols), native.ptr(g), ci(H * D), native.ptr(dst), ci(cols),
                                           native.ptr(w), native.ptr(dw), native.ptr(cos), native.ptr(sin), ci(T), ci(H),
                                           ci(D), ci(rot), cf(1e-6), ci(1), st), "bwd")
    q8, sf = mx.alloc_quantized(T, cols, "cuda")
    native.check(L.kwu_qknorm_rope_bwd_qk(native.ptr(qkv), ci(cols), native.ptr(dq), native.ptr(dk), native.ptr(d2),
                                          ci(cols), native.ptr(wq), native.ptr(wk), native.ptr(dw2[0]), native.ptr(dw2[1]),
                                          native.ptr(cos), native.ptr(sin), ci(T), ci(Hq), ci(Hkv), ci(rot), cf(1e-6),
                                          ci(1), native.ptr(q8), ci(cols), native.ptr(sf), st), "bwd_qk")
    assert torch.equal(d1, d2)
    for a, b in zip(dw1, dw2):
        torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-3)   # fp32 atomics in a different order
    q_ref, sf_ref = mx.quantize(d2)
    assert torch.equal(q8, q_ref) and torch.equal(sf, sf_ref)
    native.check_status()


def test_flash_forward_fp8_copy_of_output_equals_the_quantise_kernel():
    """The forward epilogue's MXFP8 copy of the attention output (for an MXFP8 output projection) is bit-identical
    to quantising the stored bf16 output, on a pack with ragged documents (every token lies in one query tile)."""
    from kohakuwullm_b200.models.seqinfo import SeqInfo
    from kohakuwullm_b200.ops import mxfp8 as mx
    from kohakuwullm_b200.ops import native
    from kohakuwullm_b200.ops.attention import attention_core

    torch.manual_seed(11)
    Hq, Hkv, D = 20, 4, 64
    info = SeqInfo.from_lengths([300, 77, 500, 147], device="cuda")   # 1024 tokens
    T = info.total_tokens
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda").bfloat16()
    wq = torch.ones(D, device="cuda")
    mx.clear_prequantized()
    out = attention_core(qkv, wq, wq, None, None, info.cu_seqlens, None, None, Hq, Hkv, None, 0.125, 1e-6, True,
                         emit_mx_out=True)
    out2d = out.reshape(T, Hq * D)
    got = mx.take_quantized(out2d)
    assert got is not None
    q_ref, sf_ref = mx.quantize(out2d.contiguous())
    assert torch.equal(got[0], q_ref) and torch.equal(got[1], sf_ref)
    plain = attention_core(qkv, wq, wq, None, None, info.cu_seqlens, None, None, Hq, Hkv, None, 0.125, 1e-6, True)
    assert torch.equal(plain, out)
    native.check_status()
