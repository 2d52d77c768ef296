"""Every registered component reaches a model through its config name, runs forward and backward on CPU, and does
what its name says: the routing variants, the latent-width experts, N-dimensional rotary encodings, the norm and MLP
kinds, per-layer attention backends."""

import pytest
import torch

import kohakuwullm_b200.models  # noqa: F401  (the import that must register every built-in component)
from kohakuwullm_b200.models import LMBackbone, get_preset
from kohakuwullm_b200.models.seqinfo import SeqInfo
from kohakuwullm_b200.registry import ATTENTION, MLP, NORM, POSENC, ROUTER

BASE = dict(vocab_size=128, dim=64, depth=2, heads=2, kv_heads=1, head_dim=32, mlp_hidden=128, init_std=0.1)
MOE = dict(moe_every=1, moe_num_experts=4, moe_top_k=2, moe_hidden=32)


def _step(cfg, seed=0):
    """One forward + backward on a packed batch of three documents; returns (loss, model)."""
    torch.manual_seed(seed)
    model = LMBackbone(cfg)
    info = SeqInfo.from_lengths([7, 12, 5])
    tokens = torch.randint(0, cfg.vocab_size, (24,))
    labels = torch.roll(tokens, -1)
    loss, _ = model.loss(tokens, labels, info, reduction="mean")
    loss.backward()
    return loss, model


def test_importing_the_package_registers_every_builtin_component():
    assert {"topk", "sinkhorn", "relu", "expert_choice"} <= set(ROUTER._table)
    assert {"swiglu", "geglu", "gelu", "moe", "latent_moe"} <= set(MLP._table)
    assert {"rmsnorm", "gemma_rmsnorm", "layernorm", "dyt"} <= set(NORM._table)
    assert {"rope", "none", "ndrope", "ggrope"} <= set(POSENC._table)
    assert {"flash", "sdpa", "mxfp8"} <= set(ATTENTION._table)


@pytest.mark.parametrize("overrides", [
    dict(norm="layernorm", mlp="gelu", posenc="none", tie_embeddings=True),
    dict(norm="gemma_rmsnorm", mlp="geglu", rope_scaling="ntk", rope_factor=2.0, rope_partial=0.5),
    dict(norm="dyt", rope_scaling="yarn", rope_factor=4.0, logit_soft_cap=30.0, z_loss_weight=1e-3),
    dict(attn="sdpa", sliding_window=4, global_layer_every=2, attn_sink=True, attn_num_sinks=2),
    dict(attn_sliding="sdpa", window_pattern=[4, None], attn_sink=True, qk_norm=False, attn_bias=True),
    dict(post_norm=True, scale_residual_by_depth=True, embedding_scale=True, grad_ckpt=True),
    dict(**MOE, moe_first_dense=1, moe_num_shared=2),
    dict(**MOE, moe_router_kwargs={"score": "softmax", "aux_loss_weight": 0.01, "z_loss_weight": 0.001}),
    dict(**MOE, moe_router_kwargs={"score": "sqrtsoftplus", "norm_topk_prob": False, "routed_scaling_factor": 2.0}),
    dict(**MOE, moe_router="sinkhorn"),
    dict(**MOE, moe_router="relu"),
    dict(**MOE, moe_mlp="latent_moe", moe_mlp_kwargs={"latent": 32}),
])
def test_every_component_kind_trains_one_step(overrides):
    cfg = get_preset("B200-smoke", **{**BASE, **overrides})
    loss, model = _step(cfg)
    assert torch.isfinite(loss) and 3.0 < float(loss.detach()) < 7.0
    grads = [p.grad for p in model.parameters() if p.requires_grad]
    missing = [n for n, p in model.named_parameters() if p.requires_grad and p.grad is None]
    assert not missing, missing
    assert all(torch.isfinite(g).all() for g in grads) and any(float(g.abs().sum()) > 0 for g in grads)


def test_expert_choice_router_is_registered_but_refuses_token_dispatch():
    cfg = get_preset("B200-smoke", **BASE, **MOE, moe_router="expert_choice")
    with pytest.raises(NotImplementedError):
        _step(cfg)
    router = ROUTER.get("expert_choice")(64, 4, 2, capacity_factor=1.0)
    torch.nn.init.normal_(router.weight, std=0.1)
    tok, w = router.choose(torch.randn(16, 64))
    assert tok.shape == w.shape == (4, 8) and bool((w >= 0).all())          # every expert takes its capacity


def test_sinkhorn_assignment_is_more_balanced_than_plain_topk():
    torch.manual_seed(0)
    x = torch.randn(512, 64)
    x[:, 0] = 4.0                                                          # a constant feature ...
    skew = torch.randn(8, 64) * 0.05
    skew[0, 0] = 0.5                                                       # ... that gives expert 0 a +2 head start everywhere
    counts = {}
    for name in ("topk", "sinkhorn"):
        router = ROUTER.get(name)(64, 8, 2, score="softmax")
        with torch.no_grad():
            router.weight.copy_(skew)
        router.train()
        _, w, c = router.route(x)
        counts[name] = c.float()
        assert int(c.sum()) == 512 * 2 and w.shape == (512, 2)
    spread = {k: float(v.max() / v.mean()) for k, v in counts.items()}
    assert spread["topk"] > 3.5 and spread["sinkhorn"] < 1.6, spread       # everyone picks expert 0 / close to uniform
    # logits far outside the comfortable range (hundreds of e-folds after the temperature) must not collapse it
    router = ROUTER.get("sinkhorn")(64, 8, 2)
    with torch.no_grad():
        router.weight.copy_(torch.randn(8, 64) * 3.0)
    _, _, c = router.route(torch.randn(512, 64))
    assert float(c.max()) < 2.5 * float(c.float().mean()), c


def test_sinkhorn_model_decodes_the_same_with_and_without_a_cache():
    """Balancing over the batch is a training-time rule; in evaluation each token routes on its own scores, so a
    cached decode (one token per step) and a recompute of the whole prefix agree token for token."""
    from kohakuwullm_b200.generation.engine import LocalGenerator

    torch.manual_seed(0)
    cfg = get_preset("B200-smoke", **{**BASE, **MOE, "moe_router": "sinkhorn", "vocab_size": 97, "init_std": 0.3})
    model = LMBackbone(cfg)
    prompt = torch.randint(0, 97, (3, 5))
    cached = LocalGenerator(model, eos_id=96, use_cache=True).generate(prompt, 10, temperature=0.0)
    plain = LocalGenerator(model, eos_id=96, use_cache=False).generate(prompt, 10, temperature=0.0)
    assert torch.equal(cached, plain) and len(set(cached[0, 5:].tolist())) > 1


def test_relu_router_steers_its_sparsity_coefficient_towards_the_target():
    torch.manual_seed(0)
    router = ROUTER.get("relu")(64, 8, 2, l1_init=1e-3, alpha=1.5)
    torch.nn.init.normal_(router.weight, std=0.2)
    router.train()
    idx, w, _ = router.route(torch.randn(256, 64))
    assert idx.shape == (256, 4) and bool((w >= 0).all()) and float((w == 0).float().mean()) > 0   # slots may be empty
    assert router.aux_loss is not None and float(router.aux_loss) > 0
    before = float(router.l1_coeff)
    active = float(router.active_accum[0] / router.active_accum[1])          # about half of 8 experts are active
    router.update_bias()
    after = float(router.l1_coeff)
    assert (after > before) == (active > 2) and abs(after / before - (1.5 if active > 2 else 1 / 1.5)) < 1e-5
    assert float(router.active_accum.sum()) == 0.0


def test_latent_experts_run_at_the_reduced_width_and_route_on_the_full_input():
    layer = MLP.get("latent_moe")(64, latent=16, num_experts=4, top_k=2, num_shared=1, hidden=32)
    assert layer.inner.w_in.shape == (4, 64, 16) and layer.inner.w_out.shape == (4, 16, 32)
    assert layer.router.weight.shape == (4, 64)                             # the router sees the 64-wide input
    assert layer.down.weight.shape == (16, 64) and layer.up.weight.shape == (64, 16)
    for p in layer.parameters():
        torch.nn.init.normal_(p, std=0.1)
    y = layer(torch.randn(2, 5, 64))
    assert y.shape == (2, 5, 64) and torch.isfinite(y).all()


def test_nd_rotary_encodings_rotate_by_position_vectors():
    from kohakuwullm_b200.models.components.ndrope import GGRoPE, NDRoPE

    rope = NDRoPE(head_dim=32, position_dim=2)
    pos = torch.tensor([[0.0, 0.0], [1.0, 0.0], [0.0, 1.0], [3.0, 2.0]])
    cos, sin = rope.prepare(pos)[:2]
    assert cos.shape == sin.shape and cos.shape[0] == 4
    assert torch.allclose(cos[0], torch.ones_like(cos[0])) and torch.allclose(sin[0], torch.zeros_like(sin[0]))
    assert not torch.allclose(cos[1], cos[2])                               # the two axes rotate differently
    # rotations compose: the angle at (3, 2) is 3 x the angle at (1, 0) plus 2 x the angle at (0, 1)
    ang = lambda i: torch.atan2(sin[i], cos[i])                              # noqa: E731
    want = 3 * ang(1) + 2 * ang(2)
    assert torch.allclose(torch.cos(ang(3)), torch.cos(want), atol=1e-5)
    learn = GGRoPE(head_dim=32, position_dim=2)
    assert any(p.requires_grad for p in learn.parameters())
