"""Optimizers on CPU: grouping rules, FusedAdamW == torch AdamW, stochastic rounding is unbiased and
matches its injected-draw reference, Newton-Schulz orthogonalises, low-bit casting keeps fp32 names."""

import torch

from kohakuwullm_b200.models import LMBackbone, get_preset
from kohakuwullm_b200.ops.optim import sr_cast, stochastic_round_reference
from kohakuwullm_b200.training.optim import (AdamW16, FusedAdamW, MuonW, StochasticAdamW, build_optimizer,
                                              cast_parameters_, group_parameters, newton_schulz)


def _tiny():
    torch.manual_seed(0)
    return LMBackbone(get_preset("B200-moe-991M", vocab_size=64, dim=32, depth=2, heads=2, kv_heads=1, head_dim=16,
                                 moe_num_experts=4, moe_top_k=2, moe_hidden=32, mlp_hidden=64, mxfp8=False))


def test_grouping_rules():
    model = _tiny()
    groups = group_parameters(model, weight_decay=0.1)
    decayed = {id(p) for g in groups if g["weight_decay"] > 0 for p in g["params"]}
    names = dict(model.named_parameters())
    assert id(names["embed.weight"]) not in decayed            # input embedding never decays by default
    assert id(names["blocks.0.attn.qkv_proj.weight"]) in decayed
    assert id(names["blocks.0.norm_attn.weight"]) not in decayed
    assert id(names["blocks.1.mlp.w_in"]) in decayed           # stacked experts are matrices
    with_embed = group_parameters(model, weight_decay=0.1, decay_embeddings=True)
    assert id(names["embed.weight"]) in {id(p) for g in with_embed if g["weight_decay"] > 0 for p in g["params"]}


def test_fused_adamw_matches_torch():
    torch.manual_seed(1)
    a = torch.nn.Linear(8, 8)
    b = torch.nn.Linear(8, 8)
    b.load_state_dict(a.state_dict())
    oa = torch.optim.AdamW(a.parameters(), lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1)
    ob = FusedAdamW(b.parameters(), lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1)
    for _ in range(3):
        x = torch.randn(4, 8)
        for m, o in ((a, oa), (b, ob)):
            o.zero_grad()
            m(x).pow(2).sum().backward()
            o.step()
    torch.testing.assert_close(a.weight, b.weight, rtol=1e-5, atol=1e-6)


def test_stochastic_rounding_reference_is_unbiased_and_exact():
    x = torch.full((200000,), 1.0 + 2 ** -10)       # between two bf16 values: 1.0 and 1.0078125
    draws = torch.randint(0, 1 << 16, x.shape, generator=torch.Generator().manual_seed(0))
    r = stochastic_round_reference(x, draws).float()
    assert set(r.unique().tolist()) == {1.0, 1.0078125}
    assert abs(r.mean().item() - x[0].item()) < 2e-5
    assert torch.equal(stochastic_round_reference(x, torch.zeros_like(draws)).float(), torch.ones_like(x))
    assert sr_cast(x, seed=3).dtype == torch.bfloat16


def test_newton_schulz_orthogonalises():
    torch.manual_seed(2)
    G = torch.randn(24, 40)
    X = newton_schulz(G, steps=8)
    s = torch.linalg.svdvals(X.float())
    assert s.max() < 1.3 and s.min() > 0.5


def test_low_bit_optimizers_step():
    for name in ("adamw16", "stochastic_adamw", "muon", "fused_adamw", "adamw"):
        model = _tiny()
        if name in ("adamw16", "stochastic_adamw"):
            cast_parameters_(model, torch.bfloat16)
            assert model.blocks[0].norm_attn.weight.dtype == torch.float32      # norms stay fp32
            assert model.blocks[0].attn.qkv_proj.weight.dtype == torch.bfloat16
        opt = build_optimizer(model, name=name, lr=1e-3)
        before = model.blocks[0].attn.o_proj.weight.detach().float().clone()
        x = torch.randint(0, 64, (16,))
        from kohakuwullm_b200.models import SeqInfo

        loss, _ = model.loss(x, x, SeqInfo.from_lengths([16]))
        loss.backward()
        opt.step()
        assert not torch.equal(before, model.blocks[0].attn.o_proj.weight.detach().float()), name
