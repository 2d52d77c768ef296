"""Optimizers on CPU: grouping rules, FusedAdamW == torch AdamW, stochastic rounding is unbiased and
matches its injected-draw reference, Newton-Schulz orthogonalises, low-bit casting keeps fp32 names."""

import pytest
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


def test_sharded_flat_adamw_covers_every_element_for_any_world_size():
    """ZeRO-style shard bounds: for world sizes that do not divide the padded buffer length (3, 5, 6, 7) the
    shards are still multiples of 8 elements, disjoint, and together cover the whole buffer."""
    import torch

    from kohakuwullm_b200.parallel.flat import FlatParameters
    from kohakuwullm_b200.training.optim.fused_adamw import FlatAdamW

    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(40, 56), torch.nn.Linear(56, 24))
    for world in (1, 2, 3, 5, 6, 7, 8):
        flat = FlatParameters(model, install_hooks=False)
        covered = {k: torch.zeros(g.total, dtype=torch.int32) for k, g in flat.groups.items()}
        for rank in range(world):
            opt = FlatAdamW(flat, shard=(rank, world))
            for k, g in flat.groups.items():
                lo, hi = opt._range(g)
                assert lo % 8 == 0 and (hi - lo) % 8 == 0 and 0 <= lo <= hi <= g.total
                assert opt.state[k]["exp_avg"].numel() == hi - lo
                covered[k][lo:hi] += 1
        for k, c in covered.items():
            assert bool((c == 1).all()), (world, k)


def test_muon_newton_schulz_variants_orthogonalise_and_gram_phases_equal_direct_steps():
    import torch

    from kohakuwullm_b200.training.optim.muon import (PHASES_DIRECT, PHASES_GRAM, newton_schulz,
                                                      newton_schulz_cubic)

    torch.manual_seed(0)
    g = torch.randn(3, 48, 160)           # a batch of wide matrices
    direct = newton_schulz_cubic(g, torch.float32, phases=PHASES_DIRECT)
    gram = newton_schulz_cubic(g, torch.float32, phases=PHASES_GRAM)
    torch.testing.assert_close(gram, direct, rtol=1e-3, atol=1e-3)      # the same iteration, regrouped
    for out in (direct, newton_schulz(g, 5, torch.float32)):
        sv = torch.linalg.svdvals(out)
        assert sv.min() > 0.3 and sv.max() < 1.3                       # singular values pulled towards 1
    tall = torch.randn(160, 48)
    out = newton_schulz_cubic(tall, torch.float32)
    assert out.shape == tall.shape
    torch.testing.assert_close(out, newton_schulz_cubic(tall.t().contiguous(), torch.float32).t(), rtol=1e-4, atol=1e-4)
    # batched == one matrix at a time
    single = torch.stack([newton_schulz_cubic(m, torch.float32) for m in g])
    torch.testing.assert_close(direct, single, rtol=1e-4, atol=1e-4)


def test_muonw_batches_by_shape_picks_phases_and_trains():
    import torch

    from kohakuwullm_b200.training.optim.muon import PHASES_DIRECT, PHASES_GRAM, MuonW

    torch.manual_seed(1)
    layers = torch.nn.ModuleList([torch.nn.Linear(32, 32, bias=False) for _ in range(3)]
                                 + [torch.nn.Linear(32, 96, bias=False), torch.nn.Linear(96, 8, bias=True)])
    hidden = [layers[i].weight for i in range(4)]
    rest = [{"params": [layers[4].weight], "weight_decay": 0.1}, {"params": [layers[4].bias], "weight_decay": 0.0}]
    opt = MuonW(hidden, rest, lr=1e-2, muon_lr=0.05, ns_batch_elems=2 * 32 * 32)   # two 32x32 matrices per batch
    assert opt.phases_for((32, 32)) == PHASES_DIRECT and opt.phases_for((96, 32)) == PHASES_GRAM
    assert opt._batch_size((32, 32)) == 2
    x, y = torch.randn(64, 32), torch.randn(64, 8)

    def loss_fn():
        h = x
        for i in range(3):
            h = torch.tanh(layers[i](h))
        return ((layers[4](torch.tanh(layers[3](h))) - y) ** 2).mean()

    first = float(loss_fn())
    for _ in range(30):
        opt.zero_grad()
        loss = loss_fn()
        loss.backward()
        opt.step()
    assert float(loss_fn()) < 0.7 * first
    assert "momentum_buffer" in opt.state[hidden[0]] and "exp_avg_rms" in opt.state[layers[4].weight]
    # the same run with one matrix per batch gives the same weights: batching does not change the result
    torch.manual_seed(1)
    layers2 = torch.nn.ModuleList([torch.nn.Linear(32, 32, bias=False) for _ in range(3)]
                                  + [torch.nn.Linear(32, 96, bias=False), torch.nn.Linear(96, 8, bias=True)])
    opt2 = MuonW([layers2[i].weight for i in range(4)],
                 [{"params": [layers2[4].weight], "weight_decay": 0.1}, {"params": [layers2[4].bias]}],
                 lr=1e-2, muon_lr=0.05, ns_batch_elems=1)
    h = x
    for i in range(3):
        h = torch.tanh(layers2[i](h))
    ((layers2[4](torch.tanh(layers2[3](h))) - y) ** 2).mean().backward()
    opt2.step()
    torch.manual_seed(1)
    layers3 = torch.nn.ModuleList([torch.nn.Linear(32, 32, bias=False) for _ in range(3)]
                                  + [torch.nn.Linear(32, 96, bias=False), torch.nn.Linear(96, 8, bias=True)])
    opt3 = MuonW([layers3[i].weight for i in range(4)],
                 [{"params": [layers3[4].weight], "weight_decay": 0.1}, {"params": [layers3[4].bias]}],
                 lr=1e-2, muon_lr=0.05)
    h = x
    for i in range(3):
        h = torch.tanh(layers3[i](h))
    ((layers3[4](torch.tanh(layers3[3](h))) - y) ** 2).mean().backward()
    opt3.step()
    for a, b in zip(layers2.parameters(), layers3.parameters()):
        torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("name,rel", [("adamw8bit", 0.05), ("adamwfp8", 0.08), ("adamw4bit", 0.35)])
def test_quantized_state_adamw_tracks_fp32_adamw(name, rel):
    """The three quantised-moment AdamW variants against torch AdamW on a least-squares problem: the same
    loss curve within a tolerance that widens with the coarser state, and the moments really are small."""
    import torch
    from kohakuwullm_b200.registry import OPTIMIZER
    from kohakuwullm_b200.training.optim import build  # noqa: F401  registers the names
    from kohakuwullm_b200.training.optim.quantized_state import dequantize_blocks, quantize_blocks

    torch.manual_seed(0)
    X, W_true = torch.randn(512, 96), torch.randn(96, 64)
    Y = X @ W_true

    def run(make):
        torch.manual_seed(1)
        w = torch.nn.Parameter(torch.zeros(96, 64))
        b = torch.nn.Parameter(torch.zeros(64))
        opt = make([{"params": [w], "weight_decay": 0.01}, {"params": [b], "weight_decay": 0.0}])
        losses = []
        for _ in range(200):
            loss = ((X @ w + b - Y) ** 2).mean()
            opt.zero_grad()
            loss.backward()
            opt.step()
            losses.append(float(loss))
        return losses, opt

    ref, _ = run(lambda g: torch.optim.AdamW(g, lr=2e-2, betas=(0.9, 0.95)))
    got, opt = run(lambda g: OPTIMIZER.get(name)(g, lr=2e-2, betas=(0.9, 0.95)))
    assert got[-1] < 0.2 * got[0]
    assert abs(got[-1] - ref[-1]) <= rel * ref[0] * 0.05 + rel * ref[-1], (name, got[-1], ref[-1])
    full = 2 * 4 * (96 * 64 + 64)
    assert opt.state_bytes() < (0.32 if name != "adamw4bit" else 0.2) * full + 2 * 4 * 64   # the bias keeps fp32 moments
    # round trip of the block codecs: relative error bounded by the code spacing
    x = torch.randn(1000) * torch.logspace(-3, 0, 1000)
    for fmt, tol in (("int8", 0.03), ("fp8", 0.07), ("int4", 0.4)):
        block = 128 if fmt == "int4" else 256
        back = dequantize_blocks(quantize_blocks(x, fmt, block, True), fmt, block, True, x.shape)
        assert float((back - x).norm() / x.norm()) < tol, fmt


def test_muon_embed_lr_puts_the_token_tables_in_their_own_group():
    from kohakuwullm_b200.models import LMBackbone, get_preset
    from kohakuwullm_b200.training.optim.build import build_optimizer

    cfg = get_preset("B200-smoke", vocab_size=64, dim=64, depth=1, heads=2, kv_heads=2, head_dim=32, mlp_hidden=128)
    model = LMBackbone(cfg)
    names = {id(p): n for n, p in model.named_parameters()}
    opt = build_optimizer(model, "muon", lr=5e-4, muon_lr=2e-3, embed_lr=1e-3)
    tables = [g for g in opt.param_groups if not g["use_muon"] and g["lr"] == 1e-3]
    assert len(tables) == 1 and sorted(names[id(p)] for p in tables[0]["params"]) == ["embed.weight", "head.proj.weight"]
    assert tables[0]["weight_decay"] == 0.0
    seen = [id(p) for g in opt.param_groups for p in g["params"]]
    assert len(seen) == len(set(seen)) == len(list(model.parameters()))       # every parameter in exactly one group
    plain = build_optimizer(model, "muon", lr=5e-4, muon_lr=2e-3)
    assert all(g["lr"] in (5e-4, 2e-3) for g in plain.param_groups)
