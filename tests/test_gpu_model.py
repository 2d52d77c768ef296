"""Whole-model gradients of the native path (flat buffers, fused weight gradients, every kernel in the
chain) against the same model evaluated in fp32 on the CPU with the PyTorch fallbacks."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _grads_native(cfg, packs, seed):
    from kohakuwullm_b200.models import LMBackbone
    from kohakuwullm_b200.ops import native
    from kohakuwullm_b200.training.engine import TrainEngine

    torch.manual_seed(seed)
    with torch.device("cuda"):
        model = LMBackbone(cfg)
    eng = TrainEngine(model, lr=1e-3, param_dtype=torch.bfloat16, cuda_graphs=False)
    model.train()
    weights = {n: p.detach().float().cpu() for n, p in model.named_parameters()}
    total = 0.0
    for mb in packs:
        mb = mb.to("cuda")
        loss, _ = model.loss(mb.tokens, mb.labels, mb.seq_info, reduction="sum", router_scale=eng._router_scale)
        loss.backward()
        total += float(loss.detach())
    torch.cuda.synchronize()
    native.check_status()
    grads = {n: p.main_grad.detach().float().cpu().clone() for n, p in model.named_parameters()}
    return weights, grads, total


def _grads_cpu(cfg, packs, weights):
    from kohakuwullm_b200.models import LMBackbone

    model = LMBackbone(cfg).float()
    with torch.no_grad():
        for n, p in model.named_parameters():
            p.copy_(weights[n])
    model.train()
    total = 0.0
    for mb in packs:
        loss, _ = model.loss(mb.tokens, mb.labels, mb.seq_info, reduction="sum")
        loss.backward()
        total += float(loss.detach())
    return {n: p.grad.detach().float().clone() for n, p in model.named_parameters()}, total


# MXFP8: every product carries ~5 % relative rounding noise (e4m3 operands), and the gradient of an early
# parameter has passed through about eight of them: the bound is on noise of that size, and on direction
@pytest.mark.parametrize("mxfp8,tol", [(False, 0.05), (True, 0.30)])
def test_whole_model_gradients_match_the_fp32_cpu_model(mxfp8, tol):
    from kohakuwullm_b200.data.synthetic import make_packs
    from kohakuwullm_b200.models import get_preset

    cfg = get_preset("B200-dense-546M", depth=2, vocab_size=4096, mxfp8=mxfp8)
    packs = make_packs(2, 1024, 64, 700, cfg.vocab_size, seed=21)
    weights, got, loss_gpu = _grads_native(cfg, packs, seed=0)
    cfg_cpu = get_preset("B200-dense-546M", depth=2, vocab_size=4096, mxfp8=False)
    want, loss_cpu = _grads_cpu(cfg_cpu, packs, weights)
    assert abs(loss_gpu - loss_cpu) <= 2e-2 * abs(loss_cpu), (loss_gpu, loss_cpu)
    worst = {}
    for n, g in want.items():
        rel = ((got[n] - g).norm() / g.norm().clamp(min=1e-12)).item()
        worst[n] = rel
        cos = torch.nn.functional.cosine_similarity(got[n].flatten(), g.flatten(), dim=0).item()
        assert cos > 0.95, f"{n}: gradient direction off (cosine {cos})"
    bad = {n: r for n, r in worst.items() if r > tol}
    assert not bad, f"gradients off: {sorted(bad.items(), key=lambda kv: -kv[1])[:6]}"


def test_whole_moe_model_gradients_match_the_fp32_cpu_model():
    """Same for a sparse model (router, dispatch, grouped expert products, combine). Near-tied router scores
    may pick other experts in bf16 than in fp32, so the bound is on direction and on gross size only."""
    from kohakuwullm_b200.data.synthetic import make_packs
    from kohakuwullm_b200.models import get_preset

    cfg = get_preset("B200-moe-991M", depth=2, vocab_size=4096, mxfp8=False)
    packs = make_packs(2, 1024, 64, 700, cfg.vocab_size, seed=22)
    weights, got, loss_gpu = _grads_native(cfg, packs, seed=1)
    want, loss_cpu = _grads_cpu(cfg, packs, weights)
    assert abs(loss_gpu - loss_cpu) <= 2e-2 * abs(loss_cpu), (loss_gpu, loss_cpu)
    report = {}
    for n, g in want.items():
        if g.norm() == 0:
            continue
        rel = ((got[n] - g).norm() / g.norm()).item()
        cos = torch.nn.functional.cosine_similarity(got[n].flatten(), g.flatten(), dim=0).item()
        report[n] = (round(rel, 3), round(cos, 4))
    bad = {n: v for n, v in report.items() if v[1] < 0.9 or v[0] > 0.5}
    assert not bad, f"gradients off (relative error, cosine): {sorted(bad.items(), key=lambda kv: kv[1][1])[:6]}"


def test_graph_replay_with_varying_micro_batch_sizes_matches_eager():
    """Document-aligned splits give micro-batches of a different token count almost every step. The graphed
    engine pads each one to its token bucket with a masked filler document, keeps a bounded number of graphs
    (here two, so buckets are evicted and captured again) and gives every graph its own loss scratch: replaying
    a small graph after a larger one must train exactly like the eager engine."""
    from kohakuwullm_b200.data.synthetic import make_pack
    from kohakuwullm_b200.models import LMBackbone, get_preset
    from kohakuwullm_b200.ops import native
    from kohakuwullm_b200.training.engine import TrainEngine

    cfg = get_preset("B200-smoke", depth=2, vocab_size=2048)
    sizes = [(2048, 1400), (900, 2048), (1400, 640), (2048, 900), (640, 1400), (1100, 2048)]
    steps = [[make_pack(n, 32, 512, cfg.vocab_size, seed=100 * s + i).to("cuda") for i, n in enumerate(pair)]
             for s, pair in enumerate(sizes)]
    results = {}
    for graphs in (False, True):
        torch.manual_seed(11)
        with torch.device("cuda"):
            model = LMBackbone(cfg)
        start = {n: p.detach().float().clone() for n, p in model.named_parameters()}
        eng = TrainEngine(model, lr=1e-3, param_dtype=torch.bfloat16, cuda_graphs=graphs,
                          **({"graph_token_bucket": 512, "graph_cache_size": 2} if graphs else {}))
        losses = [float(eng.step(packs)["loss"]) for packs in steps]
        torch.cuda.synchronize()
        native.check_status()
        results[graphs] = (losses, {n: p.detach().float().clone() for n, p in model.named_parameters()})
        if graphs:
            assert len(eng._graphs) <= 2
    (le, pe), (lg, pg) = results[False], results[True]
    for a, b in zip(le, lg):
        assert abs(a - b) < 2e-3 * max(abs(a), 1.0), (le, lg)
    # AdamW turns a gradient element that is noise around zero into a full +-lr step, so single elements may
    # differ by several lr between two correct runs (the padded GEMMs sum in another order); the UPDATE as a
    # whole must agree: relative distance of the two update vectors, all parameters together
    num = sum(float((pe[n] - pg[n]).double().pow(2).sum()) for n in pe)
    den = sum(float((pe[n] - start[n]).double().pow(2).sum()) for n in pe)
    rel = (num / max(den, 1e-30)) ** 0.5
    print("relative distance of the updates:", rel)
    assert rel < 0.1, rel    # measured 0.02


@pytest.mark.parametrize("name,kwargs", [("muon", {"muon_lr": 0.02}), ("adamw16", {}), ("adamw8bit", {})])
def test_engine_steps_with_other_registered_optimizers_on_the_native_path(name, kwargs):
    """The graphed native forward / backward with an optimizer that reads ``p.grad``: bf16 parameters, flat fp32
    gradients handed over per step; the loss on one repeated batch must fall and stay finite."""
    from kohakuwullm_b200.data.synthetic import make_packs
    from kohakuwullm_b200.models import LMBackbone, get_preset
    from kohakuwullm_b200.ops import native
    from kohakuwullm_b200.training.engine import TrainEngine

    cfg = get_preset("B200-smoke", depth=2, vocab_size=2048)
    torch.manual_seed(5)
    with torch.device("cuda"):
        model = LMBackbone(cfg)
    eng = TrainEngine(model, lr=2e-3, param_dtype=torch.bfloat16, optimizer=name, optimizer_kwargs=dict(kwargs))
    packs = [p.to("cuda") for p in make_packs(2, 1024, 32, 512, cfg.vocab_size, seed=9)]
    losses = [float(eng.step(packs)["loss"]) for _ in range(6)]
    torch.cuda.synchronize()
    native.check_status()
    assert all(l == l and l < 1e4 for l in losses), losses
    assert losses[-1] < losses[0] - 0.05, losses
