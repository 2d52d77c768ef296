"""Token-exact accumulation: loss and parameters after a step do not depend on how the same tokens
are split into micro-batches or across data-parallel ranks (gloo, CPU)."""

import os
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from kohakuwullm_b200.data.packing import PackedBatch, collate_packed, split_packed
from kohakuwullm_b200.data.synthetic import make_pack
from kohakuwullm_b200.models import LMBackbone, get_preset
from kohakuwullm_b200.training.engine import TrainEngine


def _model(seed=0, **kw):
    torch.manual_seed(seed)
    cfg = get_preset("B200-smoke", vocab_size=300, dim=64, depth=2, heads=2, kv_heads=1, head_dim=32,
                     mlp_hidden=128, **kw)
    return LMBackbone(cfg)


def _docs(n=6, seed=3):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, 300, (int(torch.randint(5, 40, (1,), generator=g)),), generator=g) for _ in range(n)]


def test_accumulation_is_token_exact():
    docs = _docs()
    whole = collate_packed(docs)
    results = []
    for parts in (1, 2, 3):
        eng = TrainEngine(_model(), lr=1e-2, max_grad_norm=0.0)
        out = eng.step(split_packed(whole, parts))
        flat = torch.cat([p.detach().reshape(-1) for p in eng.model.parameters()])
        results.append((float(out["loss"]), flat, float(out["grad_norm"])))
    for loss, flat, norm in results[1:]:
        assert abs(loss - results[0][0]) < 1e-5
        assert abs(norm - results[0][2]) < 1e-4 * results[0][2]
        # Adam divides by sqrt(v): elements with a vanishing gradient amplify summation-order noise,
        # so parameters are compared against the size of one update (lr = 1e-2)
        torch.testing.assert_close(flat, results[0][1], rtol=0, atol=3e-4)


def test_all_masked_step_changes_nothing():
    eng = TrainEngine(_model(), lr=1e-2)
    before = torch.cat([p.detach().reshape(-1).clone() for p in eng.model.parameters()])
    pack = make_pack(64, 8, 32, 300, seed=1)
    masked = PackedBatch(pack.tokens, torch.full_like(pack.labels, -100), pack.seq_info)
    eng.step([masked])
    after = torch.cat([p.detach().reshape(-1) for p in eng.model.parameters()])
    assert torch.equal(before, after)
    assert eng.optimizer.step_count == 0


def _ddp_worker(rank, world, port, path, compress=None):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    docs = _docs(8)
    mine = docs[rank::world]
    eng = TrainEngine(_model(), lr=1e-2, max_grad_norm=1.0, grad_compress=compress)
    out = eng.step([collate_packed(mine)])
    flat = torch.cat([p.detach().reshape(-1) for p in eng.model.parameters()])
    if rank == 0:
        torch.save({"loss": float(out["loss"]), "flat": flat, "norm": float(out["grad_norm"])}, path)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_world_two_matches_world_one():
    from tests.helpers import free_port

    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "r0.pt")
        mp.spawn(_ddp_worker, args=(2, free_port(), path), nprocs=2, join=True)
        got = torch.load(path)
    eng = TrainEngine(_model(), lr=1e-2, max_grad_norm=1.0)
    out = eng.step([collate_packed(_docs(8))])
    flat = torch.cat([p.detach().reshape(-1) for p in eng.model.parameters()])
    assert abs(got["loss"] - float(out["loss"])) < 1e-5
    assert abs(got["norm"] - float(out["grad_norm"])) < 1e-4
    torch.testing.assert_close(got["flat"], flat, rtol=0, atol=3e-4)


@pytest.mark.timeout(300)
@pytest.mark.parametrize("compress", ["bf16", "fp16"])
def test_compressed_gradient_buckets_stay_close_to_the_exact_sum(compress):
    """Gradient buckets sent in a 16-bit dtype: the loss is untouched (it is reduced separately), the gradient norm
    agrees to the wire format's precision, and the result is still a SUM (the fp16 pre-division is undone)."""
    from tests.helpers import free_port

    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "r0.pt")
        mp.spawn(_ddp_worker, args=(2, free_port(), path, compress), nprocs=2, join=True)
        got = torch.load(path)
    eng = TrainEngine(_model(), lr=1e-2, max_grad_norm=1.0)
    out = eng.step([collate_packed(_docs(8))])
    assert abs(got["loss"] - float(out["loss"])) < 1e-5
    rel = abs(got["norm"] - float(out["grad_norm"])) / float(out["grad_norm"])
    assert rel < (1e-2 if compress == "bf16" else 2e-3), rel
    with pytest.raises(ValueError):
        TrainEngine(_model(), grad_compress="int3")


def test_smoke_config_trains():
    """The CPU smoke model (fp32) learns a fixed batch."""
    torch.manual_seed(0)
    eng = TrainEngine(_model(z_loss_weight=1e-4), lr=3e-3)
    packs = [make_pack(128, 16, 64, 300, seed=s) for s in (1, 2)]
    first = float(eng.step(packs)["loss"])
    for _ in range(15):
        last = float(eng.step(packs)["loss"])
    assert last < first - 0.5
