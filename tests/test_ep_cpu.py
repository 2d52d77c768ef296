"""Expert parallelism on CPU (gloo, 2 ranks): the sharded model with the collective-based expert oracle
takes the same optimizer step as the single-process model holding all experts."""

import os
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from kohakuwullm_b200.data.packing import collate_packed
from kohakuwullm_b200.models import LMBackbone, get_preset
from kohakuwullm_b200.parallel.ep import gather_expert_state, scatter_expert_state
from kohakuwullm_b200.training.engine import TrainEngine


def _model(seed=0):
    torch.manual_seed(seed)
    cfg = get_preset("B200-smoke", vocab_size=300, dim=64, depth=2, heads=2, kv_heads=1, head_dim=32,
                     mlp_hidden=128, moe_every=1, moe_first_dense=1, moe_num_experts=8, moe_top_k=2,
                     moe_num_shared=1, moe_hidden=64)
    return LMBackbone(cfg)


def _docs(n=8, seed=5):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, 300, (int(torch.randint(5, 40, (1,), generator=g)),), generator=g) for _ in range(n)]


def _worker(rank, world, port, path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    eng = TrainEngine(_model(), lr=1e-2, max_grad_norm=1.0, expert_parallel=True)
    moe = [m for m in eng.model.modules() if getattr(m, "ep_world", 1) > 1]
    assert moe and moe[0].w_in.shape[0] == 4 and "fp32_ep" in eng.flat.groups
    out = eng.step([collate_packed(_docs()[rank::world])])
    state = gather_expert_state({k: v.detach().clone() for k, v in eng.model.state_dict().items()}, eng.model)
    # a full-model state dict loads back into the sharded model: every rank keeps its own expert slice
    back = scatter_expert_state(state, eng.model)
    for name, p in eng.model.named_parameters():
        if getattr(p, "ep_local", False):
            assert torch.equal(back[name], p.detach()), name
    eng.model.load_state_dict(back)
    if rank == 0:
        torch.save({"loss": float(out["loss"]), "norm": float(out["grad_norm"]), "state": state}, path)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_expert_parallel_step_matches_single_process():
    from tests.helpers import free_port

    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "r0.pt")
        mp.spawn(_worker, args=(2, free_port(), path), nprocs=2, join=True)
        got = torch.load(path)
    eng = TrainEngine(_model(), lr=1e-2, max_grad_norm=1.0)
    out = eng.step([collate_packed(_docs())])
    assert abs(got["loss"] - float(out["loss"])) < 1e-5
    assert abs(got["norm"] - float(out["grad_norm"])) < 1e-4
    ref = eng.model.state_dict()
    for k, v in ref.items():
        if v.is_floating_point():
            torch.testing.assert_close(got["state"][k], v, rtol=0, atol=3e-4, msg=lambda m, k=k: f"{k}: {m}")


def _ckpt_worker(rank, world, port, tmp):
    from kohakuwullm_b200.pipe import checkpoint as ckpt

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    eng = TrainEngine(_model(), lr=1e-2, max_grad_norm=1.0, expert_parallel=True)
    eng.step([collate_packed(_docs()[rank::world])])
    # whole-model checkpoint written from the expert-parallel layout
    ep_names = ckpt.expert_sharded_names(eng.model)
    assert ep_names
    opt = ckpt.gather_optimizer_state(eng.optimizer, None, None, ep_names=ep_names)
    weights = gather_expert_state(ckpt.local_state_dict(eng.model), eng.model)
    path = os.path.join(tmp, "ep.ckpt")
    if rank == 0:
        torch.save({"state_dict": weights, "optimizer_states": [opt]}, path)
    dist.barrier()
    # a fresh expert-parallel engine (other initial weights) resumes from it and takes the same second step
    fresh = TrainEngine(_model(seed=11), lr=1e-2, max_grad_norm=1.0, expert_parallel=True)
    ckpt.load(path, fresh.model, fresh.optimizer)
    fresh.global_step = eng.global_step
    batch = [collate_packed(_docs(seed=6)[rank::world])]
    a, b = eng.step(batch), fresh.step(batch)
    assert abs(float(a["loss"]) - float(b["loss"])) < 1e-6, (float(a["loss"]), float(b["loss"]))
    for (n, p), (_, q) in zip(eng.model.named_parameters(), fresh.model.named_parameters()):
        torch.testing.assert_close(p, q, rtol=0, atol=1e-6, msg=lambda m, n=n: f"{n}: {m}")
    if rank == 0:
        torch.save({"loss": float(a["loss"])}, os.path.join(tmp, "second.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_expert_parallel_checkpoint_reshards_weights_and_optimizer_state():
    """A checkpoint written by 2 expert-parallel ranks holds all experts and their AdamW state; it resumes a
    2-rank expert-parallel run exactly and a single-process run holding every expert to rounding."""
    from kohakuwullm_b200.pipe import checkpoint as ckpt
    from tests.helpers import free_port

    with tempfile.TemporaryDirectory() as tmp:
        mp.spawn(_ckpt_worker, args=(2, free_port(), tmp), nprocs=2, join=True)
        payload = torch.load(os.path.join(tmp, "ep.ckpt"), weights_only=False)
        second = torch.load(os.path.join(tmp, "second.pt"))
        eng = TrainEngine(_model(seed=3), lr=1e-2, max_grad_norm=1.0)
        full_experts = {n: p for n, p in eng.model.named_parameters() if n.endswith(("w_in", "w_out")) and p.dim() == 3}
        assert full_experts
        for n, p in full_experts.items():
            assert payload["state_dict"][n].shape == p.shape, n
            entry = payload["optimizer_states"][0]["named_optimizer_state"][n]
            assert entry["exp_avg"].numel() == p.numel() and float(entry["exp_avg"].abs().sum()) > 0
        ckpt.load(os.path.join(tmp, "ep.ckpt"), eng.model, eng.optimizer)
        eng.global_step = 1
        out = eng.step([collate_packed(_docs(seed=6))])
    assert abs(float(out["loss"]) - second["loss"]) < 1e-5


def _uneven_worker(rank, world, port, path):
    import faulthandler

    faulthandler.dump_traceback_later(120, exit=True)      # a hang here ends with every thread's stack, not a stalled suite
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    eng = TrainEngine(_model(), lr=1e-2, max_grad_norm=1.0, expert_parallel=True)
    docs = _docs(12)
    mine = [collate_packed(docs[i:i + 3]) for i in range(0, 9, 3)] if rank == 0 else [collate_packed(docs[9:])]
    out = eng.step(mine)                                    # three micro-batches on rank 0, one on rank 1
    if rank == 0:
        torch.save({"loss": float(out["loss"]), "tokens": float(out["tokens"])}, path)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_expert_parallel_ranks_with_different_micro_batch_counts_do_not_hang():
    """Every MoE layer of every micro-batch is a collective exchange: the ranks agree on the largest micro-batch count
    and the others add masked filler micro-batches. The loss equals the single-process step over all twelve documents."""
    from tests.helpers import free_port

    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "out.pt")
        mp.spawn(_uneven_worker, args=(2, free_port(), path), nprocs=2, join=True)
        got = torch.load(path)
    docs = _docs(12)
    ref = TrainEngine(_model(), lr=1e-2, max_grad_norm=1.0)
    want = ref.step([collate_packed(docs[i:i + 3]) for i in range(0, 12, 3)])
    assert got["tokens"] == float(want["tokens"])
    assert abs(got["loss"] - float(want["loss"])) < 2e-3, (got, float(want["loss"]))
