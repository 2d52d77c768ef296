"""Pipeline engine on CPU (gloo): partition properties, 1F1B/GPipe gradient equivalence with the
single-process model, checkpoint portability across splits."""

import os
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from hypothesis import given, settings, strategies as st

from kohakuwullm_b200.data.synthetic import make_pack
from kohakuwullm_b200.models import LMBackbone, get_preset
from kohakuwullm_b200.pipe.plan import partition, partition_v, plan_from_layers, plan_stages
from kohakuwullm_b200.pipe.trainer import PipelineTrainer
from kohakuwullm_b200.training.engine import TrainEngine
from kohakuwullm_b200.training.parallel.pipeline import plan_for
from kohakuwullm_b200.training.parallel.uwupipe import LMPipelineModule
from tests.helpers import free_port


@settings(max_examples=60, deadline=None)
@given(st.lists(st.floats(0.1, 10.0), min_size=2, max_size=14), st.integers(1, 6), st.floats(0, 20))
def test_partition_is_contiguous_complete_and_optimal(costs, stages, head):
    stages = min(stages, len(costs))
    bounds = partition(costs, stages, head_cost=head)
    assert bounds[0][0] == 0 and bounds[-1][1] == len(costs)
    assert all(a < b for a, b in bounds) and all(x[1] == y[0] for x, y in zip(bounds, bounds[1:]))

    def worst(bs):
        return max(sum(costs[a:b]) + (head if i == len(bs) - 1 else 0) for i, (a, b) in enumerate(bs))

    # brute force over all cut sets for small inputs
    import itertools

    best = min(worst(list(zip((0, *cuts), (*cuts, len(costs)))))
               for cuts in itertools.combinations(range(1, len(costs)), stages - 1))
    assert worst(bounds) <= best + 1e-9


def test_partition_puts_fewer_layers_next_to_an_expensive_head():
    plans = plan_stages([1.0] * 16, 4, head_cost=3.0)
    assert plans[-1].num_layers < plans[0].num_layers
    assert sum(p.num_layers for p in plans) == 16


def test_partition_v_covers_all_layers():
    bounds = partition_v([1.0] * 12, 3, head_cost=2.0)
    assert len(bounds) == 6 and bounds[0][0] == 0 and bounds[-1][1] == 12


CFG = dict(vocab_size=200, dim=64, depth=4, heads=2, kv_heads=1, head_dim=32, mlp_hidden=128)


def _batch():
    return [make_pack(48, 8, 24, 200, seed=s) for s in (1, 2, 3)]


def _reference(steps=2, optimizer="fused_adamw"):
    torch.manual_seed(1234)
    model = LMBackbone(get_preset("B200-smoke", **CFG))
    eng = TrainEngine(model, lr=1e-2, max_grad_norm=1.0, optimizer=optimizer)
    losses = [float(eng.step(_batch())["loss"]) for _ in range(steps)]
    return losses, {k: v.detach().clone() for k, v in model.state_dict().items()}


def _pipe_worker(rank, world, port, schedule, layers, out_dir, load_from, optimizer="fused_adamw"):
    import faulthandler
    faulthandler.dump_traceback_later(120, exit=True)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = get_preset("B200-smoke", **CFG)
    module = LMPipelineModule(cfg, micro_tokens=48, lr=1e-2, param_dtype=None, optimizer=optimizer)
    plans = plan_for(cfg, world, layers=layers)
    trainer = PipelineTrainer(module, plans, rank=rank, world=world, n_micro=3, schedule=schedule, max_grad_norm=1.0)
    steps = 2
    if load_from:
        trainer.load_checkpoint(load_from)
        steps = 1
    outs = [trainer.loop.step(_batch()) for _ in range(steps)]
    trainer.save_checkpoint(os.path.join(out_dir, "pipe.ckpt"))
    if rank == 0:
        torch.save([float(o.loss) for o in outs], os.path.join(out_dir, "losses.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(600)
@pytest.mark.parametrize("schedule,layers", [("1f1b", [3, 1]), ("gpipe", [2, 2]), ("1f1b", [1, 1, 1, 1]), ("1f1b", [2, 2, 0])])
def test_pipeline_matches_single_process(schedule, layers):
    # four stages: every inner rank has two neighbours, each link and direction on a group of its own;
    # [2, 2, 0]: a last stage that holds the final norm and the head only (what the planner may pick for a wide head)
    ref_losses, ref_state = _reference()
    world = len(layers)
    with tempfile.TemporaryDirectory() as tmp:
        mp.spawn(_pipe_worker, args=(world, free_port(), schedule, layers, tmp, None), nprocs=world, join=True)
        losses = torch.load(os.path.join(tmp, "losses.pt"))
        payload = torch.load(os.path.join(tmp, "pipe.ckpt"), weights_only=False)
    for a, b in zip(losses, ref_losses):
        assert abs(a - b) < 2e-5, (losses, ref_losses)
    state = payload["state_dict"]
    assert set(state) == set(ref_state)
    for k in ref_state:
        torch.testing.assert_close(state[k], ref_state[k], rtol=0, atol=5e-4, msg=k)
    named = payload["optimizer_states"][0]["named_optimizer_state"]
    assert set(named) == {k for k in ref_state if "expert_bias" not in k and "load_accum" not in k}


@pytest.mark.timeout(600)
def test_pipeline_with_a_registered_optimizer_matches_single_process():
    """Muon on the pipeline engine: every stage builds it over its own slice (hidden matrices of one shape are
    orthogonalised as a batch per stage); losses and weights equal the single-process engine with the same
    optimizer, and its position-keyed state is checkpointed by whole-model names."""
    ref_losses, ref_state = _reference(optimizer="muon")
    with tempfile.TemporaryDirectory() as tmp:
        mp.spawn(_pipe_worker, args=(2, free_port(), "1f1b", [3, 1], tmp, None, "muon"), nprocs=2, join=True)
        losses = torch.load(os.path.join(tmp, "losses.pt"))
        payload = torch.load(os.path.join(tmp, "pipe.ckpt"), weights_only=False)
    for a, b in zip(losses, ref_losses):
        assert abs(a - b) < 2e-5, (losses, ref_losses)
    for k in ref_state:
        torch.testing.assert_close(payload["state_dict"][k], ref_state[k], rtol=0, atol=5e-4, msg=k)
    named = payload["optimizer_states"][0]["named_optimizer_state"]
    assert any("momentum" in "".join(v.keys()) or "buf" in "".join(v.keys()) for v in named.values())
    assert all(k in ref_state for k in named)


@pytest.mark.timeout(600)
def test_checkpoint_loads_under_another_split_and_on_one_process():
    with tempfile.TemporaryDirectory() as tmp:
        mp.spawn(_pipe_worker, args=(2, free_port(), "1f1b", [3, 1], tmp, None), nprocs=2, join=True)
        ckpt_path = os.path.join(tmp, "pipe.ckpt")
        first = torch.load(os.path.join(tmp, "losses.pt"))
        # continue for one step under a different split ...
        other = os.path.join(tmp, "other")
        os.makedirs(other)
        mp.spawn(_pipe_worker, args=(2, free_port(), "1f1b", [1, 3], other, ckpt_path), nprocs=2, join=True)
        resumed = torch.load(os.path.join(other, "losses.pt"))[0]
        # ... and in one process
        from kohakuwullm_b200.pipe import checkpoint as ckpt

        torch.manual_seed(0)
        model = LMBackbone(get_preset("B200-smoke", **CFG))
        eng = TrainEngine(model, lr=1e-2, max_grad_norm=1.0)
        ckpt.load(ckpt_path, model, eng.optimizer)
        single = float(eng.step(_batch())["loss"])
    ref_losses, _ = _reference(steps=3)
    assert abs(resumed - ref_losses[2]) < 5e-5
    assert abs(single - ref_losses[2]) < 5e-5
    assert first[0] == pytest.approx(ref_losses[0], abs=2e-5)


def _plm_worker(rank, world, port, out_dir):
    import faulthandler
    faulthandler.dump_traceback_later(120, exit=True)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from kohakuwullm_b200.training.loop.pipeline_trainer import PipelinedLMTrainer

    tr = PipelinedLMTrainer("B200-smoke", CFG, micro_tokens=48, num_microbatches=3, layers=[3, 1], lr=1e-2,
                            device="cpu", param_dtype=None)
    losses = [float(tr.training_step(_batch()).loss) for _ in range(2)]
    state = tr.gathered_state_dict()
    prompt = torch.arange(1, 7).reshape(1, 6)
    tokens = tr.generate(prompt, 5, temperature=0.0)
    if rank == 0:
        torch.save({"losses": losses, "state": state, "tokens": tokens}, os.path.join(out_dir, "plm.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(600)
def test_pipelined_lm_trainer_trains_gathers_and_generates():
    """The LM-level pipeline trainer: same losses as one process, whole-model state on every rank, and a
    collective greedy decode that equals the single-process decode of the gathered weights."""
    from kohakuwullm_b200.generation.engine import LocalGenerator

    ref_losses, ref_state = _reference()
    with tempfile.TemporaryDirectory() as tmp:
        mp.spawn(_plm_worker, args=(2, free_port(), tmp), nprocs=2, join=True)
        got = torch.load(os.path.join(tmp, "plm.pt"), weights_only=False)
    for a, b in zip(got["losses"], ref_losses):
        assert abs(a - b) < 2e-5
    assert set(got["state"]) == set(ref_state)
    model = LMBackbone(get_preset("B200-smoke", **CFG))
    model.load_state_dict(got["state"])
    want = LocalGenerator(model, eos_id=-1).generate(torch.arange(1, 7).reshape(1, 6), 5, temperature=0.0)
    assert got["tokens"].shape == want.shape
    assert torch.equal(got["tokens"][:, :6], want[:, :6])
