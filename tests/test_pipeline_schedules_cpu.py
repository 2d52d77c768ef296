"""Multi-chunk pipeline schedules (several stages per rank) on CPU / gloo: two optimizer steps through
interleaved 1F1B and through looped breadth-first leave the same losses and the same weights as the
single-process model. Not covered here, with the reason: the two V-placed schedules put neighbouring stages on
one rank, and torch's neighbour handshake then sends from a rank to itself, which gloo cannot do; the
zero-bubble family splits the backward pass with ``stage_backward_weight``, which in torch 2.11 raises on graphs
that contain custom ``autograd.Function`` nodes (``_input_metadata`` is a legacy access pattern), and every
kernel-backed op of this model is such a node."""

import os
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from kohakuwullm_b200.data.synthetic import make_pack
from kohakuwullm_b200.models import LMBackbone, get_preset
from kohakuwullm_b200.pipe.trainer import PipelineTrainer
from kohakuwullm_b200.training.engine import TrainEngine
from kohakuwullm_b200.training.parallel.pipeline import plan_for
from kohakuwullm_b200.training.parallel.uwupipe import LMPipelineModule
from tests.helpers import free_port

CFG = dict(vocab_size=200, dim=64, depth=4, heads=2, kv_heads=1, head_dim=32, mlp_hidden=128)
N_MICRO = 4


def _batch():
    return [make_pack(48, 8, 24, 200, seed=s) for s in range(1, N_MICRO + 1)]


def _reference(steps=2):
    torch.manual_seed(1234)
    model = LMBackbone(get_preset("B200-smoke", **CFG))
    eng = TrainEngine(model, lr=1e-2, max_grad_norm=1.0)
    losses = [float(eng.step(_batch())["loss"]) for _ in range(steps)]
    return losses, {k: v.detach().clone() for k, v in model.state_dict().items()}


def _worker(rank, world, port, schedule, out_dir):
    import faulthandler
    faulthandler.dump_traceback_later(240, exit=True)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = get_preset("B200-smoke", **CFG)
    module = LMPipelineModule(cfg, micro_tokens=48, lr=1e-2, param_dtype=None)
    plans = plan_for(cfg, 2 * world, layers=[1, 1, 1, 1])          # four stages, two per rank
    trainer = PipelineTrainer(module, plans, rank=rank, world=world, n_micro=N_MICRO, schedule=schedule,
                              max_grad_norm=1.0)
    outs = [trainer.loop.step(_batch()) for _ in range(2)]
    state = {}
    for stage in module.stages:
        names = stage.global_names()
        for k, v in stage.state_dict().items():
            state[names.get(k, k)] = v.detach().clone()
    torch.save({"losses": [float(o.loss) for o in outs], "state": state, "stages": trainer.local_indices},
               os.path.join(out_dir, f"rank{rank}.pt"))
    # several stages per rank in ONE whole-model checkpoint, and back: zero the weights, load, compare
    path = os.path.join(out_dir, "multi.ckpt")
    trainer.save_checkpoint(path)
    kept = {k: v.detach().clone() for st in module.stages for k, v in st.state_dict().items()}
    with torch.no_grad():
        for st in module.stages:
            for prm in st.parameters():
                prm.zero_()
    rest = trainer.load_checkpoint(path)
    again = {k: v for st in module.stages for k, v in st.state_dict().items()}
    ok = all(torch.equal(kept[k], again[k]) for k in kept) and rest.get("global_step", 2) == 2 and trainer.loop.global_step == 2
    torch.save({"roundtrip": bool(ok)}, os.path.join(out_dir, f"roundtrip{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(900)
@pytest.mark.parametrize("schedule,placement", [("interleaved-1f1b", [[0, 2], [1, 3]]),
                                                ("looped-bfs", [[0, 2], [1, 3]])])
def test_multi_chunk_schedule_matches_single_process(schedule, placement):
    ref_losses, ref_state = _reference()
    with tempfile.TemporaryDirectory() as tmp:
        mp.spawn(_worker, args=(2, free_port(), schedule, tmp), nprocs=2, join=True)
        parts = [torch.load(os.path.join(tmp, f"rank{r}.pt"), weights_only=False) for r in range(2)]
    assert [p["stages"] for p in parts] == placement
    for a, b in zip(parts[0]["losses"], ref_losses):
        assert abs(a - b) < 5e-5, (parts[0]["losses"], ref_losses)
    merged = {}
    for p in parts:
        merged.update(p["state"])
    assert set(merged) == set(ref_state)
    for k in ref_state:
        torch.testing.assert_close(merged[k], ref_state[k], rtol=0, atol=5e-4, msg=k)


@pytest.mark.timeout(900)
def test_checkpoint_with_two_stages_per_rank_is_a_whole_model_file():
    """Interleaved 1F1B, two ranks, four stages: the checkpoint is one file keyed by whole-model names (it loads into
    a single-process model and equals the reference run), and loading it back restores every stage and the step."""
    from kohakuwullm_b200.pipe import checkpoint as ckpt

    _, ref_state = _reference()
    with tempfile.TemporaryDirectory() as tmp:
        mp.spawn(_worker, args=(2, free_port(), "interleaved-1f1b", tmp), nprocs=2, join=True)
        assert all(torch.load(os.path.join(tmp, f"roundtrip{r}.pt"))["roundtrip"] for r in range(2))
        whole = LMBackbone(get_preset("B200-smoke", **CFG))
        rest = ckpt.load(os.path.join(tmp, "multi.ckpt"), whole)
        payload = ckpt.read_payload(os.path.join(tmp, "multi.ckpt"))
    assert set(payload["state_dict"]) == set(ref_state) and rest["global_step"] == 2
    for k, v in whole.state_dict().items():
        torch.testing.assert_close(v, ref_state[k], rtol=0, atol=5e-4, msg=k)
    named = payload["optimizer_states"][0]["named_optimizer_state"]
    assert set(named) == {n for n, _ in whole.named_parameters()}        # optimizer state under whole-model names too


# ------------------------------------------------------------------ a non-LM user of the engine
def _diffusion_worker(rank, world, port, out_dir):
    import faulthandler
    faulthandler.dump_traceback_later(120, exit=True)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from kohakuwullm_b200.cli import train_diffusion_pipe as dp
    from kohakuwullm_b200.pipe.plan import plan_stages

    module = dp.build_module(dim=64, depth=4, data_dim=8, micro_rows=16, lr=2e-3, seed=7)
    trainer = PipelineTrainer(module, plan_stages([1.0] * 4, world, head_cost=0.2), rank=rank, world=world, n_micro=4,
                              schedule="1f1b", max_grad_norm=1.0)
    outs = trainer.fit(dp.stream(64, 4, 8, seed=7), 60)
    trainer.save_checkpoint(os.path.join(out_dir, "diff.ckpt"))
    if rank == 0:
        torch.save([float(o.loss) for o in outs], os.path.join(out_dir, "diff_losses.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_pipeline_engine_trains_a_diffusion_model_and_checkpoints_a_stock_optimizer():
    """The engine is architecture-free: a flow-matching MLP whose stages exchange TWO tensors, with a structured
    target and a torch AdamW, trains under 1F1B on two ranks; its checkpoint holds whole-model names for weights
    and for the (position-keyed) optimizer state."""
    with tempfile.TemporaryDirectory() as tmp:
        mp.spawn(_diffusion_worker, args=(2, free_port(), tmp), nprocs=2, join=True)
        losses = torch.load(os.path.join(tmp, "diff_losses.pt"))
        payload = torch.load(os.path.join(tmp, "diff.ckpt"), weights_only=False)
    assert sum(losses[-10:]) / 10 < 0.75 * sum(losses[:3]) / 3      # the weighted error falls (it is noisy per step)
    names = set(payload["state_dict"])
    assert {"inp.weight", "out.weight", "blocks.0.mod.weight", "blocks.3.ff.2.bias"} <= names
    named = payload["optimizer_states"][0]["named_optimizer_state"]
    assert set(named) == names and "exp_avg" in named["blocks.3.ff.2.bias"]


@pytest.mark.timeout(300)
@pytest.mark.parametrize("check", ["checkpoint", "gen-resume"])
def test_dist_check_harness_passes_on_cpu_ranks(check):
    """The stand-alone multi-process checks (run on GPUs through torchrun) end in PASS on two gloo ranks."""
    import subprocess
    import sys

    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(free_port()), "-m", "kohakuwullm_b200.cli.dist_checks", check,
           "--backend", "gloo"]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=280,
                         cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert out.stdout.strip().splitlines()[-1] == "PASS"


@pytest.mark.timeout(300)
def test_multi_stream_boundaries_give_every_stage_its_gradient():
    """Accumulator, shared-context and skip streams across four stages (so the inner ranks use one group per
    link and direction): gradients equal the single-process model on every stage."""
    from kohakuwullm_b200.cli import pipe_streams
    from tests.helpers import free_port

    assert pipe_streams.main(["--case", "all", "--stages", "4", "--port", str(free_port())]) == 0


def _pipe_cli_worker(rank, world, port, port2, tmp):
    import importlib
    import json

    from kohakuwullm_b200.utils.config import configure

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    mod = importlib.import_module("kohakuwullm_b200.cli.train_lm_pipe")
    arch = dict(vocab_size=258, dim=32, depth=4, heads=2, kv_heads=1, head_dim=16, mlp_hidden=64, moe_every=1, moe_first_dense=1,
                moe_num_experts=4, moe_top_k=2, moe_hidden=32, mxfp8=False)
    common = ["--set", "BACKEND='gloo'", "--set", "PRESET='B200-smoke'", "--set", f"ARCH_OVERRIDES={arch!r}", "--set", "MICRO_TOKENS=64",
              "--set", "NUM_MICROBATCHES=3", "--set", "CTX_MAX=48", "--set", "AUTOTUNE=False", "--set", f"DATA={os.path.join(tmp, 'web')!r}",
              "--set", "OPTIMIZER='muon'", "--set", "OPTIMIZER_KWARGS={'muon_lr': 0.01}", "--set", "WARMUP_STEPS=2",
              "--set", "AUX_LOSS_WEIGHT=0.01", "--set", "BIAS_SCHEDULE={'mode': 'linear', 'end': 10}", "--set", "LOG_INTERVAL=1",
              "--set", f"METRICS_JSONL={os.path.join(tmp, 'm.jsonl')!r}"]
    configure(mod, common + ["--set", "MAX_STEPS=3", "--set", f"CKPT_DIR={os.path.join(tmp, 'ck')!r}"])
    tr = mod.main()
    lrs = [g["lr"] for g in tr.optimizer.param_groups]
    os.environ["MASTER_PORT"] = str(port2)      # a second rendezvous in the same processes: never on the port just closed
    mod = importlib.reload(mod)
    configure(mod, common + ["--set", "MAX_STEPS=1", "--set", f"CHECKPOINT_PATH={os.path.join(tmp, 'ck', 'last.ckpt')!r}"])
    tr2 = mod.main()
    if rank == 0:
        with open(os.path.join(tmp, "result.json"), "w") as f:
            json.dump({"steps": tr.loop.global_step, "lrs": lrs, "steps2": tr2.loop.global_step}, f)


@pytest.mark.timeout(600)
def test_pipeline_training_cli_on_a_corpus_with_muon_schedule_and_weight_only_restart(tmp_path):
    """The pipeline entry point on two gloo ranks: jsonl corpus through the micro-batched loader (identical on both
    ranks), a small MoE, Muon with a warm-up / cosine schedule that scales every group, the router-bias schedule, JSONL
    metrics, a whole-model checkpoint, and a second run that starts from its weights."""
    import json
    import random

    from tests.helpers import free_port

    rng = random.Random(2)
    d = tmp_path / "web"
    d.mkdir()
    (d / "part-0.jsonl").write_text("\n".join(json.dumps({"text": "".join(rng.choice("abcdef ") for _ in range(rng.randint(10, 60)))})
                                              for _ in range(200)) + "\n")
    mp.spawn(_pipe_cli_worker, args=(2, free_port(), free_port(), str(tmp_path)), nprocs=2, join=True)
    res = json.load(open(tmp_path / "result.json"))
    assert res["steps"] == 3 and res["steps2"] == 1
    assert len(set(round(x, 9) for x in res["lrs"])) > 1           # Muon and AdamW groups keep their own rates
    rows = [json.loads(l) for l in open(tmp_path / "m.jsonl")]
    assert rows and all(r["train/loss"] == r["train/loss"] for r in rows if "train/loss" in r)
