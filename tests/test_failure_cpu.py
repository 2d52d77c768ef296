"""Failure detection on the host (no GPU involved): an exception on one rank ends the run on every rank and
reaches every rank's ``on_exception`` hook; ranks that iterate different data are caught on the first step;
loader state of another world size and damaged checkpoint files are refused with explicit messages."""

import datetime
import os
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from kohakuwullm_b200.data.synthetic import make_pack
from kohakuwullm_b200.models import LMBackbone, get_preset
from kohakuwullm_b200.pipe import checkpoint as ckpt
from kohakuwullm_b200.pipe.hooks import Callback
from kohakuwullm_b200.pipe.trainer import PipelineTrainer
from kohakuwullm_b200.training.parallel.pipeline import plan_for
from kohakuwullm_b200.training.parallel.uwupipe import LMPipelineModule, verify_same_batch
from tests.helpers import free_port

CFG = dict(vocab_size=200, dim=64, depth=4, heads=2, kv_heads=1, head_dim=32, mlp_hidden=128)


def _batch(seed=0):
    return [make_pack(48, 8, 24, 200, seed=seed + s) for s in (1, 2, 3)]


class _Record(Callback):
    def __init__(self, path, rank, fail_at=None):
        self.path, self.rank, self.fail_at = path, rank, fail_at

    def on_train_batch_end(self, loop, out, batch, step):
        if self.fail_at is not None and step == self.fail_at:
            raise RuntimeError(f"injected failure on rank {self.rank}")

    def on_exception(self, loop, exc):
        with open(self.path, "w") as f:
            f.write(f"{type(exc).__name__}: {exc}")


def _failing_worker(rank, world, port, tmp):
    import faulthandler
    faulthandler.dump_traceback_later(120, exit=True)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    # a short collective time-out: the surviving rank's next transfer fails instead of waiting for ever
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    cfg = get_preset("B200-smoke", **CFG)
    module = LMPipelineModule(cfg, micro_tokens=48, lr=1e-2, param_dtype=None)
    cb = _Record(os.path.join(tmp, f"exc{rank}.txt"), rank, fail_at=2 if rank == 1 else None)
    trainer = PipelineTrainer(module, plan_for(cfg, world, layers=[2, 2]), rank=rank, world=world, n_micro=3,
                              schedule="1f1b", callbacks=[cb])
    try:
        trainer.fit((_batch() for _ in range(50)), max_steps=50)
    except BaseException as exc:  # noqa: BLE001
        with open(os.path.join(tmp, f"raised{rank}.txt"), "w") as f:
            f.write(type(exc).__name__)
    else:
        with open(os.path.join(tmp, f"finished{rank}.txt"), "w") as f:
            f.write("ran to the end")


@pytest.mark.timeout(300)
def test_exception_on_one_rank_ends_the_run_and_reaches_every_ranks_hook():
    with tempfile.TemporaryDirectory() as tmp:
        ctx = mp.spawn(_failing_worker, args=(2, free_port(), tmp), nprocs=2, join=False)
        for p in ctx.processes:
            p.join(timeout=200)
        alive = [p for p in ctx.processes if p.is_alive()]
        for p in alive:
            p.kill()
        assert not alive, "a rank kept waiting for the one that failed"
        files = set(os.listdir(tmp))
        assert {"exc0.txt", "exc1.txt", "raised0.txt", "raised1.txt"} <= files, files
        assert "injected failure on rank 1" in open(os.path.join(tmp, "exc1.txt")).read()
        assert not any(f.startswith("finished") for f in files)


def _mismatch_worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=30))
    verify_same_batch(_batch(0), "cpu")          # identical data: passes
    try:
        verify_same_batch(_batch(100 * rank), "cpu")   # rank 1 draws other documents
    except RuntimeError as exc:
        with open(os.path.join(tmp, f"mismatch{rank}.txt"), "w") as f:
            f.write(str(exc))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_ranks_that_iterate_different_data_are_caught_on_the_first_step():
    with tempfile.TemporaryDirectory() as tmp:
        mp.spawn(_mismatch_worker, args=(2, free_port(), tmp), nprocs=2, join=True)
        for r in (0, 1):
            msg = open(os.path.join(tmp, f"mismatch{r}.txt")).read()
            assert "rank 1 loaded a different batch than rank 0" in msg


def test_loader_state_of_another_world_size_is_refused():
    from kohakuwullm_b200.data.loader.iterative import ResumableLoader

    class _Inner:
        def state_dict(self):
            return {"cursor": 3}

        def load_state_dict(self, s):
            self.loaded = s

        def __iter__(self):
            return iter(())

    loader = ResumableLoader(_Inner())
    state = loader.state_dict()
    assert state["world"] == 1
    loader.load_state_dict(state)
    with pytest.raises(ValueError, match="saved with 4 ranks and cannot resume on 1"):
        loader.load_state_dict({"world": 4, "positions": [{"cursor": 0}] * 4})


def test_truncated_or_foreign_checkpoint_file_raises_a_checkpoint_error():
    torch.manual_seed(0)
    model = LMBackbone(get_preset("B200-smoke", **CFG))
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "model.ckpt")
        ckpt.save(path, model)
        ckpt.load(path, model)                                   # the intact file loads
        data = open(path, "rb").read()
        with open(path, "wb") as f:                              # a write that was cut short
            f.write(data[: len(data) // 2])
        with pytest.raises(ckpt.CheckpointError, match="truncated or corrupt"):
            ckpt.load(path, model)
        with open(path, "wb") as f:                              # not a checkpoint at all
            f.write(b"this is a text file")
        with pytest.raises(ckpt.CheckpointError):
            ckpt.load(path, model)
        torch.save({"weights": 1}, path)                         # a torch file of another layout
        with pytest.raises(ckpt.CheckpointError, match="state_dict"):
            ckpt.load(path, model)
        with pytest.raises(FileNotFoundError):
            ckpt.load(os.path.join(tmp, "missing.ckpt"), model)


def test_spike_score_flags_a_loss_spike_and_ignores_noise():
    import random

    from kohakuwullm_b200.training.loop.health import SpikeScore

    rng = random.Random(0)
    s = SpikeScore(window=200, threshold=7.0, min_history=20)
    flagged = [s.is_spike(s.update(2.0 + 0.01 * rng.gauss(0, 1))) for _ in range(150)]
    assert not any(flagged)
    assert s.is_spike(s.update(2.5))                      # fifty sigma above the running median
    assert not s.is_spike(s.update(2.01))                 # and the detector recovers at once (median / MAD are robust)


def test_killed_loader_worker_is_reported_not_waited_for():
    """A worker process that dies (killed from outside, out of memory) must surface as an error in the trainer process
    within a second or two, not as a stalled input pipeline."""
    import os
    import random
    import signal
    import time

    import pytest

    from kohakuwullm_b200.data import ByteTokenizer
    from kohakuwullm_b200.data.loader.workers import WorkerPackLoader
    from kohakuwullm_b200.data.renderers.base import PlainRenderer
    from kohakuwullm_b200.data.sources.records import ListRecords

    tok = ByteTokenizer()
    records = ListRecords([{"text": "z" * n} for n in random.Random(2).choices(range(3, 50), k=400)])
    loader = WorkerPackLoader(records, PlainRenderer(), tok.encode, workers=1, prefetch=1, k=64, m=16, seed=3)
    it = iter(loader)
    next(it)
    os.kill(loader._procs[0].pid, signal.SIGKILL)
    t0 = time.time()
    with pytest.raises(RuntimeError, match="loader worker 0 exited"):
        for _ in range(20):                                # what the worker had already queued may still arrive
            next(it)
    assert time.time() - t0 < 30


def test_training_script_launches_its_own_ranks(tmp_path):
    """``GPUS=2`` without a launcher: the script spawns two ranks (gloo here), trains and writes one checkpoint; a rank
    that raises ends the whole run with an error instead of leaving its peer waiting."""
    import json
    import os
    import random
    import subprocess
    import sys

    rng = random.Random(3)
    d = tmp_path / "web"
    d.mkdir()
    (d / "part-0.jsonl").write_text("\n".join(json.dumps({"text": "".join(rng.choice("abcdef ") for _ in range(rng.randint(10, 60)))})
                                              for _ in range(200)) + "\n")
    arch = dict(vocab_size=258, dim=32, depth=2, heads=2, kv_heads=1, head_dim=16, mlp_hidden=64, mxfp8=False)
    base = [sys.executable, "-m", "kohakuwullm_b200.cli.train_lm_pipe", "--set", "GPUS=2", "--set", "BACKEND='gloo'",
            "--set", "PRESET='B200-smoke'", "--set", f"ARCH_OVERRIDES={arch!r}", "--set", "MICRO_TOKENS=64", "--set", "NUM_MICROBATCHES=2",
            "--set", "CTX_MAX=48", "--set", "AUTOTUNE=False", "--set", f"DATA={str(d)!r}", "--set", "MAX_STEPS=2", "--set", "WARMUP_STEPS=1"]
    env = dict(os.environ, PYTHONPATH=os.getcwd())
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT"):
        env.pop(k, None)
    ok = subprocess.run(base + ["--set", f"CKPT_DIR={str(tmp_path / 'ck')!r}"], env=env, capture_output=True, text=True, timeout=300)
    assert ok.returncode == 0, ok.stderr[-2000:]
    assert os.path.exists(tmp_path / "ck" / "last.ckpt")
    bad = subprocess.run(base + ["--set", "SCHEDULE='no-such-schedule'"], env=env, capture_output=True, text=True, timeout=300)
    assert bad.returncode != 0 and "no-such-schedule" in (bad.stderr + bad.stdout)


def test_only_rank_zero_logs_unless_asked(monkeypatch):
    import io

    from kohakuwullm_b200.utils import logging as klog

    for rank, all_ranks, expect in (("0", None, True), ("1", None, False), ("1", True, True)):
        monkeypatch.setenv("RANK", rank)
        buf = io.StringIO()
        klog.configure(stream=buf, all_ranks=all_ranks)
        klog.get_logger("t").info("event", x=1)
        assert ("event x=1" in buf.getvalue()) == expect, (rank, all_ranks, buf.getvalue())
        klog.get_logger("t").error("bad")
        assert "bad" in buf.getvalue()                      # errors from any rank
    monkeypatch.setenv("RANK", "0")
    klog.configure()


class _DictStore:
    """In-process stand-in for the job's key-value store."""

    def __init__(self):
        self.data = {}

    def set(self, key, value):
        self.data[key] = value.encode() if isinstance(value, str) else bytes(value)

    def get(self, key):
        return self.data[key]

    def check(self, keys):
        return all(k in self.data for k in keys)


def test_heartbeat_notices_a_silent_peer_and_an_announced_exit():
    """Three ranks on one store. A peer that stops beating is reported after the timeout (judged on the reader's own
    clock), one that says it leaves is reported at once, and a peer that never appeared is tolerated only for the
    timeout."""
    import time

    from kohakuwullm_b200.utils.heartbeat import HeartbeatCallback, PeerLost, RankHeartbeat

    store = _DictStore()
    hbs = [RankHeartbeat(store, r, 3, interval=0.05, timeout=0.4) for r in range(3)]
    time.sleep(0.15)
    for hb in hbs:
        hb.check(force=True)
        assert hb.alive() == [0, 1, 2]
    hbs[2].close()                                   # dies silently: no more beats, no announcement
    t0 = time.monotonic()
    with pytest.raises(PeerLost) as err:
        while time.monotonic() - t0 < 3.0:
            hbs[0].check()
            time.sleep(0.02)
    assert err.value.rank == 2 and 0.3 < time.monotonic() - t0 < 1.5 and "no heartbeat" in str(err.value)
    assert hbs[1].alive() == [0, 1]
    # an exception in a rank's own step announces the exit through the callback; the others stop at their next check
    HeartbeatCallback(hbs[1]).on_exception(None, ValueError("loss is nan"))
    with pytest.raises(PeerLost) as err:
        hbs[0].check(force=True)
    assert err.value.rank == 1 and "loss is nan" in str(err.value)
    hbs[0].close()
    late = RankHeartbeat(_DictStore(), 0, 2, interval=0.05, timeout=0.3)      # rank 1 never shows up
    late.check(force=True)
    time.sleep(0.4)
    with pytest.raises(PeerLost) as err:
        late.check(force=True)
    assert err.value.rank == 1 and "never" in str(err.value)
    late.close()
    with pytest.raises(ValueError):
        RankHeartbeat(_DictStore(), 0, 2, interval=1.0, timeout=1.5)


def _heartbeat_rank(rank, world, port, out_dir):
    import time

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    from kohakuwullm_b200.utils.heartbeat import PeerLost, RankHeartbeat

    hb = RankHeartbeat.from_env(interval=0.1, timeout=1.0, port_offset=0)
    result = "finished"
    try:
        for step in range(60):
            hb.check()
            if rank == world - 1 and step == 5:
                os._exit(0)                          # the process is gone between two steps, without a word
            time.sleep(0.05)
    except PeerLost as exc:
        result = f"lost {exc.rank}"
    with open(os.path.join(out_dir, f"r{rank}.txt"), "w") as fh:
        fh.write(result)
    if rank == 0:
        time.sleep(1.0)                              # the store's server outlives the other readers
    hb.close()


@pytest.mark.timeout(120)
def test_heartbeat_over_a_tcp_store_between_processes(tmp_path):
    """Real processes and a real TCP store: the last rank exits between steps; the survivors learn of it on the host
    within the timeout and name the rank, with no collective involved."""
    import multiprocessing as mp

    from tests.helpers import free_port

    ctx = mp.get_context("spawn")
    port = free_port()
    procs = [ctx.Process(target=_heartbeat_rank, args=(r, 3, port, str(tmp_path))) for r in range(3)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
        assert not p.is_alive()
    assert (tmp_path / "r0.txt").read_text() == "lost 2" and (tmp_path / "r1.txt").read_text() == "lost 2"
    assert not (tmp_path / "r2.txt").exists()


def _hb_trainer_rank(rank, world, port, out_dir):
    import time

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=120))
    from kohakuwullm_b200.training.loop.trainer import LMTrainer
    from kohakuwullm_b200.utils.heartbeat import HeartbeatCallback, PeerLost, RankHeartbeat

    class Trip(Callback):
        def on_train_batch_end(self, trainer, out, batch, step):
            if rank == 1 and step == 2:
                raise RuntimeError("injected failure")
            if rank == 0 and step == 2:
                time.sleep(1.0)               # the survivor reaches its next step after the failing rank said goodbye

    hb = RankHeartbeat.from_env(interval=0.1, timeout=5.0)
    trainer = LMTrainer("B200-smoke", dict(CFG), device="cpu", param_dtype=None, callbacks=[HeartbeatCallback(hb), Trip()])
    t0 = time.monotonic()
    try:
        trainer.fit((make_pack(48, 8, 24, 200, seed=s) for s in range(50)), max_steps=50)
        result = "finished"
    except PeerLost as exc:
        result = f"PeerLost {exc.rank} at step {trainer.global_step} after {time.monotonic() - t0:.1f}s: {exc}"
    except RuntimeError as exc:
        result = f"RuntimeError: {exc}"
    with open(os.path.join(out_dir, f"r{rank}.txt"), "w") as fh:
        fh.write(result)
    if rank == 0:
        time.sleep(0.5)
    os._exit(0)        # skip the process-group teardown: the peer is gone


@pytest.mark.timeout(180)
def test_trainer_with_heartbeat_stops_before_the_next_collective(tmp_path):
    """Data-parallel trainer on two gloo ranks with a 120 s collective time-out: rank 1 raises after step 2. Rank 0
    must not enter step 3's all-reduce (it would wait two minutes): the heartbeat check at the start of the step
    raises PeerLost with the failing rank's own message."""
    import multiprocessing as mp_std

    ctx = mp_std.get_context("spawn")
    port = free_port()
    procs = [ctx.Process(target=_hb_trainer_rank, args=(r, 2, port, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(100)
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.kill()
    assert not alive, "the surviving rank went into a collective with a dead peer"
    r0, r1 = (tmp_path / "r0.txt").read_text(), (tmp_path / "r1.txt").read_text()
    assert r1 == "RuntimeError: injected failure"
    assert r0.startswith("PeerLost 1 at step 2") and "injected failure" in r0, r0
