"""LMTrainer end to end on CPU: fit, counters, checkpoint, resume continues the same trajectory."""

import os
import random

import pytest

import torch

from kohakuwullm_b200.data import ByteTokenizer, IterativePackLoader, ResumableLoader
from kohakuwullm_b200.data.renderers.base import PlainRenderer
from kohakuwullm_b200.data.sources.records import ListRecords
from kohakuwullm_b200.training.loop.trainer import LMTrainer
from kohakuwullm_b200.utils.schedule import build_schedule

ARCH = dict(vocab_size=258, dim=32, depth=2, heads=2, kv_heads=1, head_dim=16, mlp_hidden=64)


def _loader():
    tok = ByteTokenizer()
    rng = random.Random(0)
    recs = ListRecords([{"text": "".join(rng.choice("abcdef ") for _ in range(rng.randint(5, 60)))} for _ in range(300)])
    return ResumableLoader(IterativePackLoader(recs, PlainRenderer(), tok.encode, k=96, m=24, bos=256, eos=257, seed=3))


def _trainer():
    return LMTrainer("B200-smoke", ARCH, lr=3e-3, grad_accum=2, device="cpu", log_interval=2,
                     lr_schedule={"mode": "cosine", "warmup": 2, "end": 20})


def test_fit_checkpoint_resume(tmp_path):
    full = _trainer()
    full.fit(_loader(), 8)
    ref = torch.cat([p.detach().reshape(-1) for p in full.backbone.parameters()])

    first = _trainer()
    loader = _loader()
    first.fit(loader, 4)
    path = os.path.join(tmp_path, "run.ckpt")
    first.save_checkpoint(path)
    snap = first.snapshot()
    assert snap.seen > 0 and snap.trained > 0 and snap.model_flops > 0

    second = _trainer()
    loader2 = _loader()
    second.load_checkpoint(path, loader2)
    assert second.global_step == 4 and second.snapshot().seen == snap.seen
    second.fit(loader2, 8)
    got = torch.cat([p.detach().reshape(-1) for p in second.backbone.parameters()])
    torch.testing.assert_close(got, ref, rtol=0, atol=2e-5)
    assert second.snapshot().seen == full.snapshot().seen


def test_schedules():
    f = build_schedule({"mode": "cosine", "warmup": 10, "end": 110, "min_value": 0.1})
    assert f(0) < f(9) <= 1.0 and abs(f(10) - 1.0) < 1e-6 and abs(f(110) - 0.1) < 1e-6
    w = build_schedule({"mode": "wsd", "warmup": 0, "end": 100, "decay_start": 80})
    assert w(50) == 1.0 and w(90) == 0.5
    p = build_schedule({"mode": "power", "s0": 100, "b": -0.5, "warmup": 10, "end": 10_000, "min_value": 0.05})
    assert p(50) == 1.0 and abs(p(400) - 0.5) < 1e-9 and abs(p(10_000) - 0.1) < 1e-9 and p(10 ** 9) == p(10_000)
    e = build_schedule({"mode": "exponential", "half_life": 100, "min_value": 0.2})
    assert abs(e(100) - 0.5) < 1e-9 and e(1000) == 0.2
    with pytest.raises(ValueError):
        build_schedule({"mode": "triangle"})


def test_composed_schedules_are_continuous_and_count_from_each_phase_start():
    from kohakuwullm_b200.utils.misc import autofill_schedule_steps

    # constant, then a cosine that must reach its floor exactly at the composition's end
    f = build_schedule({"phases": [{"mode": "constant", "end": 100}, {"mode": "cosine", "end": 200, "min_value": 0.1}]})
    assert f(0) == f(99) == 1.0 and abs(f(100) - 1.0) < 1e-9
    assert abs(f(150) - 0.55) < 1e-9 and abs(f(200) - 0.1) < 1e-9 and abs(f(5000) - 0.1) < 1e-9
    # the reference's long-run recipe: warm-up, inverse-square-root decay for 90 % of the run, cosine tail that
    # starts where the power law stopped (fractional ends refer to the composition's end, left open in the config)
    spec = {"mode": "composer", "end": -1, "schedules": [
        {"mode": "power", "end": 0.9, "s0": 2500, "b": -0.5, "warmup": None},
        {"mode": "cosine", "end": 1.0, "min_value": 0.01}]}
    g = build_schedule(autofill_schedule_steps(spec, 400_000, 2000))
    assert abs(g(1999) - 1.0) < 1e-9 and g(2500) == 1.0
    at_switch = (360_000 / 2500) ** -0.5
    assert abs(g(359_999) - at_switch) < 1e-4 and abs(g(360_000) - at_switch) < 1e-9
    assert abs(g(400_000) - 0.01 * at_switch) < 1e-9
    values = [g(s) for s in range(0, 400_001, 997)]
    assert all(b <= a + 1e-12 for a, b in zip(values[3:], values[4:]))       # monotone after the warm-up
    # a ten-step smoke run of the same recipe: 0.9 x 4 rounds onto 4, the tail phase is empty and drops out
    short = build_schedule(autofill_schedule_steps(spec, 4, 1))
    assert all(0.0 < short(s) <= 1.0 for s in range(6))
    with pytest.raises(ValueError):
        build_schedule({"phases": [{"mode": "constant", "end": 0.5}, {"mode": "cosine", "end": 1.0}]})   # no total
    with pytest.raises(ValueError):
        build_schedule({"phases": [{"mode": "constant", "end": 100}, {"mode": "cosine", "end": 100}]})


def test_reporters_write_scalars_perplexity_and_sample_tables(tmp_path, monkeypatch):
    """The metric sinks: JSONL rows carry the step and a derived perplexity; the W&B sink runs offline (no
    network here), logs scalars and turns generated samples into a table."""
    import json

    import torch

    from kohakuwullm_b200.utils.reporters import JsonlReporter, MultiReporter, WandbReporter, build_reporter

    path = tmp_path / "metrics.jsonl"
    rep = JsonlReporter(str(path))
    rep({"train/loss": torch.tensor(2.0), "train/lr": 3e-4}, 7)
    rep.samples(7, [("val", "once upon", 0, "once upon a time")])
    rows = [json.loads(line) for line in path.read_text().splitlines()]
    assert rows[0]["step"] == 7 and rows[0]["train/loss"] == 2.0
    assert abs(rows[0]["train/ppl"] - 7.389056) < 1e-4
    assert rows[1]["samples"][0][3] == "once upon a time"

    monkeypatch.setenv("WANDB_SILENT", "true")
    wb = WandbReporter("kwu-test", name="unit", mode="offline", directory=str(tmp_path / "wb"))
    assert wb.run is not None and wb.run_id
    both = MultiReporter(wb, JsonlReporter(str(tmp_path / "m2.jsonl")))
    both({"loss": 1.5, "step": 3})
    both.samples(3, [("val", "p", 0, "t")])
    both.finish()
    assert json.loads((tmp_path / "m2.jsonl").read_text().splitlines()[0])["step"] == 3
    assert any((tmp_path / "wb").rglob("*.wandb"))            # the offline run directory exists
    assert build_reporter() is None
    assert isinstance(build_reporter(jsonl=str(tmp_path / "m3.jsonl"), console_interval=10), MultiReporter)


@pytest.mark.parametrize("name,kwargs", [("muon", {"muon_lr": 0.02}), ("adamw", {}), ("adamw8bit", {"min_quantized_size": 256})])
def test_trainer_with_a_registered_optimizer_trains_checkpoints_and_resumes(tmp_path, name, kwargs):
    """Any registered optimizer can drive the trainer (it steps from the reduced, clipped flat gradients); its state is
    checkpointed by parameter name and an interrupted run continues exactly."""
    def make():
        return LMTrainer("B200-smoke", dict(ARCH), lr=5e-3, grad_accum=2, log_interval=100, device="cpu",
                         lr_schedule={"mode": "cosine", "warmup": 2, "end": 20}, optimizer=name, optimizer_kwargs=dict(kwargs))

    full = make()
    assert full.engine.generic_optimizer and not full.engine.fused_sync
    full.fit(_loader(), 6)
    ref = torch.cat([p.detach().reshape(-1) for p in full.backbone.parameters()])
    start = torch.cat([p.detach().reshape(-1) for p in make().backbone.parameters()])
    assert float((ref - start).abs().max()) > 1e-4          # it trained
    lrs = {round(g["lr"] / g["initial_lr"], 6) for g in full.engine.optimizer.param_groups}
    assert len(lrs) == 1                                      # every group follows the schedule with its own base rate

    first = make()
    loader = _loader()
    first.fit(loader, 3)
    path = os.path.join(tmp_path, "run.ckpt")
    first.save_checkpoint(path)
    second = make()
    loader2 = _loader()
    second.load_checkpoint(path, loader2)
    second.fit(loader2, 6)
    got = torch.cat([p.detach().reshape(-1) for p in second.backbone.parameters()])
    torch.testing.assert_close(got, ref, rtol=0, atol=5e-5)


def test_train_lm_cli_with_a_mixture_validation_sampling_and_weight_only_load(tmp_path, capsys):
    """The training entry point end to end on CPU: two jsonl corpora mixed with repeat weights, a held-out validation
    split, preview sampling, metrics as JSONL, a checkpoint, and a second run that starts from its weights only."""
    import importlib
    import json

    from kohakuwullm_b200.utils.config import configure

    rng = random.Random(1)
    for name, n in (("web", 60), ("code", 30)):
        d = tmp_path / name
        d.mkdir()
        (d / "part-0.jsonl").write_text("\n".join(json.dumps({"text": "".join(rng.choice("abcdef ") for _ in range(rng.randint(10, 80)))})
                                                  for _ in range(n)) + "\n")
    common = ["--set", "DEVICE='cpu'", "--set", "PRESET='B200-smoke'", "--set", f"ARCH_OVERRIDES={ARCH!r}", "--set", "BATCH_TOKENS=192",
              "--set", "CTX_MAX=96", "--set", "GRAD_ACCUM=2", "--set", "LOG_INTERVAL=2", "--set", "WARMUP_STEPS=1",
              "--set", f"SOURCES=[{{'records': {{'name': 'corpus', 'root': {str(tmp_path / 'web')!r}}}, 'repeat': 1.5, 'source': 'web'}}, "
                       f"{{'records': {{'name': 'corpus', 'root': {str(tmp_path / 'code')!r}}}, 'repeat': 2, 'source': 'code'}}]",
              "--set", "VAL_FRACTION=0.2", "--set", "VAL_INTERVAL=2", "--set", "VAL_BATCHES=2",
              "--set", "SAMPLE_INTERVAL=2", "--set", "SAMPLE_PROMPTS=['abc']", "--set", "SAMPLE_TOKENS=4",
              "--set", f"METRICS_JSONL={str(tmp_path / 'metrics.jsonl')!r}"]
    mod = importlib.import_module("kohakuwullm_b200.cli.train_lm")
    mod = importlib.reload(mod)
    configure(mod, common + ["--set", "MAX_STEPS=4", "--set", f"CKPT_DIR={str(tmp_path / 'ckpt')!r}"])
    first = mod.main()
    assert first.global_step == 4 and os.path.exists(tmp_path / "ckpt" / "last.ckpt")
    rows = [json.loads(l) for l in open(tmp_path / "metrics.jsonl")]
    assert any("val/loss" in r for r in rows)
    mod = importlib.reload(mod)
    configure(mod, common + ["--set", "MAX_STEPS=1", "--set", f"CHECKPOINT_PATH={str(tmp_path / 'ckpt' / 'last.ckpt')!r}",
                             "--set", "OPTIMIZER='adamw'", "--set", "USE_MUP=True", "--set", "BASE_DIM=16"])
    second = mod.main()
    assert second.global_step == 1                       # weights only: counters start again
    a = torch.cat([p.detach().reshape(-1) for p in first.backbone.parameters()])
    b = torch.cat([p.detach().reshape(-1) for p in second.backbone.parameters()])
    assert float((a - b).abs().max()) < 0.1              # one small step away from the loaded weights, not a fresh init
    assert len({g["lr"] for g in second.engine.optimizer.param_groups}) > 1      # muP groups
    # the padded layout: one row per document, same entry point, loss finite and falling into the same range
    mod = importlib.reload(mod)
    configure(mod, common + ["--set", "MAX_STEPS=3", "--set", "BATCH_LAYOUT='padded'", "--set", "SAMPLES_PER_BATCH=4",
                             "--set", "WARMUP_RATIO=0.34", "--set", "VAL_FRACTION=0.0", "--set", "SAMPLE_INTERVAL=0"])
    third = mod.main()
    assert third.global_step == 3 and third.loss_ema is not None and 3.0 < third.loss_ema < 7.0


def test_padded_and_packed_layouts_give_the_same_step():
    """The same documents as one packed row, as one padded batch and as a padded batch split into micro-batches:
    identical loss, gradient norm, token count and (up to summation order) parameters after the step."""
    from kohakuwullm_b200.data.loader.padded import collate_padded, split_padded
    from kohakuwullm_b200.data.packing import collate_packed
    from kohakuwullm_b200.models import LMBackbone, get_preset
    from kohakuwullm_b200.training.engine import TrainEngine

    def model():
        torch.manual_seed(0)
        return LMBackbone(get_preset("B200-smoke", vocab_size=300, dim=64, depth=2, heads=2, kv_heads=1, head_dim=32,
                                     mlp_hidden=128, sliding_window=8, global_layer_every=2, attn_sink=True))

    g = torch.Generator().manual_seed(3)
    docs = [torch.randint(0, 300, (int(torch.randint(5, 40, (1,), generator=g)),), generator=g) for _ in range(6)]
    results = []
    for batches in ([collate_packed(docs)], [collate_padded(docs)], split_padded(collate_padded(docs, pad_to_multiple=8), 3)):
        eng = TrainEngine(model(), lr=1e-2, max_grad_norm=1.0)
        out = eng.step(batches)
        flat = torch.cat([p.detach().reshape(-1) for p in eng.model.parameters()])
        results.append((float(out["loss"]), float(out["grad_norm"]), float(out["tokens"]), flat))
    for loss, norm, tokens, flat in results[1:]:
        assert abs(loss - results[0][0]) < 1e-5 and abs(norm - results[0][1]) < 1e-4 and tokens == results[0][2]
        torch.testing.assert_close(flat, results[0][3], rtol=0, atol=3e-4)
    cut = collate_padded(docs, max_length=16)
    assert cut.tokens.shape[1] == 16 and int(cut.lengths.max()) == 16


def test_every_shipped_config_names_only_knobs_of_its_entry_point(monkeypatch):
    """A config is applied with unknown keys refused, so loading each shipped file against the entry point its
    docstring names proves that no recipe carries a stale or misspelt knob; model presets must exist, schedules must
    build, source and renderer specs must name registered kinds."""
    import glob
    import importlib

    from kohakuwullm_b200.models import get_preset
    from kohakuwullm_b200.registry import DATASET, RENDERER
    from kohakuwullm_b200.utils.config import apply_overrides, load_config_file
    from kohakuwullm_b200.utils.misc import autofill_schedule_steps

    import kohakuwullm_b200.data  # noqa: F401  (registrations)

    monkeypatch.setenv("KWU_SWEEP", "12288x21_mxfp8_ckpt")
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "configs", "lm")
    files = [f for f in sorted(glob.glob(os.path.join(root, "**", "*.py"), recursive=True))
             if not os.path.basename(f).startswith("_")]
    assert len(files) >= 15
    for path in files:
        text = open(path).read()
        entry = "train_lm_pipe" if "cli.train_lm_pipe" in text else "train_lm"
        module = importlib.import_module(f"kohakuwullm_b200.cli.{entry}")
        knobs = {k: v for k, v in vars(module).items() if k.isupper()}
        apply_overrides(knobs, load_config_file(path), path)          # raises on an unknown knob
        get_preset(knobs["PRESET"], **knobs["ARCH_OVERRIDES"])
        if knobs.get("LR_SCHEDULE"):
            f = build_schedule(autofill_schedule_steps(dict(knobs["LR_SCHEDULE"]), knobs["MAX_STEPS"], knobs["WARMUP_STEPS"]))
            assert 0.0 < f(knobs["MAX_STEPS"] - 1) <= 1.0 and f(knobs["WARMUP_STEPS"]) > 0.5, path
        for src in knobs.get("SOURCES") or []:
            assert src["records"]["name"] in DATASET and src["repeat"] > 0, path
        r = knobs.get("RENDERER")
        names = [r] if isinstance(r, str) else [r["name"], *r.get("renderers", {}).values()]
        assert all(n in RENDERER for n in names), path
        if knobs.get("SCHEDULE"):
            from kohakuwullm_b200.pipe.schedules import SCHEDULES
            assert knobs["SCHEDULE"] in SCHEDULES, path
    sweep = load_config_file(os.path.join(root, "sweep", "microbatch.py"))
    assert (sweep["MICRO_TOKENS"], sweep["NUM_MICROBATCHES"]) == (12288, 21)
    assert sweep["ARCH_OVERRIDES"]["mxfp8"] and sweep["ARCH_OVERRIDES"]["grad_ckpt"] and sweep["SCHEDULE"] == "1f1b"
    monkeypatch.setenv("KWU_SWEEP", "8192x32_fp7")
    with pytest.raises(ValueError):
        load_config_file(os.path.join(root, "sweep", "microbatch.py"))


def test_every_entry_point_knob_is_named_in_the_configuration_guide():
    import importlib
    import re

    doc = open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "docs", "configs.md")).read()
    for entry in ("train_lm", "train_lm_pipe"):
        mod = importlib.import_module(f"kohakuwullm_b200.cli.{entry}")
        knobs = [k for k in vars(mod) if k.isupper() and not k.startswith("_")]
        missing = [k for k in knobs if not re.search(rf"\b{k}\b", doc)]
        assert not missing, f"{entry}: knobs without a mention in docs/configs.md: {missing}"
