"""Bench harness arithmetic that needs no GPU: contention statistics, per-step run logs, sweep classification,
the analytic FLOP budget and the preset ladder."""

import io
import json
import os
import tempfile

import pytest
import torch

from kohakuwullm_b200.bench import contention, flops_analytic, ladder, runlog, sweep


def test_contention_statistics_and_power():
    quiet = [1.0 + 0.002 * (i % 5) for i in range(200)]
    v = contention.verdict(quiet)
    assert v["verdict"] == "clean" and v["certifiable"]
    shared = quiet[:190] + [1.5] * 10                    # 5 % of the samples ran behind somebody else's kernel
    assert contention.contended_fraction(shared) == pytest.approx(0.05)
    assert contention.verdict(shared)["verdict"] == "contended: discard"
    # 20-microsecond work: the timer floor alone explains a 25 % spread, so no verdict is possible
    assert not contention.spread_has_power(0.02) and contention.spread_has_power(1.0)
    assert "too short" in contention.verdict([0.02] * 200)["verdict"]
    assert "too short" in contention.verdict(quiet[:20])["verdict"]     # too few samples for a 1 % limit
    assert contention.contended_fraction_min_iters() == 100
    assert contention.percentile([1.0, 2.0, 3.0], 0.5) == 2.0


def test_runlog_round_trip_and_clock_verdict():
    buf = io.StringIO()
    buf.write(runlog.HEADER + "\n")
    elapsed, step = 0.0, 0
    for flush in range(40):                               # 40 flushes of 10 steps, 0.5 s per step
        pending = []
        for _ in range(10):
            step += 1
            pending.append((step, step * 1000, 990, torch.tensor(990.0 * 2.5), torch.tensor(1.25), 3e-4, elapsed))
        elapsed += 5.0
        last = runlog.write_step_rows(buf, pending, elapsed)
        assert last[0] == pytest.approx(2.5) and last[2] == elapsed
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "run.csv")
        open(path, "w").write(buf.getvalue())
        run = runlog.load_run(path)
    assert run["step"][-1] == 400 and isinstance(run["tokens"][0], int)
    times = runlog.step_times(run)
    assert len(times) >= runlog.MIN_TIMING_STEPS and all(abs(t - 0.5) < 1e-6 for t in times)
    v = runlog.clock_verdict(run)
    assert v["admissible"] and v["tokens_per_s"] == pytest.approx(2000.0)
    short = {k: vals[:150] for k, vals in run.items()}
    assert not runlog.clock_verdict(short)["admissible"]


def test_sweep_rows_are_clean_contended_or_oom():
    assert sweep.parse_tag("dp8_bf16_mxfp8_ckpt") == {"strategy": "dp8_ckpt", "dtype": "bf16", "optimizer": None,
                                                      "flags": ["mxfp8", "ckpt"], "unknown": []}
    assert sweep.parse_tag("pp4_fp16_muon_weird")["unknown"] == ["weird"]
    with tempfile.TemporaryDirectory() as tmp:
        rows = {"a.json": {"preset": "X", "n_gpus": 1, "tokens_per_s": 1000.0},
                "b.json": {"preset": "X", "n_gpus": 2, "tokens_per_s": 1900.0, "step_spread": 0.4},
                "c.json": {"preset": "X", "n_gpus": 4, "ok": False},
                "d.json": {"config": {"model": "Y"}, "n_gpus": 1, "value": 5.0, "clocks": {"reasons": ["hw_slowdown"]}}}
        for name, payload in rows.items():
            json.dump(payload, open(os.path.join(tmp, name), "w"))
        got = {r["file"]: r["status"] for r in sweep.load_rows(tmp)}
        assert got == {"a.json": "clean", "b.json": "contended", "c.json": "oom", "d.json": "contended"}
        assert "| c.json | X | 4 | oom | - |" in sweep.table(sweep.load_rows(tmp))


def test_analytic_flops_agree_with_the_model_based_counter():
    from kohakuwullm_b200.models import LMBackbone, get_preset
    from kohakuwullm_b200.models.flops import FlopCounter

    assert flops_analytic.causal_pairs_per_token(100, 100, None) == pytest.approx(50.5)
    assert flops_analytic.causal_pairs_per_token(100, 100, 10) == pytest.approx((100 * 10 - 45) / 100)
    for name, kw in (("B200-smoke", {}), ("Kohaku-MoE-1B", {"depth": 3, "vocab_size": 1024})):
        cfg = get_preset(name, mxfp8=False, **kw)
        with torch.device("meta"):
            model = LMBackbone(cfg)
        budget = flops_analytic.flop_budget(cfg, len_min=256, len_max=256)
        model_flops, _ = FlopCounter(model).step_flops([256])
        # forward + backward of GEMMs and attention (the counter charges attention backward 2x, this budget 2.5x)
        matrix_3x = budget.gemm_fwd * 3 + budget.attn_fwd * 3
        assert matrix_3x == pytest.approx(model_flops / 256, rel=0.02), name
    b = flops_analytic.flop_budget("B200-dense-546M")
    assert 0.98 < b.matrix_share < 1.0 and 3.0e9 < b.total < 4.5e9


def test_ladder_census_counts_active_parameters():
    rows = ladder.ladder(("Kohaku-200M", "Kohaku-MoE-1B"))
    dense, moe = rows
    assert not dense.sparse and dense.total == dense.active
    assert moe.sparse and moe.active < moe.total / 3 and moe.router > 0
    assert "Kohaku-MoE-1B" in ladder.render(rows)


def test_plotting_svg_is_well_formed_and_complete(tmp_path):
    """The dependency-free plotter: stable colours, SI labels, round ticks, and an SVG that parses as XML and holds
    one shape per data point; a configuration that was not run leaves a gap, not a zero-height bar."""
    import xml.etree.ElementTree as ET

    from kohakuwullm_b200.bench import plotting as pl

    pal = pl.Palette()
    assert pal.color("ours") == pal.color("ours") != pal.color("reference")
    assert [pl.si_format(v) for v in (1536, 2e6, 0.25, 7, 1.4e12)] == ["1.5k", "2M", "0.25", "7", "1.4T"]
    ticks = pl.nice_ticks(0.0, 181_000.0)
    assert ticks[0] == 0.0 and ticks[-1] >= 181_000 and len(set(round(b - a, 6) for a, b in zip(ticks, ticks[1:]))) == 1
    assert pl.log_ticks(1, 8, 2.0) == [1, 2, 4, 8]

    rows = []
    for impl, scale in (("ours", 180e3), ("reference", 44e3)):
        for n in (1, 2, 8):
            if impl == "reference" and n == 8:
                continue                                            # never run: must not be drawn as a zero
            rows.append({"impl": impl, "n_gpus": n, "value": scale * n * (0.97 if n > 1 else 1.0), "status": "clean",
                         "file": f"{impl}_{n}.json", "config": {"model": "Kohaku-500M"}})
    rows.append({"impl": "ours", "n_gpus": 4, "value": 1.0, "status": "contended", "file": "bad.json"})
    fig = pl.scaling_figure(rows)
    root = ET.fromstring(fig.svg())
    ns = "{http://www.w3.org/2000/svg}"
    assert len(root.findall(f"{ns}circle")) == 2 * (3 + 2)          # value and efficiency panels, solid lines only
    assert len(root.findall(f"{ns}polyline")) == 3 * 2              # value + ideal + efficiency per series
    bars = pl.throughput_figure(rows)
    root = ET.fromstring(bars.svg())
    drawn = [r for r in root.iter(f"{ns}rect") if r.find(f"{ns}title") is not None]
    assert len(drawn) == 5 and all(float(r.get("height")) > 0 for r in drawn)
    out = pl.save_figure(bars, str(tmp_path / "plots" / "throughput.png"))
    assert out.endswith("throughput.svg") and os.path.getsize(out) > 500

    # the command line reads result files the way the sweep reader does
    import json as _json
    for r in rows:
        with open(tmp_path / r["file"], "w") as fh:
            fh.write(_json.dumps({k: v for k, v in r.items() if k not in ("status", "file")}) + "\n")
    assert pl.main([str(tmp_path), "--scaling", "--out", str(tmp_path / "scaling.svg")]) == 0
    ET.parse(tmp_path / "scaling.svg")
    empty = pl.Figure()
    assert "no data" in empty.svg()
    # per-step metric files of the trainers' JSONL sink: one panel per metric, one line per run, cut lines skipped
    for name, shift in (("a", 0.0), ("b", 0.01)):
        with open(tmp_path / f"{name}.jsonl", "w") as fh:
            for step in range(2, 12, 2):
                fh.write(_json.dumps({"step": step, "t": 0.1 * step, "train/loss": 11.15 - 0.001 * step + shift}) + "\n")
                fh.write(_json.dumps({"step": step, "t": 0.1 * step, "throughput/tokens_per_s": 1000.0 + step}) + "\n")
            fh.write('{"step": 12, "train/lo')
    runs = pl.load_metric_curves(str(tmp_path))
    assert sorted(runs) == ["a", "b"] and runs["a"]["train/loss"][0] == [2, 4, 6, 8, 10]
    assert pl.main([str(tmp_path), "--metrics", "train/loss", "throughput/tokens_per_s", "--out", str(tmp_path / "curves.svg")]) == 0
    root = ET.parse(tmp_path / "curves.svg").getroot()
    assert len(root.findall(f"{ns}polyline")) == 4
    labels = [t.text for t in root.iter(f"{ns}text")]
    assert len({x for x in labels if x and x.startswith("11.")}) >= 3        # distinct tick labels on a flat curve


def test_mxfp8_exponent_rules_and_emulated_linear():
    """Round-up never saturates; round-to-nearest picks the same scale or one binade smaller and clips the block's
    largest elements. The emulated linear under the round-up rule is the MXFP8 reference forward, and its gradients
    stay close to the unquantised ones."""
    from kohakuwullm_b200.bench import mxfp8_rounding as rd
    from kohakuwullm_b200.ops import mxfp8 as mx

    g = torch.Generator().manual_seed(0)
    x = torch.randn(48, 256, generator=g) * torch.logspace(-3, 3, 48)[:, None]
    q_up, e_up = mx.quantize_reference(x, "ceil")
    q_nr, e_nr = mx.quantize_reference(x, "nearest")
    d = e_up.int() - e_nr.int()
    assert set(d.unique().tolist()) == {0, 1}
    # round-up: the scaled block maximum is in (224, 448]; the 448 code appears only where the maximum is exact
    assert float(q_up.float().abs().max()) <= 448.0
    scaled_max = (x.view(48, 8, 32).abs().amax(-1) / torch.pow(2.0, e_up.float() - 127.0))
    assert bool(((scaled_max > 224.0 - 1e-3) & (scaled_max <= 448.0)).all())
    stats = rd.block_statistics(x)
    assert 0.3 < stats["blocks_with_smaller_scale"] < 0.7
    assert stats["saturated_share_nearest"] > stats["saturated_share_ceil"]
    with pytest.raises(ValueError):
        mx.quantize_reference(x, "floor")

    w = torch.randn(64, 256, generator=g) * 0.05
    xs = torch.randn(3, 5, 256, generator=g)
    assert torch.equal(rd.emulated_mxfp8_linear(xs, w, "ceil"), mx.mxfp8_linear_reference(xs, w))
    for rule in rd.RULES:
        a, b = xs.clone().requires_grad_(), w.clone().requires_grad_()
        rd.emulated_mxfp8_linear(a, b, rule).square().sum().backward()
        a2, b2 = xs.clone().requires_grad_(), w.clone().requires_grad_()
        (a2 @ b2.t()).square().sum().backward()
        rel = lambda u, v: float((u - v).norm() / v.norm())
        bound = 0.08 if rule == "ceil" else 0.2      # clipping the block maxima costs more than a coarser step
        assert rel(a.grad, a2.grad) < bound and rel(b.grad, b2.grad) < bound, rule


def test_mxfp8_emulation_swaps_in_place_and_restores():
    from kohakuwullm_b200.bench import mxfp8_rounding as rd
    from kohakuwullm_b200.models import LMBackbone, get_preset
    from kohakuwullm_b200.models.seqinfo import SeqInfo

    torch.manual_seed(0)
    cfg = get_preset("B200-smoke", vocab_size=128, dim=64, depth=2, heads=2, kv_heads=2, head_dim=32, mlp_hidden=128,
                     mxfp8=False)
    model = LMBackbone(cfg).eval()
    ids = torch.randint(0, 128, (2, 9))
    info = SeqInfo.padded(2, 9)
    with torch.no_grad():
        plain = model(ids, info)
        n_all = rd.emulate_mxfp8_(model, "ceil")
        up = model(ids, info)
        rd.restore_(model)
        n_attn = rd.emulate_mxfp8_(model, "nearest", scope=("attn.",))
        near = model(ids, info)
        rd.restore_(model)
        again = model(ids, info)
    assert n_all > n_attn > 0
    assert torch.equal(plain, again)
    assert not torch.equal(plain, up) and not torch.equal(up, near)
    assert float((up - plain).norm() / plain.norm()) < 0.1
    args = type("A", (), dict(vocab=64, dim=64, depth=1, lr=2e-3, steps=6, window=3, device="cpu"))()
    data = rd.chain_data(2, 4, 17, 64, 0)
    first = rd.train_arm("ceil", 0, args, data)
    assert first == rd.train_arm("ceil", 0, args, data)            # an arm is a function of its seed
    assert first != rd.train_arm("nearest", 0, args, data)


def test_lost_update_nearest_freezes_where_stochastic_moves(tmp_path):
    """At a learning rate far below half an ulp per step, round-to-nearest leaves nearly every bf16 weight
    bit-identical while stochastic rounding moves a visible share; at the peak rate both move."""
    from kohakuwullm_b200.bench import lost_update as lu

    p = torch.tensor([1.0, 0.5, 3.0], dtype=torch.bfloat16)
    assert torch.allclose(lu.half_ulp(p), torch.tensor([2.0 ** -8, 2.0 ** -9, 2.0 ** -7]))
    assert torch.allclose(lu.half_ulp(p.to(torch.float16)), torch.tensor([2.0 ** -11, 2.0 ** -12, 2.0 ** -10]))
    assert not lu.decay_survives(3e-4, 0.1, torch.bfloat16) and lu.decay_survives(3e-2, 0.5, torch.bfloat16)
    rc = lu.main(["--steps", "6", "--dim", "64", "--depth", "1", "--vocab", "64", "--rows", "4", "--length", "17",
                  "--batches", "4", "--lrs", "3e-3", "3e-7", "--arms", "nearest", "stochastic", "--device", "cpu",
                  "--out", str(tmp_path)])
    assert rc == 0
    rows = {(r["arm"], r["lr"]): r for r in json.load(open(tmp_path / "lost_update.json"))}
    assert rows[("nearest", 3e-7)]["never_moved"] > 0.97
    assert rows[("stochastic", 3e-7)]["never_moved"] < rows[("nearest", 3e-7)]["never_moved"] - 0.01
    assert rows[("nearest", 3e-3)]["never_moved"] < 0.2 and rows[("nearest", 3e-3)]["updates_above_half_ulp"] > 0.5
    assert os.path.getsize(tmp_path / "lost_update.svg") > 500


def test_stage_memory_accounts_every_parameter_once():
    """The per-stage estimate is built on the meta device: stage parameter counts add up to the whole model, the
    flat fused AdamW costs 12 bytes per parameter (divided by the data-parallel size), the quantised-state optimizers
    cost what the optimizer itself reports, and a card that is too small is reported as not fitting."""
    from kohakuwullm_b200.bench import stage_memory as sm
    from kohakuwullm_b200.models import LMBackbone, get_preset

    kw = dict(vocab_size=1024, dim=256, depth=6, heads=4, kv_heads=2, head_dim=64, mlp_hidden=512)
    cfg = get_preset("B200-smoke", **kw)
    with torch.device("meta"):
        whole = sum(p.numel() for p in LMBackbone(cfg, init=False).parameters())
    rows = sm.stage_rows("B200-smoke", 3, overrides=kw, optimizer="fused_adamw", mxfp8=True)
    assert len(rows) == 3 and abs(sum(r["params_m"] for r in rows) * 1e6 - whole) < 1
    for r in rows:
        n = r["params_m"] * 1e6
        assert abs(r["optimizer_gib"] * 2 ** 30 - 12 * n) < 1 and abs(r["grads_gib"] * 2 ** 30 - 4 * n) < 1
        assert 2 * n <= r["weights_gib"] * 2 ** 30 < 2.1 * n          # bf16 except the few fp32 gains
        assert r["mxfp8_gib"] > 0 and r["fits"]
    sharded = sm.stage_rows("B200-smoke", 3, overrides=kw, optimizer="fused_adamw", dp=8)
    assert abs(sharded[0]["optimizer_gib"] * 8 - rows[0]["optimizer_gib"]) < 1e-6
    small = sm.stage_rows("B200-smoke", 1, overrides=kw, card_gib=0.001)
    assert not small[0]["fits"] and small[0]["left_gib"] < 0
    assert sm.main(["--preset", "B200-smoke", "--set", "depth=2", "--card-gib", "0.0001"]) == 1

    # the state model of the quantised optimizers against the optimizer's own accounting
    from kohakuwullm_b200.training.optim.quantized_state import QuantizedStateAdamW

    p = torch.nn.Parameter(torch.randn(300, 256))
    p.grad = torch.randn_like(p)
    for name, fmt in (("adamw8bit", "int8"), ("adamw4bit", "int4"), ("adamwfp8", "fp8")):
        opt = QuantizedStateAdamW([p], state_format=fmt)
        opt.step()
        assert opt.state_bytes() == sm.optimizer_state_bytes([("w", p)], name), name
    with pytest.raises(ValueError):
        sm.optimizer_state_bytes([("w", p)], "lion")


@pytest.mark.timeout(120)
def test_loader_throughput_bench_counts_tokens_in_process_and_with_workers(capsys):
    """The data-path benchmark on a small synthetic corpus: one row per worker count with a positive rate and packs
    filled close to the budget, for the byte tokenizer and for a BPE trained on the corpus itself."""
    from kohakuwullm_b200.bench import loader_throughput as lt

    assert lt.main(["--documents", "300", "--doc-chars", "400", "--workers", "0", "2", "--seconds", "0.4",
                    "--pack-tokens", "2048", "--ctx-max", "1024"]) == 0
    rows = [json.loads(line) for line in capsys.readouterr().out.splitlines() if line.startswith("{")]
    runs = [r for r in rows if "workers" in r]
    assert [r["workers"] for r in runs] == [0, 2]
    assert all(r["tokens_per_s"] > 1e4 and 0.8 < r["fill"] <= 1.0 for r in runs)
    assert rows[-1]["best_tokens_per_s"] == max(r["tokens_per_s"] for r in runs)
    assert lt.main(["--documents", "200", "--doc-chars", "400", "--workers", "0", "--seconds", "0.3", "--pack-tokens", "1024",
                    "--ctx-max", "512", "--tokenizer", "bpe:600"]) == 0
    bpe = [json.loads(line) for line in capsys.readouterr().out.splitlines() if '"workers"' in line][0]
    assert bpe["tokenizer"] == "bpe:600" and bpe["tokens_per_s"] > 1e3
