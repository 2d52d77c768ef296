"""Reference arm of ``bench.py``: the UNMODIFIED reference package (installed under ``baseline/_ref``)
driven through its own public API and stock code path, for the same metric and config.

The step mirrors what the reference's own end-to-end harness does
(scripts/bench/e2e/step_throughput.py:100-195): ``LMBackbone(cfg)`` (fp32 parameters) ->
``swap_mxfp8`` -> ``build_optimizer("fused_adamw")`` -> per micro-batch ``loss(reduction="sum")`` under
bf16 autocast, ``(loss/total).backward()``, DDP ``no_sync`` on all but the last micro-batch,
``opt.step()``, ``refresh_mxfp8_weights``. Synthetic packs come from the reference's own
``kohakuwullm.bench.make_packs`` / ``make_tokens``. Nothing of this framework's models, kernels or
engine is on this path.

Import shims (the reference itself is not touched): the reference targets torch >= 2.13 and imports
``torch.nn.modules.linear_cross_entropy_options`` at module import time (only used by its
``kernel="torch"`` head, which this run does not select), and its ``bench`` package imports matplotlib
for plotting. Both names are registered as empty stand-in modules before the import.
"""

from __future__ import annotations

import contextlib
import dataclasses
import json
import os
import sys
import types
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"


def _unavailable(why: str) -> None:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why.replace("\n", " ")[:300]}))
    sys.exit(0)


def _install_shims() -> None:
    name = "torch.nn.modules.linear_cross_entropy_options"
    try:
        __import__(name)
    except ImportError:
        mod = types.ModuleType(name)

        @dataclasses.dataclass
        class LinearCrossEntropyOptions:  # only reached by kernel="torch", never selected here
            pass

        mod.LinearCrossEntropyOptions = LinearCrossEntropyOptions
        sys.modules[name] = mod
    try:
        import matplotlib  # noqa: F401
    except ImportError:
        class _Anything(types.ModuleType):
            def __getattr__(self, item):
                if item.startswith("__"):
                    raise AttributeError(item)
                return _Anything(f"{self.__name__}.{item}")

            def __call__(self, *a, **k):
                return None

        for sub in ("matplotlib", "matplotlib.pyplot", "matplotlib.ticker", "matplotlib.colors",
                    "matplotlib.lines", "matplotlib.patches", "matplotlib.cm"):
            sys.modules[sub] = _Anything(sub)


# ------------------------------------------------------------------------------------------------ configs
# The benchmark configurations expressed against the reference's own presets and config fields
# (src/kohakuwullm/models/presets.py:12-152, :278-371). "2" is what ``bench.py --impl reference`` runs.
REF_CONFIGS = {
    "2": dict(label="dense-546M (Kohaku-500M + depth 24, ffn 3584, theta 5e5)", preset="Kohaku-500M",
              overrides=dict(depth=24, mlp_hidden=3584, rope_theta=500000.0),
              micro_tokens=4096, accum=4, len_min=64, len_max=4096, log_uniform=False),
    # 991M-class DeepSeekMoE, data parallel, 8192-token packs (experts replicated: the reference has no EP)
    "3p": dict(label="moe-991M (Kohaku-MoE-1B + dim 1024, 16/4 heads, top-6, 2 shared, dense ffn 2816)",
               preset="Kohaku-MoE-1B",
               overrides=dict(dim=1024, heads=16, kv_heads=4, moe_top_k=6, moe_num_shared=2, mlp_hidden=2816,
                              moe_router_kwargs={"score_func": "sigmoid"}),
               micro_tokens=8192, accum=4, len_min=64, len_max=4096, log_uniform=False),
    # the same model under pipeline parallelism: 16 micro-batches of 4096 tokens, 1F1B (needs >= 2 GPUs)
    "3": dict(label="moe-991M under pipeline parallelism", preset="Kohaku-MoE-1B",
              overrides=dict(dim=1024, heads=16, kv_heads=4, moe_top_k=6, moe_num_shared=2, mlp_hidden=2816,
                             moe_router_kwargs={"score_func": "sigmoid"}),
              micro_tokens=4096, accum=16, len_min=64, len_max=4096, log_uniform=False, pipeline=True),
    # sliding-window 1.1B: the reference has ONE sink logit per head (attention.py:75), not four
    "5": dict(label="sliding-1.1B (Kohaku-1B + depth 28, 24/8 heads, window 1024 x3 + global, sink, YaRN x4)",
              preset="Kohaku-1B",
              overrides=dict(depth=28, heads=24, kv_heads=8, mlp_hidden=4096, sliding_window=1024,
                             global_layer_every=4, attn_sink=True, rope_scaling="yarn", rope_factor=4.0,
                             max_position=4096, attn="mxfp8"),
              micro_tokens=16384, accum=1, len_min=128, len_max=16384, log_uniform=True),
}


def _log_uniform_lengths(total: int, lo: int, hi: int, seed: int) -> list[int]:
    """Document lengths drawn log-uniform in [lo, hi], the last one cut so that they sum to ``total``."""
    import math
    import random

    rng = random.Random(seed)
    out, left = [], total
    while left > 0:
        n = int(round(math.exp(rng.uniform(math.log(lo), math.log(hi)))))
        n = max(2, min(n, left))
        if left - n == 1:      # a one-token tail document would carry no target
            n += 1
        out.append(n)
        left -= n
    return out


def _set_moe_device(torch) -> str:
    """The reference's fused expert planner refuses a card it has no measured description of
    (kernels/moe/tune.py:51-61) and says to pass one: do that, from this pool's measured peaks."""
    from kohakuwullm.kernels.gemm.device import Device
    from kohakuwullm.kernels.moe import tune

    peaks = {"bf16_tflops_sustained": 1388.6, "hbm_gbs": 6552.3}
    try:
        peaks.update(json.loads((ROOT / "MEASURED_PEAKS.json").read_text()))
    except (OSError, ValueError):
        pass
    # Device.query reads a property name that torch 2.11 spells differently (L2_cache_size), so the
    # description is filled in field by field through the public constructor
    p = torch.cuda.get_device_properties(torch.cuda.current_device())
    dev = Device(name=p.name, sms=p.multi_processor_count,
                 regs_per_sm=getattr(p, "regs_per_multiprocessor", 65536),
                 smem_per_cta=getattr(p, "shared_memory_per_block_optin", 227 * 1024),
                 smem_per_sm=getattr(p, "shared_memory_per_multiprocessor", 228 * 1024),
                 max_threads_per_sm=getattr(p, "max_threads_per_multi_processor", 2048),
                 l2_bytes=getattr(p, "L2_cache_size", getattr(p, "l2_cache_size", 126 * 2 ** 20)),
                 mma_peak=float(peaks["bf16_tflops_sustained"]), dram_bw=float(peaks["hbm_gbs"]),
                 l2_bw=3.0 * float(peaks["hbm_gbs"]))
    tune.set_device(dev)
    return dev.name


def run_reference(args, micro_tokens, grad_accum, len_min, len_max, metric, ClockSampler, timed, dist_setup):
    """Entry point of ``bench.py --impl reference``: configuration 2 with the micro-batch shape bench.py names."""
    spec = dict(REF_CONFIGS["2"], micro_tokens=micro_tokens, accum=grad_accum, len_min=len_min, len_max=len_max)
    run_reference_config(spec, args, metric, ClockSampler, timed, dist_setup)


def run_reference_config(spec, args, metric, ClockSampler, timed, dist_setup):
    if not (REF / "kohakuwullm").is_dir():
        _unavailable("baseline/_ref is not installed (pip install --no-index --no-deps --target baseline/_ref <reference checkout>)")
    sys.path.insert(0, str(REF))
    _install_shims()
    try:
        import torch
        from torch.nn.parallel import DistributedDataParallel

        from kohakuwullm.bench import make_packs, make_tokens, trained_tokens
        from kohakuwullm.models import LMBackbone, get_preset
        from kohakuwullm.models.components.moe import MoEMLP
        from kohakuwullm.models.components.seqinfo import SeqInfo
        from kohakuwullm.models.mxfp8_swap import refresh_mxfp8_weights, swap_mxfp8
        from kohakuwullm.training.optim.build import build_optimizer
        from kohakuwullm.training.optim.lowbit import cast_parameters_
    except Exception as e:  # noqa: BLE001
        _unavailable(f"reference import failed: {type(e).__name__}: {e}")

    micro_tokens, grad_accum = spec["micro_tokens"], spec["accum"]
    rank, world, local = dist_setup(args.gpus)
    dev = torch.device("cuda", local)
    use_mxfp8 = not args.no_mxfp8
    ref_dtype = getattr(args, "ref_dtype", "fp32")
    moe_path = getattr(args, "mxfp8_moe", "unfused")
    notes = []
    if spec.get("pipeline"):
        return _run_reference_pipeline(spec, args, metric, ClockSampler, timed, rank, world, local)
    try:
        torch.manual_seed(1234)
        overrides = dict(spec["overrides"])
        # torch 2.11's varlen_attn has no ``enable_gqa`` argument, so the reference's default "varlen"
        # backend cannot run here; its own Triton flash-attention backend is selected instead.
        overrides.setdefault("attn", args.ref_attn)
        if args.no_mxfp8 and overrides.get("attn") == "mxfp8":
            overrides["attn"] = args.ref_attn
        cfg = get_preset(spec["preset"], **overrides)
        cfg.max_position = max(cfg.max_position, micro_tokens) if overrides.get("rope_scaling") is None else cfg.max_position
        # fp32 parameters under bf16 autocast with fused AdamW is the reference harness's default arm (its
        # FusedAdamW refuses 16-bit parameters); --ref-dtype bf16 is its 16-bit arm (cast_parameters_ + adamw16)
        model = LMBackbone(cfg).to(device=dev, dtype=torch.float32)
        opt_name = "fused_adamw"
        if ref_dtype == "bf16":
            cast_parameters_(model, torch.bfloat16)
            opt_name = "adamw16"
        has_moe = any(isinstance(m, MoEMLP) for m in model.modules())
        if has_moe:
            notes.append(f"moe planner device: {_set_moe_device(torch)}")
        expect_refresh = 0
        if use_mxfp8:
            for m in model.modules():
                if isinstance(m, MoEMLP):
                    m.mxfp8_expert_path = moe_path
            report = swap_mxfp8(model)
            if report.blocking:
                raise RuntimeError(f"mxfp8 swap incomplete: {report.blocking}")
            expect_refresh = len(report.modules)
        if getattr(args, "ref_compile", False):
            # the reference harness's own --compile option: per-block torch.compile, reduce-overhead mode
            for i, block in enumerate(model.blocks):
                model.blocks[i] = torch.compile(block, mode="reduce-overhead")
            notes.append("blocks compiled (reduce-overhead)")

        class LossModule(torch.nn.Module):
            def __init__(self, backbone):
                super().__init__()
                self.backbone = backbone

            def forward(self, ids, labels, info):
                with torch.autocast("cuda", dtype=torch.bfloat16):
                    loss, _ = self.backbone.loss(ids, labels, info, reduction="sum")
                return loss

        wrapped = LossModule(model)
        if world > 1:
            wrapped = DistributedDataParallel(wrapped, device_ids=[local])
        opt = build_optimizer(wrapped, name=opt_name, lr=1e-4)

        budget = micro_tokens * grad_accum
        if spec.get("log_uniform"):
            infos = [SeqInfo.from_lengths(torch.tensor(_log_uniform_lengths(micro_tokens, spec["len_min"],
                                                                            spec["len_max"], 17 + rank + 1000 * i)),
                                          device=dev)
                     for i in range(grad_accum)]
        else:
            infos = make_packs(budget, micro_tokens, spec["len_min"], spec["len_max"], dev, 17 + rank)
        ids, labels = make_tokens(infos, cfg.vocab_size, dev, 17 + rank)
        total = float(trained_tokens(labels))
        if world > 1:
            import torch.distributed as dist

            t = torch.tensor([total], device=dev)
            dist.all_reduce(t)
            total = float(t.item())
        ids_host, labels_host = ids.cpu().pin_memory(), labels.cpu().pin_memory()
        last = {}

        def run_step(ids_d, labels_d):
            opt.zero_grad(set_to_none=True)
            for i, info in enumerate(infos):
                lo, hi = i * micro_tokens, (i + 1) * micro_tokens
                is_last = i == len(infos) - 1
                ctx = contextlib.nullcontext() if (world == 1 or is_last) else wrapped.no_sync()
                with ctx:
                    loss = wrapped(ids_d[lo:hi], labels_d[lo:hi], info)
                    (loss * world / total).backward()
                last["loss"] = loss.detach()
            opt.step()
            if use_mxfp8:
                got = refresh_mxfp8_weights(model)
                if got != expect_refresh:
                    raise RuntimeError(f"refreshed {got} modules, expected {expect_refresh}")

        def step_device():
            run_step(ids, labels)

        def step_e2e():
            run_step(ids_host.to(dev, non_blocking=True), labels_host.to(dev, non_blocking=True))
            last["host"] = float(last["loss"])  # device->host read of the step result

        for _ in range(args.warmup):
            step_e2e()
        torch.cuda.synchronize()
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        ms_dev, _ = timed(step_device, args.steps, world)
        ms_e2e, wall_e2e = timed(step_e2e, args.steps, world)
        clocks = sampler.stop() if rank == 0 else {}
    except Exception as e:  # noqa: BLE001
        if world > 1:
            import torch.distributed as dist

            if dist.is_initialized():
                dist.destroy_process_group()
        _unavailable(f"reference run failed: {type(e).__name__}: {e}")

    tokens_per_step = micro_tokens * grad_accum * world
    if rank == 0:
        value = tokens_per_step * args.steps / (ms_dev / 1e3)
        e2e = tokens_per_step * args.steps / (max(ms_e2e, wall_e2e) / 1e3)
        dtype = ("bf16+mxfp8" if use_mxfp8 else "bf16") + ("" if ref_dtype == "fp32" else " (bf16 parameters)")
        print(json.dumps({
            "impl": "reference", "metric": metric, "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_dev / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": dtype, "data": "synthetic",
            "config": {"model": spec["label"],
                       "global_batch": tokens_per_step, "seq_len": micro_tokens, "grad_accum": grad_accum,
                       "parallelism": f"dp{world}", "notes": notes,
                       "mxfp8_moe": moe_path if (use_mxfp8 and has_moe) else None},
            "clocks": clocks,
            "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": max(ms_e2e, wall_e2e) / args.steps,
                    "h2d_bytes_per_step": int(ids_host.numel() * 8 * 2), "d2h_bytes_per_step": 4},
            "final_loss": last.get("host"),
        }))
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


def _run_reference_pipeline(spec, args, metric, ClockSampler, timed, rank, world, local):
    """The reference's torch-pipelining path (scripts/bench/e2e/step_throughput.py:223-294): its own
    ``build_stage`` (analytic split + head calibration), ``build_schedule`` (1F1B), ``run_step`` and stage-local
    optimizer, one stage per rank."""
    import torch
    import torch.distributed as dist

    if world < 2:
        _unavailable("the pipeline configuration needs at least 2 GPUs")
    dev = torch.device("cuda", local)
    use_mxfp8 = not args.no_mxfp8
    micro_tokens, n_micro = spec["micro_tokens"], spec["accum"]
    try:
        from kohakuwullm.bench import make_packs, make_tokens, trained_tokens
        from kohakuwullm.models import get_preset
        from kohakuwullm.models.components.moe import MoEMLP
        from kohakuwullm.models.mxfp8_swap import refresh_mxfp8_weights, swap_mxfp8
        from kohakuwullm.training.parallel.pipeline_lightning import (build_schedule, build_stage, run_step,
                                                                     stage_local_optimizer)

        torch.manual_seed(1234)
        overrides = dict(spec["overrides"])
        overrides.setdefault("attn", args.ref_attn)
        cfg = get_preset(spec["preset"], **overrides)
        cfg.max_position = max(cfg.max_position, micro_tokens)
        _set_moe_device(torch)
        module, stage, plan, _ = build_stage(cfg, rank, world, dev, micro_tokens, autocast_dtype=torch.bfloat16,
                                             param_dtype=torch.float32, seq_len=micro_tokens)
        inner = getattr(module, "module", module)
        expect_refresh = 0
        if use_mxfp8:
            for m in inner.modules():
                if isinstance(m, MoEMLP):
                    m.mxfp8_expert_path = getattr(args, "mxfp8_moe", "unfused")
            swapped = swap_mxfp8(inner)
            if swapped.blocking:
                raise RuntimeError(f"mxfp8 swap incomplete: {swapped.blocking}")
            expect_refresh = len(swapped.modules)
        opt = stage_local_optimizer(module, name="fused_adamw", lr=1e-4)
        infos = make_packs(micro_tokens * n_micro, micro_tokens, spec["len_min"], spec["len_max"], dev, 17)
        ids, labels = make_tokens(infos, cfg.vocab_size, dev, 17)
        total = trained_tokens(labels)

        def loss_fn(hidden, target):
            loss, _ = module.loss(hidden, target)
            return loss / total

        schedule = build_schedule(stage, n_micro, loss_fn=loss_fn, kind="1f1b")

        def step():
            opt.zero_grad(set_to_none=True)
            module.set_seq_info(infos)
            run_step(schedule, rank, world, tokens=ids, targets=labels)
            opt.step()
            if use_mxfp8:
                got = refresh_mxfp8_weights(module)
                if got != expect_refresh:
                    raise RuntimeError(f"refreshed {got} modules, expected {expect_refresh}")

        for _ in range(args.warmup):
            step()
        torch.cuda.synchronize()
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        ms_dev, _ = timed(step, args.steps, world)
        clocks = sampler.stop() if rank == 0 else {}
    except Exception as e:  # noqa: BLE001
        if dist.is_initialized():
            dist.destroy_process_group()
        _unavailable(f"reference pipeline run failed: {type(e).__name__}: {e}")
    tokens_per_step = micro_tokens * n_micro
    if rank == 0:
        print(json.dumps({
            "impl": "reference", "metric": metric, "value": tokens_per_step * args.steps / (ms_dev / 1e3),
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_dev / args.steps, "higher_is_better": True, "scaling": "strong",
            "dtype": "bf16+mxfp8" if use_mxfp8 else "bf16", "data": "synthetic",
            "config": {"model": spec["label"], "global_batch": tokens_per_step, "seq_len": micro_tokens,
                       "grad_accum": n_micro, "parallelism": f"pp{world}", "schedule": "1f1b"},
            "clocks": clocks,
        }))
    dist.destroy_process_group()


def main(argv=None) -> None:
    """``python -m baseline.reference_arm --config {2,3,3p,5} --gpus N``: the reference on one benchmark
    configuration (under ``torch.distributed.run`` for N > 1), same JSON line as ``bench.py --impl reference``."""
    import argparse

    sys.path.insert(0, str(ROOT))
    import bench

    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="2", choices=sorted(REF_CONFIGS))
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--ref-attn", default="triton")
    ap.add_argument("--no-mxfp8", action="store_true")
    ap.add_argument("--ref-dtype", default="fp32", choices=["fp32", "bf16"])
    ap.add_argument("--ref-compile", action="store_true")
    # "unfused" by default: on this image (Triton 3.6, sm_100) the reference's fused MXFP8 expert kernels fail to
    # compile ("PassManager::run failed" in kernels/mxfp8/experts.py), its unfused path is the one that runs
    ap.add_argument("--mxfp8-moe", default="unfused", choices=["fused", "unfused"])
    args = ap.parse_args(argv)
    args.warmup = max(args.warmup, 3)
    run_reference_config(REF_CONFIGS[args.config], args, bench.METRIC, bench.ClockSampler, bench._timed,
                         bench._dist_setup)


if __name__ == "__main__":
    main()
