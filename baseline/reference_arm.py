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


def run_reference(args, micro_tokens, grad_accum, len_min, len_max, metric, ClockSampler, timed, dist_setup):
    if not (REF / "kohakuwullm").is_dir():
        _unavailable("baseline/_ref is not installed (pip install --no-index --no-deps --target baseline/_ref <reference checkout>)")
    sys.path.insert(0, str(REF))
    _install_shims()
    try:
        import torch
        from torch.nn.parallel import DistributedDataParallel

        from kohakuwullm.bench import make_packs, make_tokens, trained_tokens
        from kohakuwullm.models import LMBackbone, get_preset
        from kohakuwullm.models.mxfp8_swap import refresh_mxfp8_weights, swap_mxfp8
        from kohakuwullm.training.optim.build import build_optimizer
        from kohakuwullm.training.optim.lowbit import cast_parameters_
    except Exception as e:  # noqa: BLE001
        _unavailable(f"reference import failed: {type(e).__name__}: {e}")

    rank, world, local = dist_setup(args.gpus)
    dev = torch.device("cuda", local)
    use_mxfp8 = not args.no_mxfp8
    try:
        torch.manual_seed(1234)
        # torch 2.11's varlen_attn has no ``enable_gqa`` argument, so the reference's default "varlen"
        # backend cannot run here; its own Triton flash-attention backend is selected instead.
        cfg = get_preset("Kohaku-500M", depth=24, mlp_hidden=3584, rope_theta=500000.0, attn=args.ref_attn)
        # fp32 parameters under bf16 autocast with fused AdamW: the reference harness's default arm
        # (its FusedAdamW refuses 16-bit parameters)
        model = LMBackbone(cfg).to(device=dev, dtype=torch.float32)
        expect_refresh = 0
        if use_mxfp8:
            report = swap_mxfp8(model)
            if report.blocking:
                raise RuntimeError(f"mxfp8 swap incomplete: {report.blocking}")
            expect_refresh = len(report.modules)

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
        opt = build_optimizer(wrapped, name="fused_adamw", lr=1e-4)

        budget = micro_tokens * grad_accum
        infos = make_packs(budget, micro_tokens, len_min, len_max, dev, 17 + rank)
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
        print(json.dumps({
            "impl": "reference", "metric": metric, "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_dev / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16+mxfp8" if use_mxfp8 else "bf16", "data": "synthetic",
            "config": {"model": "dense-546M (Kohaku-500M + depth 24, ffn 3584, theta 5e5)",
                       "global_batch": tokens_per_step, "seq_len": micro_tokens, "grad_accum": grad_accum,
                       "parallelism": f"dp{world}"},
            "clocks": clocks,
            "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": max(ms_e2e, wall_e2e) / args.steps,
                    "h2d_bytes_per_step": int(ids_host.numel() * 8 * 2), "d2h_bytes_per_step": 4},
            "final_loss": last.get("host"),
        }))
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()
