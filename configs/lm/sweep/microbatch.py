"""Micro-batch sweep of the pipeline path at a fixed 262144-token optimizer step: one point per run, chosen with the
``KWU_SWEEP`` environment variable as ``<micro_tokens>x<microbatches>[_mxfp8][_ckpt][_<schedule>]``.

    KWU_SWEEP=8192x32        torchrun --nproc-per-node 8 -m kohakuwullm_b200.cli.train_lm_pipe --config configs/lm/sweep/microbatch.py
    KWU_SWEEP=16384x16_mxfp8 torchrun --nproc-per-node 8 -m kohakuwullm_b200.cli.train_lm_pipe --config configs/lm/sweep/microbatch.py
    KWU_SWEEP=8192x32_dualpipe-v ...

The points the reference publishes are 4096x64, 8192x32, 12288x21, 14336x18, 16384x16 and 32768x8, with MXFP8 experts,
activation checkpointing or the V-shaped schedule as variants; any other ``AxB`` works the same way. Every point runs
60 steps on synthetic packs and writes its per-step metrics to ``out/sweep/<point>.jsonl``; read them with
``python -m kohakuwullm_b200.bench.plotting out/sweep --metrics train/loss throughput/tokens_per_s --out out/sweep/curves.svg``.
"""

import os
import re

POINTS = ("4096x64", "8192x32", "12288x21", "14336x18", "16384x16", "32768x8")
SCHEDULES = ("gpipe", "1f1b", "interleaved-1f1b", "looped-bfs", "interleaved-zb", "zbv", "dualpipe-v")


def parse_point(text: str) -> dict:
    m = re.fullmatch(r"(\d+)x(\d+)((?:_[a-z0-9-]+)*)", text)
    if not m:
        raise ValueError(f"KWU_SWEEP={text!r}: expected <micro_tokens>x<microbatches>[_mxfp8][_ckpt][_<schedule>]")
    flags = [f for f in m.group(3).split("_") if f]
    unknown = [f for f in flags if f not in ("mxfp8", "ckpt") + SCHEDULES]
    if unknown:
        raise ValueError(f"KWU_SWEEP={text!r}: unknown part(s) {unknown}")
    schedule = next((f for f in flags if f in SCHEDULES), "1f1b")
    return {"micro_tokens": int(m.group(1)), "microbatches": int(m.group(2)), "mxfp8": "mxfp8" in flags,
            "ckpt": "ckpt" in flags, "schedule": schedule}


def config_gen() -> dict:
    name = os.environ.get("KWU_SWEEP", "8192x32")
    p = parse_point(name)
    return {
        "PRESET": "Kohaku-MoE-1B",
        "ARCH_OVERRIDES": {"max_position": 4096, "rope_theta": 100000.0, "qk_norm": True, "tie_embeddings": False,
                           "grad_ckpt": p["ckpt"], "mxfp8": p["mxfp8"]},
        "AUX_LOSS_WEIGHT": 0.0,
        "ROUTER_Z_LOSS_WEIGHT": 0.0,
        "DATA": "synthetic",
        "LEN_MIN": 64,
        "LEN_MAX": min(2048, p["micro_tokens"]),
        "MICRO_TOKENS": p["micro_tokens"],
        "NUM_MICROBATCHES": p["microbatches"],
        "SCHEDULE": p["schedule"],
        "AUTOTUNE": True,
        "OPTIMIZER": "muon",
        "OPTIMIZER_KWARGS": {"muon_lr": 2e-3, "embed_lr": 2e-3},
        "LR": 5e-4,
        "MAX_STEPS": 60,
        "WARMUP_STEPS": 10,
        "LOG_INTERVAL": 10,
        "RUN_NAME": f"sweep-{name}",
        "METRICS_JSONL": f"out/sweep/{name}.jsonl",
    }
