"""Pipeline-parallel LM training entry point (one process per GPU, e.g. under torchrun).

    torchrun --nproc-per-node 4 -m kohakuwullm_b200.cli.train_lm_pipe --config configs/lm/moe_991m_pipe.py

The stage split is measured at start-up: rank 0 times one block per distinct layer kind plus head and
embedding (``measure_costs``), broadcasts the vector, and every rank runs the same dynamic program.
``LAYERS`` pins an explicit split instead. Every rank builds the SAME micro-batched loader (stage 0 uses
the tokens, the last stage the labels). Reference: scripts/train/lm_pipe.py:198-533.
"""

from __future__ import annotations

import os
import sys

import torch

PRESET = "Kohaku-MoE-1B"
ARCH_OVERRIDES: dict = {}
MICRO_TOKENS = 4096
NUM_MICROBATCHES = 16
SCHEDULE = "1f1b"
LAYERS: list | None = None
AUTOTUNE = True
HEAD_ONLY_STAGE = True     # the measured split may leave the last stage with the final norm and the head only
LEN_MIN, LEN_MAX = 64, 4096
OPTIMIZER = "fused_adamw"      # or muon, adamw16, stochastic_adamw, adamw8bit, adamw4bit, adamwfp8, adamw, adam, sgd
OPTIMIZER_KWARGS: dict = {}
LR = 3e-4
WEIGHT_DECAY = 0.1
MAX_GRAD_NORM = 1.0
MAX_STEPS = 1000
LOG_INTERVAL = 10
CKPT_DIR = ""
CKPT_EVERY = 1000
RESUME = ""
SEED = 1234
BACKEND: str | None = None
WANDB_PROJECT = ""          # a Weights & Biases project name turns the W&B sink on (rank 0)
WANDB_MODE = "offline"      # these machines have no network: sync the run directory later
RUN_NAME = ""
METRICS_JSONL = ""          # one JSON object per report
CONSOLE_INTERVAL = 0


def main():
    from kohakuwullm_b200.data.synthetic import make_packs
    from kohakuwullm_b200.models import get_preset
    from kohakuwullm_b200.pipe import Checkpoint, LossLog, Throughput, describe, init_pipeline, shutdown
    from kohakuwullm_b200.pipe.trainer import PipelineTrainer
    from kohakuwullm_b200.training.parallel.autotune import broadcast_costs, measure_costs
    from kohakuwullm_b200.training.parallel.pipeline import plan_for
    from kohakuwullm_b200.training.parallel.uwupipe import LMPipelineModule
    from kohakuwullm_b200.utils.logging import get_logger

    log = get_logger("lm_pipe")
    ranks = init_pipeline(BACKEND)
    cfg = get_preset(PRESET, **ARCH_OVERRIDES)
    costs = None
    if AUTOTUNE and LAYERS is None:
        measured = measure_costs(cfg, MICRO_TOKENS, ranks.device) if ranks.rank == 0 else None
        costs = broadcast_costs(measured, cfg.depth, ranks.device)
    chunks = 2 if SCHEDULE in ("zbv", "dualpipe-v", "interleaved-1f1b", "looped-bfs", "interleaved-zb") else 1
    plans = plan_for(cfg, ranks.world_size * chunks, MICRO_TOKENS, layers=LAYERS, costs=costs,
                     style="v" if SCHEDULE in ("zbv", "dualpipe-v") else "loop",
                     allow_empty_last=HEAD_ONLY_STAGE and costs is not None)
    log.info("plan", split=[p.num_layers for p in plans])
    log.info("plan_detail", text="\n" + describe(plans))
    from kohakuwullm_b200.utils.reporters import build_reporter

    reporter = build_reporter(WANDB_PROJECT or None, RUN_NAME or None, {"preset": PRESET, **ARCH_OVERRIDES},
                              METRICS_JSONL or None, CONSOLE_INTERVAL, WANDB_MODE,
                              directory=CKPT_DIR or None) if ranks.rank == 0 else None
    module = LMPipelineModule(cfg, micro_tokens=MICRO_TOKENS, lr=LR, weight_decay=WEIGHT_DECAY, seed=SEED,
                              optimizer=OPTIMIZER, optimizer_kwargs=dict(OPTIMIZER_KWARGS))
    trainer = PipelineTrainer(module, plans, rank=ranks.rank, world=ranks.world_size, device=ranks.device,
                              n_micro=NUM_MICROBATCHES, schedule=SCHEDULE, max_grad_norm=MAX_GRAD_NORM,
                              callbacks=[LossLog(LOG_INTERVAL, reporter=reporter),
                                         Throughput(LOG_INTERVAL, reporter=reporter)])
    if CKPT_DIR:
        trainer.loop.callbacks.callbacks.append(Checkpoint(trainer, CKPT_DIR, every=CKPT_EVERY))
    if RESUME:
        trainer.load_checkpoint(RESUME)

    def stream():
        step = trainer.loop.global_step
        while True:  # identical on every rank: the seed depends on the step only
            yield make_packs(NUM_MICROBATCHES, MICRO_TOKENS, LEN_MIN, LEN_MAX, cfg.vocab_size, seed=SEED + step)
            step += 1

    trainer.fit(stream(), MAX_STEPS)
    if CKPT_DIR:
        trainer.save_checkpoint(os.path.join(CKPT_DIR, "last.ckpt"))
    if reporter is not None:
        reporter.finish()
    shutdown()
    return trainer


if __name__ == "__main__":
    from kohakuwullm_b200.utils.config import configure

    configure(sys.modules[__name__], sys.argv[1:])
    main()
