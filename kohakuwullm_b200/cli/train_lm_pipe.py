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
VIRTUAL_STAGES = 2          # model chunks per rank under the looped multi-chunk schedules (the V-shaped ones use 2)
LAYERS: list | None = None
AUTOTUNE = True
AUTOTUNE_DOC_LEN = 2048     # document length of the probe batch the layer costs are measured on
HEAD_ONLY_STAGE = True     # the measured split may leave the last stage with the final norm and the head only
LEN_MIN, LEN_MAX = 64, 4096
DATA = "synthetic"          # "synthetic", a corpus directory, or use SOURCES
SOURCES: list = []          # [{"records": <record spec>, "repeat": 1.0, "source": "tag"}, ...]
RENDERER = "plain"
TOKENIZER = "byte"          # "byte" or a Hugging Face tokenizer path
CTX_MAX = 4096
DOC_FILTER: str | dict = ""  # "ngram" (share of repeated 4-grams), "consecutive" (back-to-back n-gram runs), or {"name": .., **args}
LR_SCHEDULE: dict = {"mode": "cosine", "warmup": None, "end": None, "min_value": 0.1}
WARMUP_STEPS = 100
WARMUP_RATIO = 0.0                          # > 0: the warm-up is this share of MAX_STEPS (overrides WARMUP_STEPS)
PARAM_DTYPE = "bf16"                        # "bf16" (the native kernels), "fp32", or "fp16" (PyTorch paths + loss scaler)
AUX_LOSS_WEIGHT: float | None = None        # overrides the preset's router auxiliary-loss weight
ROUTER_Z_LOSS_WEIGHT: float | None = None
BIAS_SCHEDULE: dict | None = None           # schedule of the routers' bias update rate, e.g. {"mode": "linear", "end": 2000}
GRAD_SCALER = "auto"                        # loss scaling for fp16 parameters ("auto": on for fp16 only), "on", "off"
GRAD_SCALER_INIT = 65536.0
CHECKPOINT_PATH = ""                        # weights only (RESUME restores optimizer, scheduler and counters too)
SAMPLE_INTERVAL = 0                         # > 0: collective preview decode every N steps
SAMPLE_PROMPTS: list = []                   # [(name, prompt), ...]
SAMPLE_TOKENS = 64
SAMPLE_TEMPERATURE = 0.35
SAMPLE_TOP_P = 0.95
SAMPLE_TOP_K = 0
SAMPLE_MIN_P = 0.0
SAMPLE_COUNT = 4                            # completions per prompt
SAMPLE_FROM_BATCH = 0                       # > 0: also continue that many documents cut out of the batch just trained on
SAMPLE_PREFIX_TOKENS = 768                  # longest prefix kept of such a document
SAMPLE_PREFIX_FRAC = 0.25                   # where a document without turn structure is cut
SAMPLE_TURNS_ONLY = True                    # cut chat documents at a turn boundary (the assistant answers)
SAMPLE_LOCAL = True                         # True: gather the weights and decode on rank 0; False: pipelined decode
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
GPUS = 0                    # > 1 and not under a launcher: spawn that many ranks on this machine (no restarts)
BACKEND: str | None = None
WANDB_PROJECT = ""          # a Weights & Biases project name turns the W&B sink on (rank 0)
WANDB_MODE = "offline"      # these machines have no network: sync the run directory later
RUN_NAME = ""
RUN_ID = ""                 # continue this Weights & Biases run (a resumed training keeps one curve)
PROGRESS_BAR = False        # a step-driven progress bar on rank 0
HEARTBEAT = 0.0             # > 0: ranks beat into a store of their own; a peer silent for this many seconds (or one that
                            # announced its exit) ends the run between two steps, before the next collective is launched
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
    arch = dict(ARCH_OVERRIDES)
    router_kw = dict(arch.get("moe_router_kwargs") or get_preset(PRESET).moe_router_kwargs or {})
    if AUX_LOSS_WEIGHT is not None:
        router_kw["aux_loss_weight"] = AUX_LOSS_WEIGHT
    if ROUTER_Z_LOSS_WEIGHT is not None:
        router_kw["z_loss_weight"] = ROUTER_Z_LOSS_WEIGHT
    if router_kw:
        arch["moe_router_kwargs"] = router_kw
    cfg = get_preset(PRESET, **arch)
    costs = None
    if AUTOTUNE and LAYERS is None:
        measured = measure_costs(cfg, MICRO_TOKENS, ranks.device, doc_len=AUTOTUNE_DOC_LEN) if ranks.rank == 0 else None
        costs = broadcast_costs(measured, cfg.depth, ranks.device)
    chunks = 2 if SCHEDULE in ("zbv", "dualpipe-v") else \
        max(int(VIRTUAL_STAGES), 2) if SCHEDULE in ("interleaved-1f1b", "looped-bfs", "interleaved-zb") else 1
    plans = plan_for(cfg, ranks.world_size * chunks, MICRO_TOKENS, layers=LAYERS, costs=costs,
                     style="v" if SCHEDULE in ("zbv", "dualpipe-v") else "loop",
                     allow_empty_last=HEAD_ONLY_STAGE and costs is not None)
    log.info("plan", split=[p.num_layers for p in plans])
    log.info("plan_detail", text="\n" + describe(plans))
    from kohakuwullm_b200.utils.reporters import build_reporter

    reporter = build_reporter(WANDB_PROJECT or None, RUN_NAME or None, {"preset": PRESET, **ARCH_OVERRIDES},
                              METRICS_JSONL or None, CONSOLE_INTERVAL, WANDB_MODE, run_id=RUN_ID or None,
                              directory=CKPT_DIR or None) if ranks.rank == 0 else None
    from kohakuwullm_b200.utils.misc import autofill_schedule_steps

    warmup = max(1, round(WARMUP_RATIO * MAX_STEPS)) if WARMUP_RATIO > 0 else WARMUP_STEPS
    sched = autofill_schedule_steps(dict(LR_SCHEDULE), MAX_STEPS, warmup) if LR_SCHEDULE else None
    dtypes = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": None}
    if PARAM_DTYPE not in dtypes:
        raise ValueError(f"PARAM_DTYPE must be one of {sorted(dtypes)}, not {PARAM_DTYPE!r}")
    module = LMPipelineModule(cfg, micro_tokens=MICRO_TOKENS, lr=LR, weight_decay=WEIGHT_DECAY, seed=SEED,
                              param_dtype=dtypes[PARAM_DTYPE], optimizer=OPTIMIZER,
                              optimizer_kwargs=dict(OPTIMIZER_KWARGS), lr_schedule=sched)
    scaler = None
    if GRAD_SCALER == "on" or (GRAD_SCALER == "auto" and PARAM_DTYPE == "fp16" and ranks.device.type == "cuda"):
        from kohakuwullm_b200.pipe.scaler import PipelineGradScaler

        scaler = PipelineGradScaler(init_scale=GRAD_SCALER_INIT)
    trainer = PipelineTrainer(module, plans, rank=ranks.rank, world=ranks.world_size, device=ranks.device,
                              n_micro=NUM_MICROBATCHES, schedule=SCHEDULE, max_grad_norm=MAX_GRAD_NORM, scaler=scaler,
                              callbacks=[LossLog(LOG_INTERVAL, reporter=reporter),
                                         Throughput(LOG_INTERVAL, reporter=reporter)])
    tok = None
    use_corpus = DATA != "synthetic" or bool(SOURCES)
    if use_corpus or (SAMPLE_INTERVAL > 0 and (SAMPLE_PROMPTS or SAMPLE_FROM_BATCH)):      # previews need a tokenizer on synthetic packs too
        from kohakuwullm_b200.data import ByteTokenizer

        if TOKENIZER == "byte":
            tok = ByteTokenizer()
        else:
            from transformers import AutoTokenizer

            tok = AutoTokenizer.from_pretrained(TOKENIZER)
    if HEARTBEAT > 0 and ranks.world_size > 1:
        from kohakuwullm_b200.utils.heartbeat import HeartbeatCallback, RankHeartbeat

        hb = RankHeartbeat.from_env(interval=max(HEARTBEAT / 10.0, 0.05), timeout=HEARTBEAT)
        trainer.loop.callbacks.callbacks.append(HeartbeatCallback(hb))
    if PROGRESS_BAR:
        from kohakuwullm_b200.pipe.callbacks import ProgressBar

        trainer.loop.callbacks.callbacks.append(ProgressBar(MAX_STEPS))
    if BIAS_SCHEDULE:
        from kohakuwullm_b200.training.parallel.uwupipe_callbacks import RouterBiasSchedule

        trainer.loop.callbacks.callbacks.append(RouterBiasSchedule(module, dict(BIAS_SCHEDULE)))
    if SAMPLE_INTERVAL > 0 and (SAMPLE_PROMPTS or SAMPLE_FROM_BATCH) and tok is not None:
        from kohakuwullm_b200.training.parallel.uwupipe_callbacks import SamplePreview

        trainer.loop.callbacks.callbacks.append(SamplePreview(
            module, tok, [tuple(p) for p in SAMPLE_PROMPTS], every_n_steps=SAMPLE_INTERVAL, max_new_tokens=SAMPLE_TOKENS,
            temperature=SAMPLE_TEMPERATURE, top_p=SAMPLE_TOP_P, top_k=SAMPLE_TOP_K, min_p=SAMPLE_MIN_P,
            samples=SAMPLE_COUNT, from_batch=SAMPLE_FROM_BATCH, prefix_tokens=SAMPLE_PREFIX_TOKENS,
            prefix_frac=SAMPLE_PREFIX_FRAC,
            turns_only=SAMPLE_TURNS_ONLY, local=SAMPLE_LOCAL, report=getattr(reporter, "samples", None)))
    if CKPT_DIR:
        trainer.loop.callbacks.callbacks.append(Checkpoint(trainer, CKPT_DIR, every=CKPT_EVERY))
    if RESUME:
        trainer.load_checkpoint(RESUME)
    elif CHECKPOINT_PATH:
        from kohakuwullm_b200.pipe import checkpoint as ckpt

        for stage in module.stages:            # weights only: this rank's slice of the whole-model checkpoint
            ckpt.load(CHECKPOINT_PATH, stage, None, names=module.global_names(), strict=False)

    def stream():
        step = trainer.loop.global_step
        while True:  # identical on every rank: the seed depends on the step only
            yield make_packs(NUM_MICROBATCHES, MICRO_TOKENS, LEN_MIN, LEN_MAX, cfg.vocab_size, seed=SEED + step)
            step += 1

    if not use_corpus:
        batches = stream()
    else:
        # every rank iterates the SAME micro-batched loader (stage 0 uses the tokens, the last stage the labels)
        from kohakuwullm_b200.data import build_dataset, build_loader
        from kohakuwullm_b200.data.filters import build_doc_filter

        spec = {"name": "mixture", "sources": SOURCES, "seed": SEED} if SOURCES else {"name": "corpus", "root": DATA}
        records, renderer = build_dataset(spec, RENDERER)
        batches = build_loader("pipeline", records, renderer, lambda s: tok.encode(s), k=MICRO_TOKENS, m=MICRO_TOKENS // 16,
                               num_microbatches=NUM_MICROBATCHES, ctx_max=CTX_MAX, seed=SEED,
                               doc_filter=build_doc_filter(DOC_FILTER),
                               bos=getattr(tok, "bos_token_id", None), eos=getattr(tok, "eos_token_id", None))
    trainer.fit(batches, MAX_STEPS)
    if CKPT_DIR:
        trainer.save_checkpoint(os.path.join(CKPT_DIR, "last.ckpt"))
    if reporter is not None:
        reporter.finish()
    shutdown()
    return trainer


if __name__ == "__main__":
    from kohakuwullm_b200.utils.config import configure

    configure(sys.modules[__name__], sys.argv[1:])
    from kohakuwullm_b200.utils.launch import maybe_self_launch

    if not maybe_self_launch("kohakuwullm_b200.cli.train_lm_pipe", GPUS):
        main()
