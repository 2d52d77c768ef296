"""Data-parallel LM training entry point.

    python -m kohakuwullm_b200.cli.train_lm --config configs/lm/smoke/debug.py --set MAX_STEPS=50
    torchrun --nproc-per-node 8 -m kohakuwullm_b200.cli.train_lm --config configs/lm/dense_546m.py

Knobs are the UPPER_CASE globals below; a config file overrides same-named globals and ``--set`` one
more (see ``kohakuwullm_b200.utils.config``). Reference: scripts/train/lm.py:48-421.
"""

from __future__ import annotations

import os
import sys

import torch
import torch.distributed as dist

PRESET = "Kohaku-500M"
ARCH_OVERRIDES: dict = {}
DATA = "synthetic"              # "synthetic" or a corpus directory (jsonl / txt shards)
SOURCES: list = []              # a mixture instead of DATA: [{"records": <record spec>, "repeat": 1.0, "source": "tag"}, ...]
RENDERER = "plain"              # a renderer name or spec ("plain", "chatml", "qa", "tipo", {"name": "per_source", ...})
NUM_WORKERS = 0                 # > 0: render + tokenise + pack in that many worker processes
PREFETCH_FACTOR = 4             # packs each worker process keeps ready ahead of the trainer
VAL_FRACTION = 0.0              # hold this share of the records out (hash split) and validate on it
VAL_INTERVAL = 500
VAL_BATCHES = 8
CHECKPOINT_PATH = ""            # load weights only from this checkpoint (RESUME also restores optimizer, counters, loader)
HEAD_KWARGS: dict = {}          # e.g. {"chunk": 4096}
GRAD_CKPT = False               # recompute every block in backward
USE_MUP = False                 # muP learning-rate / weight-decay groups relative to BASE_DIM
BASE_DIM = 256
SAMPLE_INTERVAL = 0             # > 0: decode SAMPLE_PROMPTS every N steps and log the text (and a W&B table)
SAMPLE_PROMPTS: list = []
SAMPLE_TOKENS = 64
SAMPLE_TEMPERATURE = 0.8
SAMPLE_TOP_P = 0.95
SAMPLE_TOP_K = 0
SAMPLE_MIN_P = 0.0
TOKENIZER = "byte"              # "byte" or a Hugging Face tokenizer path
BATCH_LAYOUT = "packed"         # "padded": one row per document (SAMPLES_PER_BATCH rows cut to CTX_MAX), eager launches and
                                # explicit-mask attention; same loss per token, for ablations and readable debugging
SAMPLES_PER_BATCH = 8
PAD_TOKEN_ID = 0
BATCH_TOKENS = 16384            # tokens per rank per optimizer step
GRAD_ACCUM = 4
CTX_MAX = 4096
DOC_FILTER: str | dict = ""     # "ngram" (share of repeated 4-grams), "consecutive" (back-to-back n-gram runs), or {"name": .., **args}
LEN_MIN, LEN_MAX = 64, 4096
OPTIMIZER = "fused_adamw"      # or muon, adamw16, stochastic_adamw, adamw8bit, adamw4bit, adamwfp8, adamw, adam, sgd
OPTIMIZER_KWARGS: dict = {}     # e.g. {"muon_lr": 0.02}
GRAD_SYNC = "auto"             # fused (reduce-scatter + AdamW + all-gather over peer memory) with fused_adamw on GPUs, else nccl
GRAD_COMPRESS = ""             # "bf16" / "fp16": NCCL gradient buckets cross the wire in that dtype (nccl sync only)
EXPERT_PARALLEL = False        # split the experts of every MoE layer over the ranks (the rest stays data parallel)
EP_CAPACITY = 2.0
EP_ON_OVERFLOW = "raise"       # or "count": drop pairs that find no room and report ep_dropped_pairs
LR = 3e-4
WEIGHT_DECAY = 0.1
BETAS = (0.9, 0.95)
EPS = 1e-8
MAX_GRAD_NORM = 1.0
WARMUP_STEPS = 100
WARMUP_RATIO = 0.0              # > 0: the warm-up is this share of MAX_STEPS (overrides WARMUP_STEPS)
MAX_STEPS = 1000
LR_SCHEDULE = {"mode": "cosine", "warmup": None, "end": None, "min_value": 0.1}
LOG_INTERVAL = 10
CKPT_DIR = ""
CKPT_EVERY = 1000
RESUME = ""
SEED = 1234
GPUS = 0                    # > 1 and not under a launcher: spawn that many ranks on this machine (no restarts)
DEVICE = "auto"
WANDB_PROJECT = ""          # a Weights & Biases project name turns the W&B sink on (rank 0)
WANDB_MODE = "offline"      # these machines have no network: sync the run directory later
RUN_NAME = ""
RUN_ID = ""                 # continue this Weights & Biases run (a resumed training keeps one curve)
PROGRESS_BAR = False        # a step-driven progress bar on rank 0
HEARTBEAT = 0.0             # > 0: ranks beat into a store of their own; a peer silent for this many seconds (or one that
                            # announced its exit) ends the run between two steps, before the next collective is launched
METRICS_JSONL = ""          # one JSON object per report


def _synthetic_stream(vocab, rank):
    from kohakuwullm_b200.data.synthetic import make_pack

    step = 0
    while True:
        yield make_pack(BATCH_TOKENS, LEN_MIN, LEN_MAX, vocab, seed=SEED * 7919 + step * 64 + rank)
        step += 1


def main():
    from kohakuwullm_b200.pipe.callbacks import Checkpoint
    from kohakuwullm_b200.training.loop.callbacks import ThroughputCallback
    from kohakuwullm_b200.training.loop.trainer import LMTrainer
    from kohakuwullm_b200.utils.misc import autofill_schedule_steps

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    use_cuda = torch.cuda.is_available() and DEVICE != "cpu"
    device = torch.device("cuda", local) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl" if use_cuda else "gloo", **({"device_id": device} if use_cuda else {}))
    warmup = max(1, round(WARMUP_RATIO * MAX_STEPS)) if WARMUP_RATIO > 0 else WARMUP_STEPS
    sched = autofill_schedule_steps(dict(LR_SCHEDULE), MAX_STEPS, warmup)
    arch = dict(ARCH_OVERRIDES)
    if GRAD_CKPT:
        arch["grad_ckpt"] = True
    opt_kwargs = dict(OPTIMIZER_KWARGS)
    if USE_MUP:
        opt_kwargs["mup_base_dim"] = BASE_DIM
    trainer = LMTrainer(PRESET, arch, lr=LR, betas=BETAS, weight_decay=WEIGHT_DECAY, head_kwargs=dict(HEAD_KWARGS) or None,
                        max_grad_norm=MAX_GRAD_NORM, grad_accum=GRAD_ACCUM, lr_schedule=sched, device=device,
                        log_interval=LOG_INTERVAL, seed=SEED, optimizer=("adamw" if USE_MUP and OPTIMIZER == "fused_adamw" else OPTIMIZER),
                        optimizer_kwargs=opt_kwargs,
                        grad_sync=GRAD_SYNC, expert_parallel=EXPERT_PARALLEL, ep_capacity_factor=EP_CAPACITY,
                        ep_on_overflow=EP_ON_OVERFLOW, grad_compress=GRAD_COMPRESS or None, eps=EPS)
    tok, val_loader = None, None
    if DATA == "synthetic" and not SOURCES:
        loader = _synthetic_stream(trainer.config.vocab_size, rank)
    else:
        from kohakuwullm_b200.data import ByteTokenizer, build_dataset, build_loader

        spec = {"name": "mixture", "sources": SOURCES, "seed": SEED} if SOURCES else {"name": "corpus", "root": DATA}
        records, renderer = build_dataset(spec, RENDERER)
        if TOKENIZER == "byte":
            tok = ByteTokenizer()
        else:
            from transformers import AutoTokenizer

            tok = AutoTokenizer.from_pretrained(TOKENIZER)
        encode = lambda s: tok.encode(s)  # noqa: E731
        from kohakuwullm_b200.data.filters import build_doc_filter

        common = dict(k=BATCH_TOKENS, m=BATCH_TOKENS // 16, ctx_max=CTX_MAX, seed=SEED, doc_filter=build_doc_filter(DOC_FILTER),
                      bos=getattr(tok, "bos_token_id", None), eos=getattr(tok, "eos_token_id", None))
        if VAL_FRACTION > 0:
            from kohakuwullm_b200.data.sources.records import SplitRecords

            held_out = SplitRecords(records, VAL_FRACTION, "val", SEED)
            records = SplitRecords(records, VAL_FRACTION, "train", SEED)
            val_loader = lambda: build_loader("ddp", held_out, renderer, encode, rank=rank, world=world, **common)  # noqa: E731
        if BATCH_LAYOUT not in ("packed", "padded"):
            raise ValueError(f"BATCH_LAYOUT must be 'packed' or 'padded', not {BATCH_LAYOUT!r}")
        if BATCH_LAYOUT == "padded":
            # whole documents, one per row; every rank reads its own stride of the records, epoch after epoch
            mine = [i for i in range(len(records)) if i % world == rank]
            view = type("RankShard", (), {"__len__": lambda self: len(mine),
                                          "__getitem__": lambda self, i: records[mine[i]]})()
            per_epoch = build_loader("map", view, renderer, encode, layout="padded", samples_per_batch=SAMPLES_PER_BATCH,
                                     ctx_max=CTX_MAX, pad_id=PAD_TOKEN_ID, seed=SEED + rank, num_workers=NUM_WORKERS,
                                     bos=common["bos"], eos=common["eos"])

            def _epochs():
                while True:
                    yield from per_epoch

            loader = _epochs()
        elif NUM_WORKERS > 0:
            loader = build_loader("workers", records, renderer, encode, rank=rank, world=world, workers=NUM_WORKERS,
                                  prefetch=PREFETCH_FACTOR, **common)
        else:
            loader = build_loader("ddp", records, renderer, encode, rank=rank, world=world, **common)
    from kohakuwullm_b200.utils.reporters import build_reporter

    reporter = build_reporter(WANDB_PROJECT or None, RUN_NAME or None, {"preset": PRESET}, METRICS_JSONL or None, 0,
                              WANDB_MODE, run_id=RUN_ID or None, directory=CKPT_DIR or None)
    callbacks = [ThroughputCallback(interval=LOG_INTERVAL * 2, reporter=reporter)]
    if HEARTBEAT > 0 and world > 1:
        from kohakuwullm_b200.utils.heartbeat import HeartbeatCallback, RankHeartbeat

        callbacks.append(HeartbeatCallback(RankHeartbeat.from_env(interval=max(HEARTBEAT / 10.0, 0.05), timeout=HEARTBEAT)))
    if PROGRESS_BAR:
        from kohakuwullm_b200.training.loop.callbacks import StepProgressBar

        callbacks.append(StepProgressBar(MAX_STEPS))
    if SAMPLE_INTERVAL > 0 and SAMPLE_PROMPTS and tok is not None:
        from kohakuwullm_b200.training.loop.callbacks import SampleLogCallback

        callbacks.append(SampleLogCallback(list(SAMPLE_PROMPTS), tok, SAMPLE_INTERVAL, SAMPLE_TOKENS, reporter,
                                           temperature=SAMPLE_TEMPERATURE, top_p=SAMPLE_TOP_P, top_k=SAMPLE_TOP_K,
                                           min_p=SAMPLE_MIN_P))
    if val_loader is not None:
        from kohakuwullm_b200.training.loop.callbacks import ValidationCallback

        callbacks.append(ValidationCallback(val_loader, VAL_INTERVAL, VAL_BATCHES, reporter))
    trainer.callbacks.callbacks.extend(callbacks)
    if CKPT_DIR:
        trainer.callbacks.callbacks.append(Checkpoint(trainer, CKPT_DIR, every=CKPT_EVERY))
    if RESUME:
        trainer.load_checkpoint(RESUME, loader if hasattr(loader, "load_state_dict") else None)
    elif CHECKPOINT_PATH:
        from kohakuwullm_b200.pipe import checkpoint as ckpt

        ckpt.load(CHECKPOINT_PATH, trainer.backbone, None, strict=False)      # weights only: a fresh optimizer and step count
        if trainer.engine.has_mxfp8:
            trainer.backbone.refresh_mxfp8()
    trainer.fit(loader, MAX_STEPS)
    if CKPT_DIR:
        trainer.save_checkpoint(os.path.join(CKPT_DIR, "last.ckpt"))
    if world > 1:
        dist.destroy_process_group()
    return trainer


if __name__ == "__main__":
    from kohakuwullm_b200.utils.config import configure

    configure(sys.modules[__name__], sys.argv[1:])
    from kohakuwullm_b200.utils.launch import maybe_self_launch

    if not maybe_self_launch("kohakuwullm_b200.cli.train_lm", GPUS):
        main()
