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
RENDERER = "plain"
TOKENIZER = "byte"              # "byte" or a Hugging Face tokenizer path
BATCH_TOKENS = 16384            # tokens per rank per optimizer step
GRAD_ACCUM = 4
CTX_MAX = 4096
LEN_MIN, LEN_MAX = 64, 4096
OPTIMIZER = "fused_adamw"      # or muon, adamw16, stochastic_adamw, adamw8bit, adamw4bit, adamwfp8, adamw, adam, sgd
OPTIMIZER_KWARGS: dict = {}     # e.g. {"muon_lr": 0.02}
GRAD_SYNC = "auto"             # fused (reduce-scatter + AdamW + all-gather over peer memory) with fused_adamw on GPUs, else nccl
EXPERT_PARALLEL = False        # split the experts of every MoE layer over the ranks (the rest stays data parallel)
EP_CAPACITY = 2.0
EP_ON_OVERFLOW = "raise"       # or "count": drop pairs that find no room and report ep_dropped_pairs
LR = 3e-4
WEIGHT_DECAY = 0.1
BETAS = (0.9, 0.95)
MAX_GRAD_NORM = 1.0
WARMUP_STEPS = 100
MAX_STEPS = 1000
LR_SCHEDULE = {"mode": "cosine", "warmup": None, "end": None, "min_value": 0.1}
LOG_INTERVAL = 10
CKPT_DIR = ""
CKPT_EVERY = 1000
RESUME = ""
SEED = 1234
DEVICE = "auto"
WANDB_PROJECT = ""          # a Weights & Biases project name turns the W&B sink on (rank 0)
WANDB_MODE = "offline"      # these machines have no network: sync the run directory later
RUN_NAME = ""
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
    sched = autofill_schedule_steps(dict(LR_SCHEDULE), MAX_STEPS, WARMUP_STEPS)
    trainer = LMTrainer(PRESET, dict(ARCH_OVERRIDES), lr=LR, betas=BETAS, weight_decay=WEIGHT_DECAY,
                        max_grad_norm=MAX_GRAD_NORM, grad_accum=GRAD_ACCUM, lr_schedule=sched, device=device,
                        log_interval=LOG_INTERVAL, seed=SEED, optimizer=OPTIMIZER, optimizer_kwargs=dict(OPTIMIZER_KWARGS),
                        grad_sync=GRAD_SYNC, expert_parallel=EXPERT_PARALLEL, ep_capacity_factor=EP_CAPACITY,
                        ep_on_overflow=EP_ON_OVERFLOW)
    if DATA == "synthetic":
        loader = _synthetic_stream(trainer.config.vocab_size, rank)
    else:
        from kohakuwullm_b200.data import ByteTokenizer, build_dataset, build_loader

        records, renderer = build_dataset({"name": "corpus", "root": DATA}, RENDERER)
        if TOKENIZER == "byte":
            tok = ByteTokenizer()
        else:
            from transformers import AutoTokenizer

            tok = AutoTokenizer.from_pretrained(TOKENIZER)
        loader = build_loader("ddp", records, renderer, lambda s: tok.encode(s), rank=rank, world=world,
                              k=BATCH_TOKENS, m=BATCH_TOKENS // 16, ctx_max=CTX_MAX, seed=SEED,
                              bos=getattr(tok, "bos_token_id", None), eos=getattr(tok, "eos_token_id", None))
    from kohakuwullm_b200.utils.reporters import build_reporter

    reporter = build_reporter(WANDB_PROJECT or None, RUN_NAME or None, {"preset": PRESET}, METRICS_JSONL or None, 0,
                              WANDB_MODE, directory=CKPT_DIR or None)
    callbacks = [ThroughputCallback(interval=LOG_INTERVAL * 2, reporter=reporter)]
    trainer.callbacks.callbacks.extend(callbacks)
    if CKPT_DIR:
        trainer.callbacks.callbacks.append(Checkpoint(trainer, CKPT_DIR, every=CKPT_EVERY))
    if RESUME:
        trainer.load_checkpoint(RESUME, loader if hasattr(loader, "load_state_dict") else None)
    trainer.fit(loader, MAX_STEPS)
    if CKPT_DIR:
        trainer.save_checkpoint(os.path.join(CKPT_DIR, "last.ckpt"))
    if world > 1:
        dist.destroy_process_group()
    return trainer


if __name__ == "__main__":
    from kohakuwullm_b200.utils.config import configure

    configure(sys.modules[__name__], sys.argv[1:])
    main()
