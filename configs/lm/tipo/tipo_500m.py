"""Prompt-optimisation model on the dense Kohaku-500M, data parallel on 8 B200, full caption mixture.

    python -m kohakuwullm_b200.cli.train_lm --config configs/lm/tipo/tipo_500m.py            # spawns GPUS ranks
    torchrun --nproc-per-node 8 -m kohakuwullm_b200.cli.train_lm --config configs/lm/tipo/tipo_500m.py

MXFP8 linears; Muon on the hidden matrices with AdamW on gains, embedding and head (an axis indexed by token id has
no singular values to equalise). Untied embeddings: tying serves two objectives with one matrix and only holds up on a
very large corpus. The model needs the 65536-id tokenizer built by ``cli/build_tokenizer.py``.
"""

import os
import runpy

_src = runpy.run_path(os.path.join(os.path.dirname(os.path.abspath(__file__)), "_sources.py"))

PRESET = "Kohaku-500M"
ARCH_OVERRIDES = {"max_position": 4096, "rope_theta": 100000.0, "qk_norm": True, "tie_embeddings": False, "mxfp8": True}

SOURCES = _src["caption_sources"]()
RENDERER = "tipo"
TOKENIZER = "models/tokenizer"
NUM_WORKERS = 8
CTX_MAX = 2048
BATCH_TOKENS = 32768            # per rank and micro-batch; 8 ranks x 2 = 524288 tokens per optimizer step
GRAD_ACCUM = 2
VAL_FRACTION = 0.002
VAL_INTERVAL = 2000

GPUS = 8
OPTIMIZER = "muon"
OPTIMIZER_KWARGS = {"muon_lr": 0.02}
GRAD_SYNC = "nccl"              # the fused peer-memory step shards the flat AdamW only
GRAD_COMPRESS = "bf16"          # gradient buckets cross NVLink in bf16
LR = 3e-4
BETAS = (0.9, 0.95)
WEIGHT_DECAY = 0.1
MAX_GRAD_NORM = 1.0
MAX_STEPS = 40_000              # about one weighted pass (~19 B trained tokens)
WARMUP_STEPS = 400
LR_SCHEDULE = {"mode": "cosine", "warmup": None, "end": None, "min_value": 0.05}

RUN_NAME = "tipo-500m"
WANDB_PROJECT = "kohakuwullm-b200"
LOG_INTERVAL = 20
CKPT_DIR = "out/ckpt/tipo-500m"
CKPT_EVERY = 5000
SAMPLE_INTERVAL = 2000
SAMPLE_PROMPTS = ["target: <|long|>\ntags: 1girl, solo, outdoors, cherry blossoms\nlong: "]
SAMPLE_TOKENS = 128
