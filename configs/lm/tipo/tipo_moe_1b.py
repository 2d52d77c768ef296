"""Prompt-optimisation model on Kohaku-MoE-1B (991M total, 248M active), data parallel on 8 B200.

    torchrun --nproc-per-node 8 -m kohakuwullm_b200.cli.train_lm --config configs/lm/tipo/tipo_moe_1b.py

Every rank holds all experts; routed expert GEMMs and the dense projections run in MXFP8, routers balance by bias
updates (no auxiliary loss). ``tipo_moe_1b_ep.py`` shards the experts instead, ``tipo_moe_1b_pp4.py`` pipelines.
"""

import os
import runpy

_src = runpy.run_path(os.path.join(os.path.dirname(os.path.abspath(__file__)), "_sources.py"))

PRESET = "Kohaku-MoE-1B"
ARCH_OVERRIDES = {"max_position": 4096, "rope_theta": 100000.0, "qk_norm": True, "tie_embeddings": False, "mxfp8": True}

SOURCES = _src["caption_sources"]()
RENDERER = "tipo"
TOKENIZER = "models/tokenizer"
NUM_WORKERS = 8
CTX_MAX = 2048
BATCH_TOKENS = 16384
GRAD_ACCUM = 4
VAL_FRACTION = 0.002
VAL_INTERVAL = 2000

GPUS = 8
OPTIMIZER = "fused_adamw"
LR = 5e-4
WEIGHT_DECAY = 0.1
MAX_GRAD_NORM = 1.0
MAX_STEPS = 100_000
WARMUP_STEPS = 2000
LR_SCHEDULE = {"phases": [{"mode": "power", "end": 0.9, "s0": 2500, "b": -0.5, "warmup": None},
                          {"mode": "cosine", "end": 1.0, "min_value": 0.01}], "end": None}

RUN_NAME = "tipo-moe-1b"
WANDB_PROJECT = "kohakuwullm-b200"
LOG_INTERVAL = 20
CKPT_DIR = "out/ckpt/tipo-moe-1b"
CKPT_EVERY = 5000
SAMPLE_INTERVAL = 2000
SAMPLE_PROMPTS = ["target: <|long|>\ntags: 1girl, solo, outdoors, cherry blossoms\nlong: "]
SAMPLE_TOKENS = 128
