"""Prompt-optimisation model on Kohaku-MoE-1B over 4 pipeline stages: MXFP8 experts, bias-balanced routers, Muon,
packed documents and collective previews at once (the validation recipe of the pipeline path).

    torchrun --nproc-per-node 4 -m kohakuwullm_b200.cli.train_lm_pipe --config configs/lm/tipo/tipo_moe_1b_pp4.py

32 micro-batches of 8192 tokens per optimizer step (262144 tokens); the stage split is measured at start-up.
"""

import os
import runpy

_src = runpy.run_path(os.path.join(os.path.dirname(os.path.abspath(__file__)), "_sources.py"))

PRESET = "Kohaku-MoE-1B"
ARCH_OVERRIDES = {"max_position": 4096, "rope_theta": 100000.0, "qk_norm": True, "tie_embeddings": False, "mxfp8": True}
AUX_LOSS_WEIGHT = 0.0
ROUTER_Z_LOSS_WEIGHT = 0.0
BIAS_SCHEDULE = {"mode": "cosine", "end": 100_000, "min_value": 0.1}      # the bias update rate decays with the run

SOURCES = _src["caption_sources"]()
RENDERER = "tipo"
TOKENIZER = "models/tokenizer"
CTX_MAX = 2048

GPUS = 4
MICRO_TOKENS = 8192
NUM_MICROBATCHES = 32
SCHEDULE = "1f1b"
AUTOTUNE = True

OPTIMIZER = "muon"
OPTIMIZER_KWARGS = {"muon_lr": 2e-3, "embed_lr": 2e-3}
LR = 5e-4
WEIGHT_DECAY = 0.1
MAX_GRAD_NORM = 1.0
MAX_STEPS = 100_000
WARMUP_STEPS = 2000
LR_SCHEDULE = {"phases": [{"mode": "power", "end": 0.9, "s0": 2500, "b": -0.5, "warmup": None},
                          {"mode": "cosine", "end": 1.0, "min_value": 0.01}], "end": None}

RUN_NAME = "tipo-moe-1b-pp4"
WANDB_PROJECT = "kohakuwullm-b200"
LOG_INTERVAL = 20
CKPT_DIR = "out/ckpt/tipo-moe-1b-pp4"
CKPT_EVERY = 2000
SAMPLE_INTERVAL = 2000
SAMPLE_PROMPTS = [("caption", "target: <|long|>\ntags: 1girl, solo, outdoors, cherry blossoms\nlong: ")]
SAMPLE_TOKENS = 128
SAMPLE_TEMPERATURE = 1.0
