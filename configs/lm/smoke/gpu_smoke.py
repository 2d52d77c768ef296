"""Twenty steps of a small dense model on one GPU with synthetic packs: does the whole native path run?

    python -m kohakuwullm_b200.cli.train_lm --config configs/lm/smoke/gpu_smoke.py

bf16 parameters, tcgen05 GEMMs and attention, flat fused AdamW, CUDA-graph replay of the micro-batches.
"""

PRESET = "Nano-100M"
ARCH_OVERRIDES = {"max_position": 2048}
DATA = "synthetic"
BATCH_TOKENS = 8192
GRAD_ACCUM = 2
CTX_MAX = 2048
LEN_MIN, LEN_MAX = 64, 2048
LR = 6e-4
MAX_STEPS = 20
WARMUP_STEPS = 5
LOG_INTERVAL = 5
