"""DeepSeekMoE ~991M under pipeline parallelism: measured split, 1F1B, 16 micro-batches of 4096 tokens.

    torchrun --nproc-per-node 4 -m kohakuwullm_b200.cli.train_lm_pipe --config configs/lm/moe_991m_pipe.py
"""

PRESET = "B200-moe-991M"
MICRO_TOKENS = 4096
NUM_MICROBATCHES = 16
SCHEDULE = "1f1b"
AUTOTUNE = True
LR = 3e-4
