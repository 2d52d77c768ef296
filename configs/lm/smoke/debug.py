"""CPU smoke run: d256, 4 layers, 4 query / 2 KV heads, FFN 704, vocab 65536, z-loss 1e-4; packs of
2048 tokens with documents uniform in [16, 512]; AdamW 3e-4, betas (0.9, 0.95), wd 0.1; 50 steps, accum 2."""

PRESET = "B200-smoke"
ARCH_OVERRIDES = {}
DATA = "synthetic"
BATCH_TOKENS = 2048
GRAD_ACCUM = 2
LEN_MIN, LEN_MAX = 16, 512
LR = 3e-4
WEIGHT_DECAY = 0.1
BETAS = (0.9, 0.95)
MAX_STEPS = 50
WARMUP_STEPS = 5
LOG_INTERVAL = 10
DEVICE = "cpu"
