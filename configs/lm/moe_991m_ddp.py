"""DeepSeekMoE ~991M, data parallel: 8192-token packs x 4 accumulation per GPU, experts in MXFP8 grouped GEMMs."""

PRESET = "B200-moe-991M"
BATCH_TOKENS = 32768
GRAD_ACCUM = 4
CTX_MAX = 4096
LEN_MIN, LEN_MAX = 64, 4096
LR = 3e-4
MAX_STEPS = 10000
WARMUP_STEPS = 500
