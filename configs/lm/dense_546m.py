"""Dense ~546M, MXFP8 linears, DDP with token-exact accumulation 4 x 4096-token packs per GPU."""

PRESET = "B200-dense-546M"
BATCH_TOKENS = 16384
GRAD_ACCUM = 4
CTX_MAX = 4096
LEN_MIN, LEN_MAX = 64, 4096
LR = 3e-4
MAX_STEPS = 10000
WARMUP_STEPS = 500
