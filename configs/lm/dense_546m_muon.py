"""Dense ~546M with Muon on the hidden matrices (AdamW on embeddings, norms and the head), NCCL gradient sync."""

PRESET = "B200-dense-546M"
OPTIMIZER = "muon"
OPTIMIZER_KWARGS = {"muon_lr": 0.02}
BATCH_TOKENS = 16384
GRAD_ACCUM = 4
CTX_MAX = 4096
LEN_MIN, LEN_MAX = 64, 4096
LR = 3e-4
MAX_STEPS = 10000
WARMUP_STEPS = 500
