"""DeepSeekMoE ~991M with the experts of every layer split over the ranks (expert parallel), everything else data
parallel. The receive buffers hold ``EP_CAPACITY`` times the mean rows per rank; with ``EP_ON_OVERFLOW = "count"`` a
layer whose router overloads one rank drops the excess pairs and reports ``ep_dropped_pairs`` instead of ending the run."""

PRESET = "B200-moe-991M"
EXPERT_PARALLEL = True
EP_CAPACITY = 3.0
EP_ON_OVERFLOW = "count"
BATCH_TOKENS = 32768
GRAD_ACCUM = 4
CTX_MAX = 4096
LEN_MIN, LEN_MAX = 64, 4096
LR = 3e-4
MAX_STEPS = 10000
WARMUP_STEPS = 500
