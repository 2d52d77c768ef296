"""Kohaku-MoE-1B for ten pipeline steps with a collective preview: training throughput and the pipelined generation
path in one short run on synthetic packs.

    torchrun --nproc-per-node 4 -m kohakuwullm_b200.cli.train_lm_pipe --config configs/lm/smoke/pipegen_bench.py
"""

PRESET = "Kohaku-MoE-1B"
ARCH_OVERRIDES = {"max_position": 4096, "rope_theta": 100000.0, "qk_norm": True, "tie_embeddings": False, "mxfp8": True,
                  "vocab_size": 258}        # the byte tokenizer, so that the preview needs no tokenizer files
AUX_LOSS_WEIGHT = 0.0
ROUTER_Z_LOSS_WEIGHT = 0.0
DATA = "synthetic"
TOKENIZER = "byte"
LEN_MIN, LEN_MAX = 50, 600
MICRO_TOKENS = 16384
NUM_MICROBATCHES = 8
SCHEDULE = "1f1b"
AUTOTUNE = False
OPTIMIZER = "muon"
OPTIMIZER_KWARGS = {"muon_lr": 2e-3, "embed_lr": 2e-3}
LR = 5e-4
MAX_STEPS = 10
WARMUP_STEPS = 2
LOG_INTERVAL = 1
SAMPLE_INTERVAL = 5
SAMPLE_PROMPTS = [("bytes", "Once upon a time")]
SAMPLE_TOKENS = 32
