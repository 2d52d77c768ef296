"""Ten pipeline steps of Kohaku-MoE-1B on synthetic packs with a collective preview in the middle and at the end:
training throughput and the generation path through the stages, measured in one short run.

    torchrun --nproc-per-node 4 -m kohakuwullm_b200.cli.train_lm_pipe --config configs/lm/smoke/pipegen_bench.py
    python -m kohakuwullm_b200.cli.train_lm_pipe --config configs/lm/smoke/pipegen_bench.py --set GPUS=4

The byte tokenizer (vocabulary 258) keeps the run free of tokenizer files; `SAMPLE_LOCAL = False` would decode
through the pipeline instead of gathering the weights on rank 0.
"""

# what is trained
PRESET = "Kohaku-MoE-1B"
ARCH_OVERRIDES = {"vocab_size": 258, "max_position": 4096, "rope_theta": 100000.0, "tie_embeddings": False, "mxfp8": True}
AUX_LOSS_WEIGHT = ROUTER_Z_LOSS_WEIGHT = 0.0

# on what: random documents of 50 to 600 tokens, 8 micro-batches of 16384 tokens per step
DATA, TOKENIZER = "synthetic", "byte"
LEN_MIN, LEN_MAX = 50, 600
MICRO_TOKENS, NUM_MICROBATCHES = 16384, 8

# how
SCHEDULE, AUTOTUNE = "1f1b", False
OPTIMIZER, OPTIMIZER_KWARGS = "muon", {"muon_lr": 2e-3, "embed_lr": 2e-3}
LR, WARMUP_STEPS, MAX_STEPS = 5e-4, 2, 10
LOG_INTERVAL = 1

# the preview
SAMPLE_INTERVAL, SAMPLE_TOKENS, SAMPLE_COUNT = 5, 32, 2
SAMPLE_PROMPTS = [("bytes", "Once upon a time")]
