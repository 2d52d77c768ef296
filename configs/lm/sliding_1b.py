"""Gemma-shaped sliding-window ~1.1B: window 1024 on 3 of 4 layers, 4 sink logits per head, YaRN x4 from
4096, packs of 16384 tokens with log-uniform document lengths."""

PRESET = "B200-sliding-1B"
BATCH_TOKENS = 16384
GRAD_ACCUM = 1
CTX_MAX = 16384
LEN_MIN, LEN_MAX = 128, 16384
LR = 2e-4
