"""``gpu_smoke.py`` with every eligible linear in MXFP8 (block-scaled e4m3 operands, fp32 accumulation).

    python -m kohakuwullm_b200.cli.train_lm --config configs/lm/smoke/gpu_smoke.py --config configs/lm/smoke/smoke_mxfp8.py

The conversion report printed at start-up lists what was converted and the share of per-token matmul work per bucket;
the loss of the first twenty steps should track the bf16 run to the second decimal.
"""

ARCH_OVERRIDES = {"mxfp8": True}
