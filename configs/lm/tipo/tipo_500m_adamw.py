"""The dense prompt-optimisation recipe with the flat fused AdamW instead of Muon: the gradient reduce-scatter, the
update of each rank's shard and the all-gather of the bf16 weights run as one kernel over NVLink peer memory.

    torchrun --nproc-per-node 8 -m kohakuwullm_b200.cli.train_lm --config configs/lm/tipo/tipo_500m.py \
        --config configs/lm/tipo/tipo_500m_adamw.py

Given AFTER ``tipo_500m.py`` it overrides only the optimizer section.
"""

OPTIMIZER = "fused_adamw"
OPTIMIZER_KWARGS = {}
GRAD_SYNC = "auto"
GRAD_COMPRESS = ""
LR = 6e-4
RUN_NAME = "tipo-500m-adamw"
CKPT_DIR = "out/ckpt/tipo-500m-adamw"
