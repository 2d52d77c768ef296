"""``tipo_moe_1b.py`` with the experts of every MoE layer sharded over the 8 ranks (expert parallel + data parallel).

    torchrun --nproc-per-node 8 -m kohakuwullm_b200.cli.train_lm --config configs/lm/tipo/tipo_moe_1b.py \
        --config configs/lm/tipo/tipo_moe_1b_ep.py

Token rows travel to the owning rank's receive buffer over NVLink and come back weighted; expert gradients need no
all-reduce. Capacity 2.0 leaves room for twice the uniform share per rank; pairs beyond it are dropped and counted.
"""

EXPERT_PARALLEL = True
EP_CAPACITY = 2.0
EP_ON_OVERFLOW = "count"
RUN_NAME = "tipo-moe-1b-ep8"
CKPT_DIR = "out/ckpt/tipo-moe-1b-ep8"
