"""Closed-form FLOPs per token of a preset, split into tensor-core work (weight GEMMs, attention products) and
vector work (norms, activations, softmax, rotary), without building the model.

Conventions: one multiply-accumulate is 2 FLOPs; backward costs twice the forward; activation checkpointing
charges the block forward once more. Attention is counted from the attended (query, key) pairs per token of
documents uniform on ``[len_min, len_max]`` (token-weighted, summed exactly), with the per-layer window of the
preset. The vector terms are small integers per element, meant for the matrix/vector split, not for rooflines.
Reference: src/kohakuwullm/bench/model/flops_analytic.py:1-164.
"""

from __future__ import annotations

from dataclasses import dataclass

from kohakuwullm_b200.models.components.mlp import resolve_hidden
from kohakuwullm_b200.models.flops import attention_pairs
from kohakuwullm_b200.models.presets import LMArchConfig, get_preset

MAC = 2.0


@dataclass(frozen=True)
class FlopBudget:
    name: str
    gemm_fwd: float
    gemm_bwd: float
    attn_fwd: float
    attn_bwd: float
    vector_fwd: float
    vector_bwd: float
    pairs_per_token: float

    @property
    def matrix(self) -> float:
        return self.gemm_fwd + self.gemm_bwd + self.attn_fwd + self.attn_bwd

    @property
    def vector(self) -> float:
        return self.vector_fwd + self.vector_bwd

    @property
    def total(self) -> float:
        return self.matrix + self.vector

    @property
    def matrix_share(self) -> float:
        return self.matrix / self.total

    @property
    def gemm_only(self) -> float:
        return self.gemm_fwd + self.gemm_bwd


def causal_pairs_per_token(len_min: int, len_max: int, window: int | None) -> float:
    pairs = tokens = 0.0
    for n in range(len_min, len_max + 1):
        pairs += attention_pairs(n, window)
        tokens += n
    return pairs / tokens


def block_macs(cfg: LMArchConfig, layer: int) -> float:
    """Weight multiply-accumulates per token of one block (MoE layers at their active experts)."""
    q_dim, kv_dim = cfg.heads * cfg.head_dim, cfg.kv_heads * cfg.head_dim
    macs = cfg.dim * (q_dim + 2 * kv_dim) + q_dim * cfg.dim
    if cfg.moe_layers[layer]:
        h = cfg.moe_hidden or resolve_hidden(cfg.dim, cfg.mlp_ratio, None, 128, glu=True)
        macs += (cfg.moe_top_k + cfg.moe_num_shared) * 3 * cfg.dim * h + cfg.dim * cfg.moe_num_experts
    else:
        h = resolve_hidden(cfg.dim, cfg.mlp_ratio, cfg.mlp_hidden, 128, glu=True)
        macs += 3 * cfg.dim * h
    return float(macs)


def flop_budget(preset: str | LMArchConfig, len_min: int = 64, len_max: int = 4096, **overrides) -> FlopBudget:
    cfg = get_preset(preset, **overrides) if isinstance(preset, str) else preset
    gemm = sum(block_macs(cfg, i) for i in range(cfg.depth)) + cfg.dim * cfg.vocab_size
    q_dim = cfg.heads * cfg.head_dim
    pairs = sum(causal_pairs_per_token(len_min, len_max, w) for w in cfg.windows)   # summed over layers
    attn = 2.0 * q_dim * pairs          # QK^T and PV: two products of q_dim MACs per pair
    # vector work per token: two norms (~8 ops/element), rotary (6 per q/k element), SwiGLU (~10 per hidden
    # element), softmax (~6 per pair per head)
    width = sum((cfg.moe_hidden or 0) * (cfg.moe_top_k + cfg.moe_num_shared) if cfg.moe_layers[i]
                else resolve_hidden(cfg.dim, cfg.mlp_ratio, cfg.mlp_hidden, 128, glu=True) for i in range(cfg.depth))
    vector = cfg.depth * (16.0 * cfg.dim + 6.0 * (q_dim + cfg.kv_heads * cfg.head_dim)) + 10.0 * width \
        + 6.0 * cfg.heads * pairs
    ckpt = 1.0 if cfg.grad_ckpt else 0.0
    name = preset if isinstance(preset, str) else "config"
    return FlopBudget(name, MAC * gemm, (2.0 + ckpt) * MAC * gemm, MAC * attn, (2.5 + ckpt) * MAC * attn,
                      vector, (2.0 + ckpt) * vector, pairs / max(cfg.depth, 1))
