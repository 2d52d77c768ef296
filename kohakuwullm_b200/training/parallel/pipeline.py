"""LM-aware pipeline pieces: the stage module, the analytic cost model and ``plan_for``.

``LMStage`` is a contiguous slice of a built :class:`LMBackbone` that SHARES the backbone's Parameter
objects: stage 0 owns the embedding, the last stage the final norm and the head. The per-micro-batch
``SeqInfo`` objects are registered with ``set_seq_info`` and never sent between ranks. When any layer
of the WHOLE model produces a router auxiliary loss, every boundary also carries the ``(1,)`` fp32
accumulator stream, so all ranks agree on the boundary signature. Parameter names map to whole-model
names through ``global_names`` (block ``i`` of a stage is block ``i + start_layer`` of the model), which
is what makes checkpoints portable across splits. Reference:
src/kohakuwullm/training/parallel/pipeline.py:40-508.
"""

from __future__ import annotations

import warnings
from typing import Sequence

import torch
from torch import nn

from kohakuwullm_b200.models.backbone import LMBackbone
from kohakuwullm_b200.models.block import DecoderBlock
from kohakuwullm_b200.models.presets import LMArchConfig
from kohakuwullm_b200.models.seqinfo import SeqInfo
from kohakuwullm_b200.pipe import streams
from kohakuwullm_b200.pipe.plan import StagePlan, plan_from_layers, plan_stages

HEAD_INEFFICIENCY = 1.55  # the head's GEMMs run below block-GEMM efficiency; measured scale overrides it


# ------------------------------------------------------------------ analytic costs
def block_cost(config: LMArchConfig, layer: int, seq_len: int) -> float:
    """Relative per-token cost of one block (multiply-accumulates)."""
    q_dim = config.heads * config.head_dim
    kv_dim = config.kv_heads * config.head_dim
    attn_proj = config.dim * (q_dim + 2 * kv_dim) + q_dim * config.dim
    window = config.window_for(layer)
    span = min(seq_len, window) if window else seq_len
    attn = 2 * q_dim * span / (1 if window else 2)
    if config.moe_layers[layer]:
        hidden = config.moe_hidden or int(config.dim * config.moe_ratio * 2 / 3)
        mlp = 3 * config.dim * hidden * (config.moe_top_k + config.moe_num_shared)
    else:
        hidden = config.mlp_hidden or int(config.dim * config.mlp_ratio * 2 / 3)
        mlp = 3 * config.dim * hidden
    return float(attn_proj + attn + mlp)


def block_params(config: LMArchConfig, layer: int) -> float:
    q_dim = config.heads * config.head_dim
    kv_dim = config.kv_heads * config.head_dim
    n = config.dim * (q_dim + 2 * kv_dim) + q_dim * config.dim
    if config.moe_layers[layer]:
        hidden = config.moe_hidden or int(config.dim * config.moe_ratio * 2 / 3)
        n += 3 * config.dim * hidden * (config.moe_num_experts + config.moe_num_shared)
    else:
        hidden = config.mlp_hidden or int(config.dim * config.mlp_ratio * 2 / 3)
        n += 3 * config.dim * hidden
    return float(n)


def head_cost(config: LMArchConfig, head_scale: float | None = None) -> float:
    return float(config.dim * config.vocab_size * (head_scale if head_scale is not None else HEAD_INEFFICIENCY))


def plan_for(config: LMArchConfig, num_stages: int, seq_len: int = 4096, *, layers: Sequence[int] | None = None,
             style: str = "loop", costs=None, head_scale: float | None = None,
             allow_empty_last: bool = False) -> list[StagePlan]:
    """Stage plan for ``config``: explicit ``layers`` pin, measured ``costs`` (``LayerCosts``) or the
    analytic model."""
    if layers is not None:
        if sum(layers) != config.depth:
            raise ValueError(f"layers {list(layers)} do not add up to depth {config.depth}")
        return plan_from_layers(layers)
    if costs is not None:
        layer_costs, embed, head = list(costs.layers), costs.embed, costs.head
    else:
        layer_costs = [block_cost(config, i, seq_len) for i in range(config.depth)]
        embed, head = 0.0, head_cost(config, head_scale)
    params = [block_params(config, i) for i in range(config.depth)]
    emb_params = float(config.vocab_size * config.dim)
    if style == "v":
        return plan_stages(layer_costs, num_stages, style="v", embed_cost=embed, head_cost=head)
    return plan_stages(layer_costs, num_stages, embed_cost=embed, head_cost=head, layer_params=params,
                       embed_params=emb_params, head_params=0.0 if config.tie_embeddings else emb_params,
                       allow_empty_last=allow_empty_last)


def model_has_router_loss(config: LMArchConfig) -> bool:
    """Decided from the WHOLE model so that every rank builds the same boundary signature."""
    if not any(config.moe_layers):
        return False
    kw = config.moe_router_kwargs or {}
    return bool(kw.get("aux_loss_weight") or kw.get("z_loss_weight"))


# ------------------------------------------------------------------ the stage module
class LMStage(nn.Module):
    def __init__(self, backbone: LMBackbone, plan: StagePlan, boundary_dtype: torch.dtype | None = None):
        super().__init__()
        cfg = backbone.config
        self.config, self.plan = cfg, plan
        self.is_first, self.is_last = plan.is_first, plan.is_last
        self.boundary_dtype = boundary_dtype
        self.has_aux = model_has_router_loss(cfg)
        self.pos_enc = backbone.pos_enc
        self.embed_scale = backbone.embed_scale
        self.grad_ckpt = backbone.grad_ckpt
        if self.is_first:
            self.embed = backbone.embed
        self.blocks = nn.ModuleList(backbone.blocks[i] for i in range(plan.start_layer, plan.end_layer))
        if self.is_last:
            self.final_norm = backbone.final_norm
            if backbone.head.tied and not self.is_first:
                warnings.warn("tied embeddings are untied: embedding and head live on different stages")
                backbone.head.untie()
            self.head = backbone.head
        if plan.num_stages > 1:
            for blk in self.blocks:  # a split model never reduces router load across pipeline ranks
                router = getattr(blk.mlp, "router", None)
                if router is not None:
                    router.reduce_load = False
        self._seq_infos: list[SeqInfo] = []
        self._fwd_counter = 0

    # ------------------------------------------------------------------ names
    def global_names(self) -> dict[str, str]:
        """stage-local parameter/buffer name -> whole-model name."""
        out = {}
        for name, _ in list(self.named_parameters()) + list(self.named_buffers()):
            parts = name.split(".")
            if parts[0] == "blocks":
                parts[1] = str(int(parts[1]) + self.plan.start_layer)
            out[name] = ".".join(parts)
        return out

    # ------------------------------------------------------------------ layout
    def set_seq_info(self, infos: Sequence[SeqInfo]) -> None:
        self._seq_infos = list(infos)
        self._fwd_counter = 0

    def forward_micro(self, mb: int, *inputs):
        info = self._seq_infos[mb]
        if self.is_first:
            tokens = inputs[0] if inputs else self._tokens[mb]
            x = self.embed(tokens)
            if self.embed_scale != 1.0:
                x = x * self.embed_scale
            aux = streams.accumulator(x.device) if self.has_aux else None
        else:
            carrier = streams.split_streams(inputs)
            x, aux = carrier.hidden, carrier.aux
        rope = self.pos_enc.prepare(info.position_ids)
        plan = None
        if info.packed and x.is_cuda and x.dtype == torch.bfloat16 and self.config.head_dim == 64:
            from kohakuwullm_b200.ops import attention as attn_ops

            if attn_ops.native.available():
                plan = attn_ops.attention_plan(info.cu_seqlens, info.total_tokens)
        pending = None
        for i, blk in enumerate(self.blocks):
            x, pending = blk.forward_deferred(x, pending, info, rope, None, self.plan.start_layer + i, plan)
            if aux is not None:
                router = getattr(blk.mlp, "router", None)
                aux = streams.accumulate(aux, getattr(router, "aux_loss", None) if router is not None else None)
        if self.is_last:
            if pending is None:
                hidden = self.final_norm(x)
            else:
                hidden, _ = self.final_norm(pending, residual=x)
            return (hidden, aux) if aux is not None else hidden
        x = DecoderBlock.merge(x, pending)
        if self.boundary_dtype is not None:
            x = x.to(self.boundary_dtype)
        return (x, aux) if aux is not None else x

    def forward(self, *inputs):
        """Schedule-driven entry point: the micro-batch index is the running forward counter."""
        mb = self._fwd_counter % max(len(self._seq_infos), 1)
        self._fwd_counter += 1
        return self.forward_micro(mb, *inputs)

    def set_tokens(self, tokens: Sequence[torch.Tensor]) -> None:
        self._tokens = list(tokens)

    # ------------------------------------------------------------------ router maintenance
    @torch.no_grad()
    def update_router_bias(self, rate_scale: float = 1.0):
        stats = []
        for blk in self.blocks:
            router = getattr(blk.mlp, "router", None)
            if router is not None and hasattr(router, "update_bias"):
                stats.append(router.update_bias(rate_scale))
        return stats


class AutocastStage(nn.Module):
    """Runs a stage (and the loss) under autocast."""

    def __init__(self, stage: LMStage, dtype: torch.dtype | None):
        super().__init__()
        self.stage, self.dtype = stage, dtype

    def forward(self, *inputs):
        if self.dtype is None or not inputs or not inputs[0].is_cuda:
            return self.stage(*inputs)
        with torch.autocast("cuda", dtype=self.dtype):
            return self.stage(*inputs)
