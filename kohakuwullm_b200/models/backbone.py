"""``LMBackbone``: embedding -> decoder blocks -> final norm, a pure function of
``(tokens, seq_info)``; the loss lives in the separate :class:`LMHead` it owns.

The block loop carries the residual stream as ``(x, pending)`` so every residual add is fused into
the following RMSNorm kernel, builds the rotary tables and the attention work list ONCE per forward
and hands them to every layer. Reference: src/kohakuwullm/models/backbone.py:21-322.
"""

from __future__ import annotations

import math

import torch
from torch import nn
from torch.utils.checkpoint import checkpoint

from kohakuwullm_b200.models.block import DecoderBlock
from kohakuwullm_b200.models.head import LMHead
from kohakuwullm_b200.models.presets import LMArchConfig
from kohakuwullm_b200.models.seqinfo import SeqInfo
from kohakuwullm_b200.ops import attention as attn_ops
from kohakuwullm_b200.registry import NORM, POSENC, build

# imported for their registrations
from kohakuwullm_b200.models.components import attention as _a, mlp as _m, moe as _e, norm as _n, posenc as _p  # noqa: F401,E501
from kohakuwullm_b200.models.components import moe_variants as _v, ndrope as _r  # noqa: F401,E402  (registrations)


def build_block(config: LMArchConfig, layer: int) -> DecoderBlock:
    """The one block factory (also used by the pipeline cost autotuner)."""
    attn_kwargs = dict(heads=config.heads, kv_heads=config.kv_heads, head_dim=config.head_dim,
                       qk_norm=config.qk_norm, qk_norm_affine=config.qk_norm_affine, bias=config.attn_bias,
                       window=config.window_for(layer), sink=config.attn_sink,
                       num_sinks=config.attn_num_sinks, norm_eps=config.norm_eps)
    if config.moe_layers[layer]:
        mlp_spec = config.moe_mlp or "moe"
        mlp_kwargs = dict(num_experts=config.moe_num_experts, top_k=config.moe_top_k,
                          num_shared=config.moe_num_shared, hidden=config.moe_hidden, ratio=config.moe_ratio,
                          multiple_of=config.mlp_multiple_of, router=config.moe_router,
                          router_kwargs=dict(config.moe_router_kwargs), **config.moe_mlp_kwargs)
    else:
        mlp_spec = config.mlp
        mlp_kwargs = dict(hidden=config.mlp_hidden, ratio=config.mlp_ratio, multiple_of=config.mlp_multiple_of)
    return DecoderBlock(config.dim, config.norm, config.attn_for(layer), mlp_spec, norm_eps=config.norm_eps,
                        post_norm=config.post_norm, residual_scale=config.residual_scale,
                        attn_kwargs=attn_kwargs, mlp_kwargs=mlp_kwargs)


class LMBackbone(nn.Module):
    def __init__(self, config: LMArchConfig, head_kwargs: dict | None = None, init: bool = True):
        super().__init__()
        self.config = config
        self.embed = nn.Embedding(config.vocab_size, config.dim)
        self.embed_scale = math.sqrt(config.dim) if config.embedding_scale else 1.0
        self.pos_enc = build(config.posenc, POSENC, head_dim=config.head_dim, theta=config.rope_theta,
                             scaling=config.rope_scaling, factor=config.rope_factor,
                             max_position=config.max_position, partial=config.rope_partial)
        self.blocks = nn.ModuleList(build_block(config, i) for i in range(config.depth))
        self.final_norm = build(config.norm, NORM, dim=config.dim, eps=config.norm_eps)
        self.head = LMHead(config.dim, config.vocab_size,
                           tied_weight=self.embed.weight if config.tie_embeddings else None,
                           z_loss_weight=config.z_loss_weight, logit_soft_cap=config.logit_soft_cap,
                           **(head_kwargs or {}))
        self.grad_ckpt = config.grad_ckpt
        if init:
            self.initialize_weights()
        if config.mxfp8:
            self._swap_to_mxfp8()

    # ------------------------------------------------------------------ init
    @torch.no_grad()
    def initialize_weights(self) -> None:
        """normal(init_std); residual-output projections scaled by 1/sqrt(2*depth); optional muP
        width scaling ``sqrt(base/fan_in)`` on hidden matrices (never on the embedding)."""
        cfg = self.config
        out_scale = 1.0 / math.sqrt(2.0 * cfg.depth)
        for name, p in self.named_parameters():
            if p.dim() < 2:
                if name.endswith("bias"):
                    p.zero_()
                continue  # norm scales keep their constructor values
            if name.endswith("sink"):
                p.zero_()
                continue
            std = cfg.init_std
            if cfg.mup_base_dim and not name.startswith("embed"):
                std *= math.sqrt(cfg.mup_base_dim / p.shape[-1])
            if ".o_proj." in name or ".w_out." in name or name.endswith(".w_out") or ".fc2." in name:
                std *= out_scale
            p.normal_(0.0, std)

    def _swap_to_mxfp8(self) -> None:
        from kohakuwullm_b200.models.mxfp8_swap import swap_mxfp8

        report = swap_mxfp8(self)
        self.mxfp8_report = report    # census of per-token matmul work by bucket + unclaimed parameters
        if report.blocking:
            raise RuntimeError(f"MXFP8 conversion incomplete: {report.blocking}")
        if report.unaccounted:
            import warnings

            warnings.warn(f"MXFP8 conversion: matmul-shaped parameters that no rule claimed stay 16-bit: "
                          f"{report.unaccounted}")
        from kohakuwullm_b200.models.mxfp8_swap import wire_fused_quantisation

        wire_fused_quantisation(self)

    def refresh_mxfp8(self) -> int:
        from kohakuwullm_b200.models.mxfp8_swap import refresh_mxfp8_weights

        return refresh_mxfp8_weights(self)

    # ------------------------------------------------------------------ forward
    def embed_tokens(self, tokens: torch.Tensor) -> torch.Tensor:
        from kohakuwullm_b200.ops.elementwise import embedding

        return embedding(tokens, self.embed.weight, self.embed_scale)

    def prepare(self, seq_info: SeqInfo, device, dtype):
        """Per-forward constants shared by every layer: rotary tables and the attention work list."""
        rope = self.pos_enc.prepare(seq_info.position_ids)
        plan = None
        if seq_info.packed and device.type == "cuda" and dtype == torch.bfloat16 and self.config.head_dim == 64 \
                and attn_ops.native.available():
            plan = attn_ops.attention_plan(seq_info.cu_seqlens, seq_info.total_tokens)
        return rope, plan

    def run_blocks(self, x, seq_info, rope, plan, cache=None, start: int = 0, end: int | None = None,
                   taps: list | None = None):
        pending = None
        end = len(self.blocks) if end is None else end
        for i in range(start, end):
            blk = self.blocks[i]
            if self.grad_ckpt and self.training and cache is None:
                x, pending = checkpoint(blk.forward_deferred, x, pending, seq_info, rope, None, i, plan,
                                        use_reentrant=False)
            else:
                x, pending = blk.forward_deferred(x, pending, seq_info, rope, cache, i, plan)
            if taps is not None:
                taps.append(DecoderBlock.merge(x, pending))
        return x, pending

    def forward(self, tokens: torch.Tensor, seq_info: SeqInfo, cache=None, taps: list | None = None):
        """tokens (T,) packed or (B,S) padded -> final-normed hidden states of the same leading shape."""
        if self.config.mxfp8:
            from kohakuwullm_b200.ops.mxfp8 import clear_prequantized

            clear_prequantized()
        x = self.embed_tokens(tokens)
        rope, plan = self.prepare(seq_info, x.device, x.dtype)
        x, pending = self.run_blocks(x, seq_info, rope, plan, cache=cache, taps=taps)
        if cache is not None:
            cache.advance()
        if pending is None:
            return self.final_norm(x)
        hidden, _ = self.final_norm(pending, residual=x)
        return hidden

    # ------------------------------------------------------------------ loss
    def router_losses(self) -> torch.Tensor | None:
        total = None
        for blk in self.blocks:
            router = getattr(blk.mlp, "router", None)
            aux = getattr(router, "aux_loss", None) if router is not None else None
            if aux is not None:
                total = aux if total is None else total + aux
        return total

    def loss(self, tokens, labels, seq_info, reduction: str = "mean", router_scale: float | torch.Tensor = 1.0):
        hidden = self.forward(tokens, seq_info)
        loss, logs = self.head.loss(hidden, labels, reduction)
        aux = self.router_losses()
        if aux is not None:
            loss = loss + aux * router_scale
            logs["router_loss"] = aux.detach()
        return loss, logs

    @torch.no_grad()
    def update_router_bias(self, rate_scale: float = 1.0) -> dict[str, torch.Tensor]:
        """One balancing step on every router; returns stacked device stats (read them on an interval)."""
        stats: list[dict[str, torch.Tensor]] = []
        routers = [r for r in (getattr(blk.mlp, "router", None) for blk in self.blocks)
                   if r is not None and hasattr(r, "update_bias")]
        # one collective for the whole model: routers that share (expert count, group) have their per-layer
        # loads stacked into one (layers, experts) tensor and reduced together, instead of one all-reduce each
        reduced: dict[int, torch.Tensor] = {}
        pools: dict[tuple, list] = {}
        for r in routers:
            if hasattr(r, "wants_load_reduce") and r.wants_load_reduce():
                pools.setdefault((r.load_accum.numel(), id(r.load_group)), []).append(r)
        for members in pools.values():
            stacked = torch.stack([r.load_accum for r in members])
            torch.distributed.all_reduce(stacked, group=members[0].load_group)
            for r, row in zip(members, stacked):
                reduced[id(r)] = row
        for r in routers:
            stats.append(r.update_bias(rate_scale, reduced.get(id(r))) if id(r) in reduced else r.update_bias(rate_scale))
        if not stats:
            return {}
        return {
            "moe/load_imbalance_max": torch.stack([s["max_over_mean"] for s in stats]).max(),
            "moe/load_imbalance_mean": torch.stack([s["max_over_mean"] for s in stats]).mean(),
            "moe/load_min_over_mean": torch.stack([s["min_over_mean"] for s in stats]).min(),
            "moe/dead_experts": torch.stack([s["dead"] for s in stats]).sum(),
        }

    def param_summary(self) -> dict[str, int]:
        from kohakuwullm_b200.utils.misc import count_active_parameters, count_parameters

        total = count_parameters(self)
        emb = self.embed.weight.numel()
        return {"total": total, "active": count_active_parameters(self), "embedding": emb,
                "head": 0 if self.head.tied else self.head.weight.numel()}
