"""DeepSeekMoE-style routed feed-forward: top-k router with aux-loss-free bias balancing, stacked
expert weights, shared experts.

Routing contract (reference: src/kohakuwullm/models/components/moe.py:49-249):
  * score = sigmoid | softmax | sqrtsoftplus of the fp32 gate logits;
  * the per-expert ``expert_bias`` buffer steers SELECTION only: top-k is taken over ``score + bias``
    but the gate weight is the unbiased score (optionally normalised over the k picks and scaled);
  * ``load_accum`` counts routed tokens per expert; once per optimizer step ``update_bias`` moves the
    bias by ``rate * sign(mean_load - load)`` and clears the counter;
  * optional Switch-style auxiliary loss ``w * E * sum_e f_e P_e`` and router z-loss.

Expert evaluation (``MoEMLP``): tokens are counting-sorted by expert, each expert's rows run through
``w_in[e]`` -> SwiGLU -> ``w_out[e]`` and are combined with the gate weights in a deterministic
segment sum (no atomics). ``expert_path``:
  ``"grouped"``  native grouped tcgen05 GEMMs over the expert-sorted rows (GPU, bf16)
  ``"eager"``    per-expert loop in PyTorch (CPU, tests; the reference calls it ``dense_fallback``)
After ``parallel.ep.shard_experts`` the layer holds only its rank's experts and tokens travel to the
owning rank and back over peer memory (or, on CPU, through the collective-based oracle).
"""

from __future__ import annotations

import torch
import torch.distributed as dist
from torch import nn

from kohakuwullm_b200.models.components.mlp import GLUMLP, resolve_hidden
from kohakuwullm_b200.ops import moe as moe_ops
from kohakuwullm_b200.registry import MLP, ROUTER


class TopKRouter(nn.Module):
    def __init__(self, dim: int, num_experts: int, top_k: int, score: str = "sigmoid",
                 norm_topk_prob: bool = True, routed_scaling_factor: float = 1.0,
                 bias_update_rate: float = 1e-3, aux_loss_weight: float = 0.0,
                 z_loss_weight: float = 0.0, num_groups: int = 1, topk_groups: int = 1,
                 reduce_load: bool = True, **_unused):
        super().__init__()
        if score not in ("sigmoid", "softmax", "sqrtsoftplus"):
            raise ValueError(f"unknown router score {score!r}")
        self.dim, self.num_experts, self.top_k = dim, num_experts, top_k
        self.score = score
        self.norm_topk_prob = norm_topk_prob
        self.routed_scaling_factor = routed_scaling_factor
        self.bias_update_rate = bias_update_rate
        self.aux_loss_weight, self.z_loss_weight = aux_loss_weight, z_loss_weight
        self.num_groups, self.topk_groups = num_groups, topk_groups
        self.reduce_load = reduce_load
        self.load_group = None
        self.weight = nn.Parameter(torch.empty(num_experts, dim))
        self.register_buffer("expert_bias", torch.zeros(num_experts))
        self.register_buffer("load_accum", torch.zeros(num_experts))
        self.aux_loss: torch.Tensor | None = None
        self.last_stats: dict[str, float] = {}

    # ------------------------------------------------------------------
    def scores(self, logits: torch.Tensor) -> torch.Tensor:
        if self.score == "sigmoid":
            return torch.sigmoid(logits)
        if self.score == "softmax":
            return torch.softmax(logits, dim=-1)
        return torch.sqrt(torch.nn.functional.softplus(logits))

    def route(self, x: torch.Tensor):
        """x (T, dim) -> idx (T,k), weight (T,k) fp32, counts (E,) int32."""
        if moe_ops.router_supported(x, self.weight, self.num_groups):
            idx, w, counts, logits = moe_ops.router_topk(
                x, self.weight, self.expert_bias, self.load_accum if self.training else None, self.top_k,
                self.score, self.norm_topk_prob, self.routed_scaling_factor)
            self.aux_loss = self._aux(logits, self.scores(logits), counts) \
                if (self.training and (self.aux_loss_weight or self.z_loss_weight)) else None
            return idx, w, counts
        logits = torch.nn.functional.linear(x.float(), self.weight.float())
        s = self.scores(logits)
        biased = s + self.expert_bias.to(s.dtype)
        if self.num_groups > 1:
            T = s.shape[0]
            g = biased.view(T, self.num_groups, -1)
            strength = g.topk(2, dim=-1).values.sum(-1)                      # top-2 sum per group
            keep = torch.zeros_like(strength, dtype=torch.bool)
            keep.scatter_(1, strength.topk(self.topk_groups, dim=-1).indices, True)
            biased = g.masked_fill(~keep[..., None], float("-inf")).view(T, -1)
        idx = biased.topk(self.top_k, dim=-1).indices
        w = s.gather(1, idx)
        if self.norm_topk_prob:
            w = w / (w.sum(-1, keepdim=True) + 1e-20)
        w = w * self.routed_scaling_factor
        counts = torch.bincount(idx.reshape(-1), minlength=self.num_experts).to(torch.int32)
        if self.training:
            with torch.no_grad():
                self.load_accum += counts.to(self.load_accum.dtype)
        self.aux_loss = self._aux(logits, s, counts) if self.training else None
        return idx, w, counts

    def _aux(self, logits, s, counts):
        loss = None
        if self.aux_loss_weight:
            T = s.shape[0]
            f = counts.float() / max(T * self.top_k, 1)
            p = (s / (s.sum(-1, keepdim=True) + 1e-20)).mean(0)
            loss = self.aux_loss_weight * self.num_experts * (f * p).sum()
        if self.z_loss_weight:
            z = self.z_loss_weight * torch.logsumexp(logits, -1).pow(2).mean()
            loss = z if loss is None else loss + z
        return loss

    def wants_load_reduce(self) -> bool:
        return bool(self.reduce_load and dist.is_available() and dist.is_initialized()
                    and dist.get_world_size(self.load_group) > 1)

    @torch.no_grad()
    def update_bias(self, rate_scale: float = 1.0, reduced_load: torch.Tensor | None = None) -> dict[str, torch.Tensor]:
        """Aux-loss-free balancing step; returns device-side stats (no host sync here). ``reduced_load``: this
        router's load already summed over the data-parallel group (the backbone reduces all routers' loads in
        ONE collective per step and hands each its row); without it the router reduces its own."""
        if reduced_load is not None:
            load = reduced_load
        else:
            load = self.load_accum.clone()
            if self.wants_load_reduce():
                dist.all_reduce(load, group=self.load_group)
        mean = load.mean()
        self.expert_bias += (self.bias_update_rate * rate_scale) * torch.sign(mean - load)
        denom = mean.clamp(min=1e-9)
        stats = {"max_over_mean": load.max() / denom, "min_over_mean": load.min() / denom,
                 "dead": (load == 0).sum().float()}
        self.load_accum.zero_()
        return stats


ROUTER.register("topk", TopKRouter)


class MoEMLP(nn.Module):
    def __init__(self, dim: int, num_experts: int = 64, top_k: int = 8, num_shared: int = 1,
                 hidden: int | None = None, ratio: float = 4.0, multiple_of: int = 128,
                 router="topk", router_kwargs: dict | None = None, expert_path: str | None = None,
                 router_dim: int | None = None, **_unused):
        super().__init__()
        from kohakuwullm_b200.registry import build

        self.dim, self.num_experts, self.top_k = dim, num_experts, top_k
        self.hidden = resolve_hidden(dim, ratio, hidden, multiple_of, glu=True)
        self.router = build(router, ROUTER, dim=router_dim or dim, num_experts=num_experts, top_k=top_k,
                            **(router_kwargs or {}))
        self.w_in = nn.Parameter(torch.empty(num_experts, 2 * self.hidden, dim))
        self.w_out = nn.Parameter(torch.empty(num_experts, dim, self.hidden))
        self.shared = GLUMLP(dim, hidden=self.hidden * num_shared) if num_shared > 0 else None
        self.expert_path = expert_path  # None: chosen from the input device at call time
        # expert parallelism (kohakuwullm_b200.parallel.ep.shard_experts fills these in)
        self.ep, self.ep_group, self.ep_world, self.ep_rank = None, None, 1, 0
        self.mxfp8_experts = False
        self._q_in = self._q_out = None

    def active_parameters(self) -> int:
        per_expert = self.w_in[0].numel() + self.w_out[0].numel()
        n = self.top_k * per_expert + self.router.weight.numel()
        if self.shared is not None:
            n += sum(p.numel() for p in self.shared.parameters())
        return n

    # ------------------------------------------------------------------ MXFP8 protocol
    def mxfp8_matmuls(self) -> list[str]:
        """Bare-parameter products this module can run in MXFP8 (both expert GEMMs)."""
        ok = self.dim % 128 == 0 and self.hidden % 128 == 0
        return ["w_in", "w_out"] if ok else []

    def enable_mxfp8(self) -> None:
        if self.mxfp8_matmuls():
            self.mxfp8_experts = True
            self._q_in = self._q_out = None

    @torch.no_grad()
    def refresh_mxfp8(self) -> bool:
        """Rebuild the cached fp8 copies of the expert weights (after every optimizer step)."""
        if not self.mxfp8_experts or not moe_ops.native.available() or not self.w_in.is_cuda \
                or self.w_in.dtype != torch.bfloat16:
            return False
        from kohakuwullm_b200.ops.mxfp8 import GroupedQuantizedWeight

        if self._q_in is None or self._q_in.shape != tuple(self.w_in.shape):
            self._q_in, self._q_out = GroupedQuantizedWeight(self.w_in), GroupedQuantizedWeight(self.w_out)
        else:
            self._q_in.refresh(self.w_in)
            self._q_out.refresh(self.w_out)
        return True

    def _quantized(self, flat):
        if not self.mxfp8_experts or not moe_ops.native_supported(flat, self.w_in):
            return None, None
        if self._q_in is None or self._q_in.shape != tuple(self.w_in.shape):
            self.refresh_mxfp8()
        return self._q_in, self._q_out

    def forward(self, x):
        shape = x.shape
        flat = x.reshape(-1, shape[-1])
        idx, w, counts = self.router.route(flat)
        if self.ep_world > 1:
            from kohakuwullm_b200.parallel import ep as ep_ops

            if self.ep is not None and moe_ops.native_supported(flat, self.w_in):
                q_in, q_out = self._quantized(flat)
                y = ep_ops.ep_routed_experts(self.ep, flat, idx, w, counts, self.w_in, self.w_out, q_in, q_out)
            else:
                y = ep_ops.reference_ep_forward(flat, idx, w, self.w_in, self.w_out, self.ep_group)
            if self.shared is not None:
                y = y + self.shared(flat)
            return y.reshape(shape)
        path = self.expert_path or ("grouped" if moe_ops.native_supported(flat, self.w_in) else "eager")
        if path == "grouped":
            q_in, q_out = self._quantized(flat)
            y = moe_ops.routed_experts(flat, idx, w, counts, self.w_in, self.w_out, q_in, q_out)
        else:
            y = moe_ops.routed_experts_reference(flat, idx, w, self.w_in, self.w_out)
        if self.shared is not None:
            y = y + self.shared(flat)
        return y.reshape(shape)


MLP.register("moe", MoEMLP)
