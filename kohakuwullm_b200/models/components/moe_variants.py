"""Routing and expert-layer variants next to the DeepSeekMoE default.

``sinkhorn``       while training: assignment from a Sinkhorn-balanced matrix (3 iterations, temperature 0.05,
                   log domain), gate weight from the raw softmax; in evaluation: each token's own top-k;
``expert_choice``  every expert takes its ``capacity`` best tokens (kept for experiments; it has no
                   token-choice ``route`` and raises if wired into ``MoEMLP``);
``relu``           ReMoE: ``relu(logits)`` gates, sparsity steered by an L1 coefficient that is multiplied by
                   ``alpha ** sign(target - observed)`` every step; tokens with more than ``max_slots``
                   active experts keep the strongest ones;
``PerLayerEmbedding``  a small per-layer token embedding added through a zero-initialised up-projection;
``latent_moe``     experts run at a reduced ``latent`` width: down-projection -> inner MoE (routed on the
                   full-width input) -> up-projection, shared expert at full width.
Reference: src/kohakuwullm/models/components/moe_variants.py:16-340.
"""

from __future__ import annotations

import torch
from torch import nn

from kohakuwullm_b200.models.components.mlp import GLUMLP, Linear
from kohakuwullm_b200.models.components.moe import MoEMLP, TopKRouter
from kohakuwullm_b200.registry import MLP, ROUTER


class SinkhornRouter(TopKRouter):
    def __init__(self, *args, iterations: int = 3, temperature: float = 0.05, **kw):
        kw.setdefault("score", "softmax")
        super().__init__(*args, **kw)
        self.iterations, self.temperature = iterations, temperature

    def route(self, x):
        logits = torch.nn.functional.linear(x.float(), self.weight.float())
        if not self.training:
            # the balanced assignment depends on which tokens share the batch, which is not causal: decoding one
            # token at a time and recomputing the whole prefix would pick different experts. Evaluation and
            # generation therefore take the plain top-k of each token's own scores.
            s = torch.softmax(logits, -1)
            w, idx = s.topk(self.top_k, dim=-1)
            if self.norm_topk_prob:
                w = w / (w.sum(-1, keepdim=True) + 1e-20)
            self.aux_loss = None
            counts = torch.bincount(idx.reshape(-1), minlength=self.num_experts).to(torch.int32)
            return idx, w * self.routed_scaling_factor, counts
        with torch.no_grad():
            # in the log domain: dividing logits by a small temperature spans hundreds of e-folds, which underflows
            # a plain exp() to a matrix of floor values and collapses the assignment onto one expert
            cost = logits / self.temperature
            for _ in range(self.iterations):
                cost = cost - torch.logsumexp(cost, dim=0, keepdim=True)      # balance experts
                cost = cost - torch.logsumexp(cost, dim=1, keepdim=True)      # normalise tokens
            idx = cost.topk(self.top_k, dim=-1).indices
        s = torch.softmax(logits, -1)
        w = s.gather(1, idx)
        if self.norm_topk_prob:
            w = w / (w.sum(-1, keepdim=True) + 1e-20)
        counts = torch.bincount(idx.reshape(-1), minlength=self.num_experts).to(torch.int32)
        if self.training:
            with torch.no_grad():
                self.load_accum += counts.to(self.load_accum.dtype)
        self.aux_loss = self._aux(logits, s, counts) if self.training else None
        return idx, w * self.routed_scaling_factor, counts


class ExpertChoiceRouter(nn.Module):
    def __init__(self, dim: int, num_experts: int, top_k: int, capacity_factor: float = 1.0, **_unused):
        super().__init__()
        self.num_experts, self.top_k, self.capacity_factor = num_experts, top_k, capacity_factor
        self.weight = nn.Parameter(torch.empty(num_experts, dim))
        self.aux_loss = None

    def choose(self, x):
        """(E, capacity) token indices and their gate weights."""
        s = torch.softmax(torch.nn.functional.linear(x.float(), self.weight.float()), -1)
        cap = max(1, int(self.capacity_factor * x.shape[0] * self.top_k / self.num_experts))
        w, tok = s.t().topk(min(cap, x.shape[0]), dim=-1)
        return tok, w

    def route(self, x):
        raise NotImplementedError("expert-choice routing picks tokens per expert; MoEMLP dispatches per token")


class ReLURouter(TopKRouter):
    """ReMoE. ``top_k`` is the TARGET number of active experts per token."""

    def __init__(self, *args, l1_init: float = 1e-8, alpha: float = 1.2, max_slots: int | None = None, **kw):
        super().__init__(*args, **kw)
        self.alpha = alpha
        self.max_slots = max_slots or 2 * self.top_k
        self.register_buffer("l1_coeff", torch.tensor(l1_init))
        self.register_buffer("active_accum", torch.zeros(2))   # (active experts, tokens)

    def route(self, x):
        logits = torch.nn.functional.linear(x.float(), self.weight.float())
        g = torch.relu(logits)
        k = min(self.max_slots, self.num_experts)
        w, idx = g.topk(k, dim=-1)                           # inactive slots carry weight 0
        counts = torch.bincount(idx[w > 0].reshape(-1), minlength=self.num_experts).to(torch.int32)
        if self.training:
            with torch.no_grad():
                self.load_accum += counts.to(self.load_accum.dtype)
                self.active_accum += torch.stack([(g > 0).sum().float(), torch.tensor(float(x.shape[0]), device=x.device)])
            self.aux_loss = self.l1_coeff * g.sum(-1).mean()
        else:
            self.aux_loss = None
        return idx, w, torch.bincount(idx.reshape(-1), minlength=self.num_experts).to(torch.int32)

    @torch.no_grad()
    def update_bias(self, rate_scale: float = 1.0):
        observed = self.active_accum[0] / self.active_accum[1].clamp(min=1)
        self.l1_coeff *= self.alpha ** torch.sign(observed - self.top_k)
        self.active_accum.zero_()
        return super().update_bias(0.0)


ROUTER.register("sinkhorn", SinkhornRouter)
ROUTER.register("expert_choice", ExpertChoiceRouter)
ROUTER.register("relu", ReLURouter)


class PerLayerEmbedding(nn.Module):
    def __init__(self, vocab_size: int, dim: int, ple_dim: int = 64):
        super().__init__()
        self.embed = nn.Embedding(vocab_size, ple_dim)
        self.up = Linear(ple_dim, dim)
        nn.init.zeros_(self.up.weight)

    def forward(self, hidden, tokens):
        return hidden + self.up(self.embed(tokens).to(hidden.dtype))


class LatentMoEMLP(nn.Module):
    def __init__(self, dim: int, latent: int | None = None, num_experts: int = 64, top_k: int = 8, num_shared: int = 1,
                 hidden: int | None = None, **kw):
        super().__init__()
        latent = latent or dim // 2
        self.down = Linear(dim, latent)
        self.up = Linear(latent, dim)
        self.inner = MoEMLP(latent, num_experts=num_experts, top_k=top_k, num_shared=0, hidden=hidden, router_dim=dim, **kw)
        self.shared = GLUMLP(dim, hidden=(hidden or latent) * num_shared) if num_shared else None
        self.router = self.inner.router

    def forward(self, x):
        from kohakuwullm_b200.ops import moe as moe_ops

        flat = x.reshape(-1, x.shape[-1])
        idx, w, counts = self.inner.router.route(flat)              # routed on the full-width input
        z = self.down(flat)
        if moe_ops.native_supported(z, self.inner.w_in):
            y = moe_ops.routed_experts(z, idx, w, counts, self.inner.w_in, self.inner.w_out)
        else:
            y = moe_ops.routed_experts_reference(z, idx, w, self.inner.w_in, self.inner.w_out)
        out = self.up(y)
        if self.shared is not None:
            out = out + self.shared(flat)
        return out.reshape(x.shape)


MLP.register("latent_moe", LatentMoEMLP)
