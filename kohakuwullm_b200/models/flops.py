"""Analytic FLOP accounting (model FLOPs for MFU, hardware FLOPs for HFU).

Per token: ``2 * (active parameters - embedding)`` for the blocks' matmuls plus ``2 * dim * vocab`` for
the head; attention adds ``4 * q_dim * pairs`` where ``pairs`` is the number of (query, key) pairs the
batch's own document lengths give: ``L(L+1)/2`` for a full-causal layer and ``L*w - w(w-1)/2`` (L > w) for a
window of ``w``. Training multiplies by 3 (forward + backward); hardware FLOPs add one more forward of the
blocks under activation checkpointing. Reference: src/kohakuwullm/models/flops.py:17-96.
"""

from __future__ import annotations

from typing import Sequence

from kohakuwullm_b200.utils.misc import count_active_parameters


def attention_pairs(length: int, window: int | None) -> float:
    L = float(length)
    if window is None or window >= length:
        return L * (L + 1) / 2
    w = float(window)
    return L * w - w * (w - 1) / 2


class FlopCounter:
    def __init__(self, backbone):
        cfg = backbone.config
        self.config = cfg
        self.embed_params = backbone.embed.weight.numel()
        head = 0 if backbone.head.tied else backbone.head.weight.numel()
        self.active_block_params = count_active_parameters(backbone) - self.embed_params - head
        self.head_flops_per_token = 2.0 * cfg.dim * cfg.vocab_size
        self.q_dim = cfg.heads * cfg.head_dim
        self.windows = cfg.windows
        self.grad_ckpt = cfg.grad_ckpt

    def forward_flops(self, lengths: Sequence[int], stage_layers: range | None = None, with_head: bool = True) -> float:
        tokens = float(sum(lengths))
        layers = range(self.config.depth) if stage_layers is None else stage_layers
        share = len(layers) / self.config.depth
        flops = 2.0 * self.active_block_params * share * tokens
        for layer in layers:
            w = self.windows[layer]
            flops += 4.0 * self.q_dim * sum(attention_pairs(n, w) for n in lengths)
        if with_head:
            flops += self.head_flops_per_token * tokens
        return flops

    def step_flops(self, lengths: Sequence[int], stage_layers: range | None = None, with_head: bool = True):
        """``(model_flops, hardware_flops)`` of one training pass over documents of these lengths."""
        fwd = self.forward_flops(lengths, stage_layers, with_head)
        model = 3.0 * fwd
        hardware = model
        if self.grad_ckpt:
            hardware += self.forward_flops(lengths, stage_layers, with_head=False)
        return model, hardware
