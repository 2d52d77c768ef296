"""Rotary position encoding with linear / NTK / YaRN context scaling, and NoPE.

``prepare(position_ids)`` is called once per forward and returns the per-token half tables
``(cos, sin)`` of shape (tokens, rot/2) in fp32; attention layers consume them through the fused
QK-norm + RoPE kernel. Scaling rules (reference: src/kohakuwullm/models/components/posenc.py:21-168):

* ``linear``: positions divided by ``factor``;
* ``ntk``:    base multiplied by ``factor ** (d / (d - 2))``;
* ``yarn``:   per-frequency blend between interpolated and original frequencies with a linear ramp
              between the correction dims of ``beta_fast`` = 32 and ``beta_slow`` = 1 rotations over
              ``original_context``; ``attn_scale = 0.1 ln(factor) + 1`` is folded into cos and sin.
"""

from __future__ import annotations

import math
from typing import NamedTuple

import torch
from torch import nn

from kohakuwullm_b200.registry import POSENC


class RotaryCache(NamedTuple):
    cos: torch.Tensor | None
    sin: torch.Tensor | None


def _yarn_correction_dim(rotations: float, dim: int, base: float, context: int) -> float:
    return dim * math.log(context / (rotations * 2 * math.pi)) / (2 * math.log(base))


def build_inv_freq(head_dim: int, theta: float, scaling: str | None, factor: float,
                   original_context: int, partial: float = 1.0, beta_fast: float = 32.0,
                   beta_slow: float = 1.0) -> tuple[torch.Tensor, float, float]:
    """Returns ``(inv_freq (rot/2,), position_scale, attn_scale)``."""
    rot = int(head_dim * partial) // 2 * 2
    idx = torch.arange(0, rot, 2, dtype=torch.float64)
    pos_scale, attn_scale = 1.0, 1.0
    if scaling in (None, "none"):
        inv = theta ** (-idx / rot)
    elif scaling == "linear":
        inv = theta ** (-idx / rot)
        pos_scale = 1.0 / factor
    elif scaling == "ntk":
        base = theta * factor ** (rot / max(rot - 2, 1))
        inv = base ** (-idx / rot)
    elif scaling == "yarn":
        extrap = theta ** (-idx / rot)
        interp = extrap / factor
        low = max(math.floor(_yarn_correction_dim(beta_fast, rot, theta, original_context)), 0)
        high = min(math.ceil(_yarn_correction_dim(beta_slow, rot, theta, original_context)), rot // 2 - 1)
        if high == low:
            high = low + 1e-3
        ramp = ((torch.arange(rot // 2, dtype=torch.float64) - low) / (high - low)).clamp(0, 1)
        inv = interp * ramp + extrap * (1 - ramp)
        attn_scale = 0.1 * math.log(factor) + 1.0 if factor > 1 else 1.0
    else:
        raise ValueError(f"unknown rope scaling {scaling!r}")
    return inv.float(), pos_scale, attn_scale


class RoPE(nn.Module):
    def __init__(self, head_dim: int, theta: float = 10000.0, scaling: str | None = None,
                 factor: float = 1.0, max_position: int = 8192, partial: float = 1.0, **_unused):
        super().__init__()
        inv, self.pos_scale, self.attn_scale = build_inv_freq(head_dim, theta, scaling, factor,
                                                              max_position, partial)
        self.register_buffer("inv_freq", inv, persistent=False)
        self.rot = 2 * inv.numel()

    def prepare(self, position_ids: torch.Tensor) -> RotaryCache:
        pos = position_ids.reshape(-1).to(torch.float32) * self.pos_scale
        ang = pos[:, None] * self.inv_freq[None, :].to(pos.device)
        cos, sin = ang.cos(), ang.sin()
        if self.attn_scale != 1.0:
            cos, sin = cos * self.attn_scale, sin * self.attn_scale
        return RotaryCache(cos.contiguous(), sin.contiguous())


class NoPE(nn.Module):
    def __init__(self, head_dim: int = 0, **_unused):
        super().__init__()

    def prepare(self, position_ids: torch.Tensor) -> RotaryCache:
        return RotaryCache(None, None)


POSENC.register("rope", RoPE)
POSENC.register("nope", NoPE)
POSENC.register("none", NoPE)
