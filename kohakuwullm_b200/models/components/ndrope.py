"""N-dimensional rotary encodings for tokens that carry a position VECTOR (image patches, time + space).

Each rotary frequency ``k`` has a unit direction ``u_k`` in position space and a magnitude ``w_k``
(log-spaced); the rotation angle of a token at position ``p`` is ``w_k * <u_k, p>``.
``NDRoPE`` spreads the directions with the golden-angle (2-D) / generalized golden-ratio Kronecker sequence
(N-D) so every pair of axes is mixed evenly; ``GGRoPE`` is the same with learnable directions;
``axial`` assigns whole frequency bands to single axes. A share ``zero_freq_ratio`` of the frequencies is
pinned to zero (pure content channels). Reference: src/kohakuwullm/models/components/ndrope.py:20-143.
"""

from __future__ import annotations

import math

import torch
from torch import nn

from kohakuwullm_b200.models.components.posenc import RotaryCache
from kohakuwullm_b200.registry import POSENC


def _generalized_golden(ndim: int) -> float:
    """Positive root of x^(n+1) = x + 1 (the golden ratio for n = 1)."""
    x = 2.0
    for _ in range(64):
        x = (1 + x) ** (1.0 / (ndim + 1))
    return x


def kronecker_directions(n_freq: int, ndim: int) -> torch.Tensor:
    """(n_freq, ndim) unit vectors from the low-discrepancy Kronecker sequence of the generalized golden ratio."""
    if ndim == 1:
        return torch.ones(n_freq, 1)
    g = _generalized_golden(ndim - 1)
    alphas = torch.tensor([(1.0 / g) ** (j + 1) for j in range(ndim - 1)], dtype=torch.float64)
    k = torch.arange(1, n_freq + 1, dtype=torch.float64)[:, None]
    u = (0.5 + k * alphas[None, :]) % 1.0
    if ndim == 2:
        ang = math.pi * u[:, 0]
        d = torch.stack([ang.cos(), ang.sin()], -1)
    else:
        # inverse-CDF map of the cube to the half-sphere via normalised Gaussians
        z = torch.erfinv((2 * torch.cat([u, ((k * (1.0 / g) ** ndim + 0.5) % 1.0)], -1) - 1).clamp(-0.999999, 0.999999))
        d = z / z.norm(dim=-1, keepdim=True).clamp(min=1e-9)
    return d.float()


class NDRoPE(nn.Module):
    learned = False

    def __init__(self, head_dim: int, ndim: int = 2, theta: float = 10000.0, zero_freq_ratio: float = 0.0,
                 variant: str = "golden", partial: float = 1.0, **_unused):
        super().__init__()
        rot = int(head_dim * partial) // 2 * 2
        n = rot // 2
        n_zero = int(n * zero_freq_ratio)
        mags = theta ** (-torch.arange(n - n_zero, dtype=torch.float32) / max(n - n_zero, 1))
        mags = torch.cat([mags, torch.zeros(n_zero)])
        if variant == "axial":
            dirs = torch.zeros(n, ndim)
            dirs[torch.arange(n), torch.arange(n) % ndim] = 1.0
        else:
            dirs = kronecker_directions(n, ndim)
        self.ndim, self.rot = ndim, rot
        self.register_buffer("inv_freq", mags, persistent=False)
        if self.learned:
            self.freq_dirs = nn.Parameter(dirs)
        else:
            self.register_buffer("freq_dirs", dirs, persistent=False)

    def prepare(self, position_ids: torch.Tensor) -> RotaryCache:
        """position_ids (..., ndim) (a trailing axis of size 1 is added for plain 1-D positions)."""
        pos = position_ids.to(torch.float32)
        if pos.dim() == 1 or pos.shape[-1] != self.ndim:
            pos = pos.reshape(-1, 1).expand(-1, self.ndim) if self.ndim > 1 and pos.dim() == 1 else pos.reshape(-1, self.ndim)
        pos = pos.reshape(-1, self.ndim)
        dirs = torch.nn.functional.normalize(self.freq_dirs.float(), dim=-1) if self.learned else self.freq_dirs
        ang = (pos @ dirs.t().to(pos.device)) * self.inv_freq.to(pos.device)[None, :]
        return RotaryCache(ang.cos().contiguous(), ang.sin().contiguous())


class GGRoPE(NDRoPE):
    """Generalized-golden directions as a learnable parameter (kept fp32 by ``cast_parameters_``)."""

    learned = True


POSENC.register("ndrope", NDRoPE)
POSENC.register("ggrope", GGRoPE)
