"""Normalisation layers. Weights stay fp32 whatever the compute dtype.

``rmsnorm`` runs the native fused kernel on bf16 CUDA input (optionally fused with the residual
add, see :func:`kohakuwullm_b200.ops.elementwise.rmsnorm`) and plain PyTorch elsewhere.
Reference: src/kohakuwullm/models/components/norm.py:16-101.
"""

from __future__ import annotations

import torch
from torch import nn

from kohakuwullm_b200.ops.elementwise import rmsnorm
from kohakuwullm_b200.registry import NORM


class RMSNorm(nn.Module):
    one_plus = False

    def __init__(self, dim: int, eps: float = 1e-6, affine: bool = True):
        super().__init__()
        self.dim, self.eps = dim, eps
        init = torch.zeros(dim) if self.one_plus else torch.ones(dim)
        self.weight = nn.Parameter(init) if affine else None
        # set by the MXFP8 wiring: the output / the input gradient feeds an MXFP8 linear, so the kernel
        # writes the fp8 copy in the same pass
        self.emit_mx = False
        self.emit_mx_grad = False

    def forward(self, x, residual=None):
        """``norm(x)``, or with ``residual``: ``(norm(x + residual), x + residual)``."""
        return rmsnorm(x, self.weight, self.eps, self.one_plus, residual, self.emit_mx, self.emit_mx_grad)

    def extra_repr(self):
        return f"{self.dim}, eps={self.eps}, affine={self.weight is not None}"


class GemmaRMSNorm(RMSNorm):
    """Scale is ``1 + weight`` with a zero-initialised weight."""

    one_plus = True


class LayerNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6, affine: bool = True):
        super().__init__()
        self.norm = nn.LayerNorm(dim, eps=eps, elementwise_affine=affine)

    def forward(self, x, residual=None):
        h = x if residual is None else x + residual
        y = self.norm(h.float()).to(h.dtype)
        return y if residual is None else (y, h)


class DyT(nn.Module):
    """Dynamic tanh: ``weight * tanh(alpha * x) + bias`` — a normalisation-free stand-in."""

    def __init__(self, dim: int, eps: float = 1e-6, affine: bool = True, alpha_init: float = 0.5):
        super().__init__()
        self.alpha = nn.Parameter(torch.full((1,), alpha_init))
        self.weight = nn.Parameter(torch.ones(dim))
        self.bias = nn.Parameter(torch.zeros(dim))

    def forward(self, x, residual=None):
        h = x if residual is None else x + residual
        y = (self.weight * torch.tanh(self.alpha * h.float()) + self.bias).to(h.dtype)
        return y if residual is None else (y, h)


NORM.register("rmsnorm", RMSNorm)
NORM.register("rmsnorm_native", RMSNorm)
NORM.register("rmsnorm_triton", RMSNorm)  # name kept so reference configs load; same native kernel
NORM.register("gemma_rmsnorm", GemmaRMSNorm)
NORM.register("layernorm", LayerNorm)
NORM.register("dyt", DyT)
