"""Low-precision parameter storage.

``cast_parameters_`` moves a model's matrices to a 16-bit dtype in place while the numerically
delicate parameters stay fp32: anything whose qualified name contains one of ``KEEP_FP32_DEFAULT``
(norm scales, router gates, rotary tables, sink logits, biases). Reference:
src/kohakuwullm/training/optim/lowbit.py:10-60.
"""

from __future__ import annotations

import torch
from torch import nn

KEEP_FP32_DEFAULT = ("norm", "router", "inv_freq", "freq_dirs", "sink", "bias")


def keeps_fp32(name: str, keep=KEEP_FP32_DEFAULT) -> bool:
    return any(key in name for key in keep)


@torch.no_grad()
def cast_parameters_(module: nn.Module, dtype: torch.dtype, keep_fp32=KEEP_FP32_DEFAULT) -> nn.Module:
    for name, p in module.named_parameters():
        if p.is_floating_point() and not keeps_fp32(name, keep_fp32):
            p.data = p.data.to(dtype)
    for name, b in module.named_buffers():
        if b.is_floating_point() and not keeps_fp32(name, keep_fp32) and b.dtype != torch.float32:
            b.data = b.data.to(dtype)
    return module
