"""Dense feed-forward blocks.

``GLUMLP`` keeps gate and value in ONE projection ``w_in`` (dim -> 2*hidden) so a single GEMM feeds
the fused SwiGLU kernel, which reads the two halves in place. Reference:
src/kohakuwullm/models/components/mlp.py:15-126.
"""

from __future__ import annotations

import torch
from torch import nn

from kohakuwullm_b200.ops.elementwise import swiglu
from kohakuwullm_b200.ops.gemm import linear
from kohakuwullm_b200.registry import MLP


def resolve_hidden(dim: int, ratio: float = 4.0, hidden: int | None = None, multiple_of: int = 128,
                   glu: bool = True) -> int:
    """Hidden width: explicit value, else ``ratio * dim`` (times 2/3 for gated units), rounded UP."""
    if hidden is not None:
        return int(hidden)
    h = dim * ratio * (2.0 / 3.0 if glu else 1.0)
    return int(-(-h // multiple_of) * multiple_of)


class Linear(nn.Module):
    """Weight-only (optionally biased) linear layer running on the tcgen05 GEMM."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None
        # set by swap_mxfp8: marks the layer as MXFP8; the quantised copies are built lazily on the
        # weight's device and dropped whenever the module is moved or cast
        self.mxfp8 = False
        self._qweight = None

    def _apply(self, fn, recurse=True):
        self._qweight = None
        return super()._apply(fn, recurse)

    def quantized_weight(self, rows_hint: int = 4096):
        """The MXFP8 copies, built at first use; ``rows_hint`` (the row count of the first input) picks the GEMM
        tile widths the copies' scales are laid out for."""
        from kohakuwullm_b200.ops.mxfp8 import QuantizedWeight

        if self._qweight is None:
            self._qweight = QuantizedWeight(self.weight.detach(), rows_hint)
        return self._qweight

    def refresh_quantized_weight(self) -> bool:
        """Re-quantise after an optimizer step. Returns True when this layer holds MXFP8 copies."""
        if not self.mxfp8 or self._qweight is None:
            return self.mxfp8
        self._qweight.refresh(self.weight.detach())
        return True

    def forward(self, x):
        if self.mxfp8 and self.bias is None:
            from kohakuwullm_b200.ops import mxfp8 as mx

            if mx.supported(x, self.weight):
                return mx.mxfp8_linear(x, self.weight, self.quantized_weight(x.numel() // x.shape[-1]))
        return linear(x, self.weight, self.bias)

    def extra_repr(self):
        return f"{self.in_features} -> {self.out_features}, bias={self.bias is not None}"


class GLUMLP(nn.Module):
    activation = "silu"

    def __init__(self, dim: int, hidden: int | None = None, ratio: float = 4.0, multiple_of: int = 128,
                 bias: bool = False, **_unused):
        super().__init__()
        self.dim = dim
        self.hidden = resolve_hidden(dim, ratio, hidden, multiple_of, glu=True)
        self.w_in = Linear(dim, 2 * self.hidden, bias)
        self.w_out = Linear(self.hidden, dim, bias)

    def forward(self, x):
        h = self.w_in(x)
        if self.activation == "silu":
            # with MXFP8 projections the activation kernel also writes the fp8 copies its neighbours consume
            a = swiglu(h, emit_mx=self.w_out.mxfp8, emit_mx_grad=self.w_in.mxfp8)
        else:
            g, v = h.chunk(2, dim=-1)
            a = torch.nn.functional.gelu(g, approximate="tanh") * v
        return self.w_out(a)


class GeGLUMLP(GLUMLP):
    activation = "gelu"


class GELUMLP(nn.Module):
    def __init__(self, dim: int, hidden: int | None = None, ratio: float = 4.0, multiple_of: int = 128,
                 bias: bool = False, **_unused):
        super().__init__()
        self.hidden = resolve_hidden(dim, ratio, hidden, multiple_of, glu=False)
        self.fc1 = Linear(dim, self.hidden, bias)
        self.fc2 = Linear(self.hidden, dim, bias)

    def forward(self, x):
        return self.fc2(torch.nn.functional.gelu(self.fc1(x)))


MLP.register("swiglu", GLUMLP)
MLP.register("swiglu_native", GLUMLP)
MLP.register("swiglu_triton", GLUMLP)  # name kept so reference configs load
MLP.register("geglu", GeGLUMLP)
MLP.register("gelu", GELUMLP)
