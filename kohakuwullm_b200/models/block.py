"""Pre-norm decoder block: ``x + attn(norm(x))`` then ``x + mlp(norm(x))``.

The residual stream is carried as ``(x, pending)``: ``pending`` is a branch output that has not been
added yet, so the add is fused into the next RMSNorm kernel (one pass instead of add + norm). A caller
that wants the plain tensor adds ``pending`` itself (``DecoderBlock.merge``). Reference:
src/kohakuwullm/models/block.py:12-73.
"""

from __future__ import annotations

from torch import nn

from kohakuwullm_b200.registry import ATTENTION, MLP, NORM, build


class DecoderBlock(nn.Module):
    def __init__(self, dim, norm, attn, mlp, norm_eps=1e-6, post_norm=False, residual_scale=1.0,
                 attn_kwargs=None, mlp_kwargs=None):
        super().__init__()
        self.norm_attn = build(norm, NORM, dim=dim, eps=norm_eps)
        self.attn = build(attn, ATTENTION, dim=dim, **(attn_kwargs or {}))
        self.norm_mlp = build(norm, NORM, dim=dim, eps=norm_eps)
        self.mlp = build(mlp, MLP, dim=dim, **(mlp_kwargs or {}))
        self.post_attn = build(norm, NORM, dim=dim, eps=norm_eps) if post_norm else None
        self.post_mlp = build(norm, NORM, dim=dim, eps=norm_eps) if post_norm else None
        self.residual_scale = residual_scale

    @staticmethod
    def merge(x, pending):
        return x if pending is None else x + pending

    def forward_deferred(self, x, pending, seq_info, rope=None, cache=None, layer=0, plan=None):
        """Returns ``(x, pending)``; the true hidden state is ``x + pending``."""
        s = self.residual_scale
        if pending is None:
            n = self.norm_attn(x)
        else:
            n, x = self.norm_attn(pending, residual=x)
        a = self.attn(n, seq_info, rope, cache=cache, layer=layer, plan=plan)
        if self.post_attn is not None:
            a = self.post_attn(a)
        if s != 1.0:
            a = a * s
        n, x = self.norm_mlp(a, residual=x)
        m = self.mlp(n)
        if self.post_mlp is not None:
            m = self.post_mlp(m)
        if s != 1.0:
            m = m * s
        return x, m

    def forward(self, x, seq_info, rope=None, cache=None, layer=0, plan=None):
        x, pending = self.forward_deferred(x, None, seq_info, rope, cache, layer, plan)
        return x + pending
