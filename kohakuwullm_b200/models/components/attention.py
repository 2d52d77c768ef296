"""Self-attention layer: fused QKV projection, per-head QK-RMSNorm, RoPE, GQA, sliding window,
attention sinks.

Training (packed) path::

    qkv = x @ Wqkv^T                                  one tcgen05 GEMM
    q,k = rope(rmsnorm_head(qkv[q|k]))                one fused kernel per tensor, reading the
                                                      strided q / k slices of ``qkv`` in place
    out = flash(q, k, v=qkv[v-slice], cu_seqlens)     tcgen05 flash attention, v read in place by TMA
    y   = out @ Wo^T

Padded path (``seq_info.packed`` false: evaluation, KV-cache decode): explicit-mask softmax in
PyTorch with the same sink semantics. The q/k/v projections are stored as ONE parameter
``qkv_proj.weight`` with rows ordered ``[q heads | k heads | v heads]``; ``split_qkv`` gives the three
views an exporter needs. Reference: src/kohakuwullm/models/components/attention.py:18-471.
"""

from __future__ import annotations

import math

import torch
from torch import nn

from kohakuwullm_b200.models.components.mlp import Linear
from kohakuwullm_b200.ops import attention as attn_ops
from kohakuwullm_b200.ops.attention import varlen_attention
from kohakuwullm_b200.ops.elementwise import qknorm_rope
from kohakuwullm_b200.registry import ATTENTION


class Attention(nn.Module):
    backend = "flash"

    def __init__(self, dim: int, heads: int, kv_heads: int | None = None, head_dim: int | None = None,
                 qk_norm: bool = True, qk_norm_affine: bool = True, bias: bool = False,
                 window: int | None = None, sink: bool = False, num_sinks: int = 1,
                 norm_eps: float = 1e-6, **_unused):
        super().__init__()
        self.dim, self.heads = dim, heads
        self.kv_heads = kv_heads or heads
        self.head_dim = head_dim or dim // heads
        self.window = window
        self.q_dim = self.heads * self.head_dim
        self.kv_dim = self.kv_heads * self.head_dim
        self.qkv_proj = Linear(dim, self.q_dim + 2 * self.kv_dim, bias)
        self.o_proj = Linear(self.q_dim, dim, bias)
        self.qk_norm = qk_norm
        self.norm_eps = norm_eps
        if qk_norm and qk_norm_affine:
            self.q_norm = nn.Parameter(torch.ones(self.head_dim))
            self.k_norm = nn.Parameter(torch.ones(self.head_dim))
        else:
            self.q_norm = self.k_norm = None
        # learned sink logits: softmax columns with a zero value
        self.sink = nn.Parameter(torch.zeros(self.heads, num_sinks)) if sink else None
        self.scale = 1.0 / math.sqrt(self.head_dim)

    # ------------------------------------------------------------------ helpers
    def split_qkv(self):
        w = self.qkv_proj.weight
        return w[: self.q_dim], w[self.q_dim: self.q_dim + self.kv_dim], w[self.q_dim + self.kv_dim:]

    def _sink_lse(self):
        return None if self.sink is None else torch.logsumexp(self.sink.float(), dim=-1)

    def _project(self, x2, rope):
        """x2 (T, dim) -> q (T,H,D), k (T,Hkv,D), v (T,Hkv,D) with norm and rotation applied."""
        T = x2.shape[0]
        qkv = self.qkv_proj(x2)
        q = qkv[:, : self.q_dim].view(T, self.heads, self.head_dim)
        k = qkv[:, self.q_dim: self.q_dim + self.kv_dim].view(T, self.kv_heads, self.head_dim)
        v = qkv[:, self.q_dim + self.kv_dim:].view(T, self.kv_heads, self.head_dim)
        cos, sin = (rope.cos, rope.sin) if rope is not None else (None, None)
        if self.qk_norm or cos is not None:
            q = qknorm_rope(q, self.q_norm, cos, sin, self.norm_eps, self.qk_norm)
            k = qknorm_rope(k, self.k_norm, cos, sin, self.norm_eps, self.qk_norm)
        return q, k, v

    # ------------------------------------------------------------------ forward
    def forward(self, x, seq_info, rope=None, cache=None, layer: int = 0, plan=None):
        if seq_info.packed and cache is None:
            T = x.shape[0]
            cos, sin = (rope.cos, rope.sin) if rope is not None else (None, None)
            if type(self) is Attention and attn_ops.attention_core_supported(x, self.head_dim, self.q_norm,
                                                                             self.k_norm, cos):
                qkv = self.qkv_proj(x)
                out = attn_ops.attention_core(qkv, self.q_norm, self.k_norm, cos, sin, seq_info.cu_seqlens,
                                              plan, self._sink_lse(), self.heads, self.kv_heads, self.window,
                                              self.scale, self.norm_eps, self.qk_norm,
                                              emit_mx_grad=bool(getattr(self.qkv_proj, "mxfp8", False)),
                                              emit_mx_out=bool(getattr(self.o_proj, "mxfp8", False)))
                return self.o_proj(out.reshape(T, self.q_dim))
            q, k, v = self._project(x, rope)
            out = varlen_attention(q, k, v, seq_info.cu_seqlens, seq_info.max_seqlen, window=self.window,
                                   sink_lse=self._sink_lse(), scale=self.scale, plan=plan)
            return self.o_proj(out.reshape(T, self.q_dim))
        return self._forward_padded(x, seq_info, rope, cache, layer)

    def _forward_padded(self, x, seq_info, rope, cache, layer):
        B, S, _ = x.shape
        q, k, v = self._project(x.reshape(B * S, -1), rope)
        q = q.view(B, S, self.heads, self.head_dim)
        k = k.view(B, S, self.kv_heads, self.head_dim)
        v = v.view(B, S, self.kv_heads, self.head_dim)
        q_pos = seq_info.position_ids  # (B, S) absolute positions of the queries
        if cache is not None:
            k, v, k_pos, k_valid = cache.append(layer, k, v, q_pos)
            if S == 1 and not torch.is_grad_enabled() and attn_ops.decode_supported(q[:, 0], k) \
                    and q.is_contiguous():
                # one new token per row: split-KV decode kernel straight over the cache buffers
                out = attn_ops.decode_attention(q[:, 0], k, v, cache.length + 1, self.window, self.scale, self.sink)
                return self.o_proj(out.reshape(B, 1, self.q_dim))
        else:
            k_pos = q_pos
            k_valid = torch.ones(B, S, dtype=torch.bool, device=x.device)
        out = self.attend(q, k, v, q_pos, k_pos, k_valid)
        return self.o_proj(out.reshape(B, S, self.q_dim))

    def attend(self, q, k, v, q_pos, k_pos, k_valid):
        """Explicit-mask attention for padded / cached layouts. q (B,S,H,D); k,v (B,L,Hkv,D)."""
        group = self.heads // self.kv_heads
        qf = q.float().permute(0, 2, 1, 3)                                  # (B,H,S,D)
        kf = k.float().permute(0, 2, 1, 3).repeat_interleave(group, 1)     # (B,H,L,D)
        vf = v.float().permute(0, 2, 1, 3).repeat_interleave(group, 1)
        scores = torch.matmul(qf, kf.transpose(-1, -2)) * self.scale       # (B,H,S,L)
        ok = (k_pos[:, None, :] <= q_pos[:, :, None]) & k_valid[:, None, :]
        if self.window is not None:
            ok &= (q_pos[:, :, None] - k_pos[:, None, :]) < self.window
        scores = scores.masked_fill(~ok[:, None], float("-inf"))
        lse = torch.logsumexp(scores, dim=-1)
        sink = self._sink_lse()
        if sink is not None:
            lse = torch.logaddexp(lse, sink[None, :, None])
        p = torch.exp(scores - lse[..., None])
        p = torch.nan_to_num(p, nan=0.0)
        return torch.matmul(p, vf).permute(0, 2, 1, 3).to(q.dtype)          # (B,S,H,D)


class SDPAAttention(Attention):
    """Always the explicit-mask PyTorch path (packed input is processed as one padded row)."""

    backend = "sdpa"

    def forward(self, x, seq_info, rope=None, cache=None, layer: int = 0, plan=None):
        if seq_info.packed and cache is None:
            from kohakuwullm_b200.ops.attention import varlen_attention_reference

            T = x.shape[0]
            q, k, v = self._project(x, rope)
            out = varlen_attention_reference(q, k, v, seq_info.cu_seqlens, self.window, self._sink_lse(),
                                             self.scale)
            return self.o_proj(out.reshape(T, self.q_dim))
        return self._forward_padded(x, seq_info, rope, cache, layer)


class MXFP8Attention(Attention):
    """Attention whose score product sees MXFP8 operands: q and k are quantised per head (e4m3, one
    power-of-two scale per 32 channels; k after subtracting its per-channel mean over the pack, which the
    softmax cannot see) before ``QK^T``; ``PV`` and every gradient product stay 16-bit, and gradients pass
    straight through the quantisation. e4m3 values times a power of two are exact in bf16, so the flash
    kernels read the dequantised operands and produce exactly the block-scaled product (fp32 accumulate);
    with head_dim 64 these kernels are bound by the softmax arithmetic, not by the tensor pipe, so an fp8
    MMA for the score tile would not make them faster. Reference:
    src/kohakuwullm/kernels/mxfp8/attention.py:30-267, attention_quant.py:17-78."""

    backend = "mxfp8"

    def forward(self, x, seq_info, rope=None, cache=None, layer: int = 0, plan=None):
        if seq_info.packed and cache is None:
            T = x.shape[0]
            q, k, v = self._project(x, rope)
            q = attn_ops.quantize_heads(q, smooth=False)
            k = attn_ops.quantize_heads(k, smooth=True)
            out = varlen_attention(q, k, v, seq_info.cu_seqlens, seq_info.max_seqlen, window=self.window,
                                   sink_lse=self._sink_lse(), scale=self.scale, plan=plan)
            return self.o_proj(out.reshape(T, self.q_dim))
        return self._forward_padded(x, seq_info, rope, cache, layer)


ATTENTION.register("flash", Attention)
ATTENTION.register("mxfp8", MXFP8Attention)
# backend names of the reference resolve to the one native implementation
for _alias in ("varlen", "triton", "native"):
    ATTENTION.register(_alias, Attention)
ATTENTION.register("sdpa", SDPAAttention)
ATTENTION.register("flex", SDPAAttention)
