"""Bindings of the 16-bit optimizer / stochastic-rounding kernels plus their PyTorch references.
``stochastic_round_reference`` takes the 16-bit draws explicitly, so the kernel (given the same draws)
can be checked bit for bit. Reference: src/kohakuwullm/kernels/optim/stochastic_round.py:241-270."""

from __future__ import annotations

import ctypes

import torch

from kohakuwullm_b200.ops import native

c_ll, c_ull, c_float, c_int = ctypes.c_longlong, ctypes.c_ulonglong, ctypes.c_float, ctypes.c_int


def stochastic_round_reference(x: torch.Tensor, draws: torch.Tensor) -> torch.Tensor:
    """fp32 -> bf16: add the 16-bit draw to the bits that bf16 discards, truncate."""
    bits = x.float().contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    finite = (bits & 0x7F800000) != 0x7F800000
    bits = torch.where(finite, (bits + draws.to(torch.int64)) & 0xFFFFFFFF, bits)
    hi = (bits >> 16).to(torch.int32).to(torch.int16)
    return hi.view(torch.bfloat16)


def _use_native(t: torch.Tensor) -> bool:
    return t.is_cuda and native.available()


def sr_cast(x: torch.Tensor, seed: int = 0, offset: int = 0, draws: torch.Tensor | None = None) -> torch.Tensor:
    out = torch.empty_like(x, dtype=torch.bfloat16)
    if _use_native(x):
        rc = native.require().kwu_sr_cast(native.ptr(x), native.ptr(out), c_ll(x.numel()), c_ull(seed), c_ull(offset),
                                          native.ptr(draws), native.stream_ptr())
        native.check(rc, "sr_cast")
        return out
    if draws is None:
        g = torch.Generator().manual_seed(seed + offset)
        draws = torch.randint(0, 1 << 16, x.shape, generator=g)
    return stochastic_round_reference(x, draws.reshape(x.shape))


def sr_update_(p: torch.Tensor, u: torch.Tensor, decay: float, alpha: float, seed: int = 0, offset: int = 0,
               draws: torch.Tensor | None = None) -> None:
    """``p = SR(p * (1 - decay) + alpha * u)`` in place (p bf16, u fp32)."""
    if _use_native(p):
        rc = native.require().kwu_sr_update(native.ptr(p), native.ptr(u), c_ll(p.numel()), c_float(decay), c_float(alpha),
                                            c_ull(seed), c_ull(offset), native.ptr(draws), native.stream_ptr())
        native.check(rc, "sr_update")
        return
    v = p.float() * (1 - decay) + alpha * u.float()
    if draws is None:
        g = torch.Generator().manual_seed(seed + offset)
        draws = torch.randint(0, 1 << 16, p.shape, generator=g)
    p.copy_(stochastic_round_reference(v, draws.reshape(p.shape)))


class GroupedWriteback:
    """One launch for the stochastic write-back of a whole model (chunk table of raw pointers).
    Element ``i`` of tensor ``t`` uses random number ``sum(numel of tensors before t) + i``, exactly what a
    per-tensor loop with the same running offset uses, so both give identical bits."""

    def __init__(self, params: list[torch.Tensor], updates: list[torch.Tensor]):
        import struct

        self.params, self.updates = params, updates
        L = native.require()
        rec = L.kwu_sr_chunk_bytes()
        self._fmt = "<QQqQff"
        assert struct.calcsize(self._fmt) == rec, (struct.calcsize(self._fmt), rec)
        self._struct = struct
        self.table = torch.empty(len(params) * rec, dtype=torch.uint8, device=params[0].device)

    def step(self, decays: list[float], alphas: list[float], seed: int) -> None:
        blob, offset = b"", 0
        for p, u, d, a in zip(self.params, self.updates, decays, alphas):
            blob += self._struct.pack(self._fmt, p.data_ptr(), u.data_ptr(), p.numel(), offset, d, a)
            offset += p.numel()
        self.table.copy_(torch.frombuffer(bytearray(blob), dtype=torch.uint8), non_blocking=True)
        rc = native.require().kwu_sr_grouped(native.ptr(self.table), c_int(len(self.params)), c_ull(seed), native.stream_ptr())
        native.check(rc, "sr_grouped")


def adamw16_step_(p, m, sv, g, *, lr, betas, eps, wd, step, grad_scale=1.0, stochastic=False, seed=0, offset=0):
    """AdamW with p, m and sqrt(v) in bf16 (fp32 math). ``g`` may be bf16 or fp32."""
    if _use_native(p) and p.dtype == torch.bfloat16:
        g16 = g if g.dtype == torch.bfloat16 else None
        g32 = g if g.dtype == torch.float32 else None
        rc = native.require().kwu_adamw16(native.ptr(p), native.ptr(m), native.ptr(sv), native.ptr(g16), native.ptr(g32),
                                          c_ll(p.numel()), c_float(lr), c_float(betas[0]), c_float(betas[1]), c_float(eps),
                                          c_float(wd), c_int(step), c_float(grad_scale), c_int(int(stochastic)), c_ull(seed),
                                          c_ull(offset), native.stream_ptr())
        native.check(rc, "adamw16")
        return
    # eager twin (CPU / other dtypes)
    gf = g.float() * grad_scale
    mf = m.float().mul(betas[0]).add(gf, alpha=1 - betas[0])
    vf = sv.float().pow(2).mul(betas[1]).addcmul(gf, gf, value=1 - betas[1])
    root = vf.sqrt()
    bc1, bc2 = 1 - betas[0] ** step, 1 - betas[1] ** step
    pf = p.float() * (1 - lr * wd) - lr * (mf / bc1) / (root / bc2 ** 0.5 + eps)
    p.copy_(pf.to(p.dtype))
    m.copy_(mf.to(m.dtype))
    sv.copy_(root.to(sv.dtype))
