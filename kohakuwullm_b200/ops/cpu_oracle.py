"""ctypes binding of the C++ CPU oracles (``csrc/cpu/oracle.cpp`` -> ``_kwu_cpu.so``).

Each function takes and returns CPU fp32 (or integer) tensors and restates one kernel family's rule in
plain loops; tests compare the CUDA kernels AND the PyTorch references against it. The library is built
on first use when missing (host compiler only, no GPU toolchain needed).
"""

from __future__ import annotations

import ctypes
from pathlib import Path

import torch

_PKG = Path(__file__).resolve().parent.parent
_lib = None
c_int, c_float, c_ll = ctypes.c_int, ctypes.c_float, ctypes.c_longlong


def lib():
    global _lib
    if _lib is None:
        path = _PKG / "_kwu_cpu.so"
        if not path.exists():
            from kohakuwullm_b200.build import build_cpu

            build_cpu()
        _lib = ctypes.CDLL(str(path))
        _lib.kwo_bf16_round.restype = ctypes.c_float
        _lib.kwo_bf16_round.argtypes = [ctypes.c_float]
        _lib.kwo_e4m3_to_float.restype = ctypes.c_float
        _lib.kwo_e4m3_to_float.argtypes = [ctypes.c_ubyte]
        _lib.kwo_e4m3_from_float.restype = ctypes.c_ubyte
        _lib.kwo_e4m3_from_float.argtypes = [ctypes.c_float]
        _lib.kwo_draw16.restype = ctypes.c_uint
        _lib.kwo_draw16.argtypes = [ctypes.c_ulonglong, ctypes.c_ulonglong]
    return _lib


def _p(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _f(t):
    return None if t is None else t.detach().to("cpu", torch.float32).contiguous()


def rmsnorm_fwd(x, w=None, eps=1e-6, one_plus=False):
    x, w = _f(x), _f(w)
    out = torch.empty_like(x)
    lib().kwo_rmsnorm_fwd(_p(x), _p(w), _p(out), _p(None), c_int(x.shape[0]), c_int(x.shape[1]), c_float(eps),
                          c_int(int(one_plus)))
    return out


def rmsnorm_bwd(x, w, dy, eps=1e-6, one_plus=False):
    x, w, dy = _f(x), _f(w), _f(dy)
    dx = torch.empty_like(x)
    dw = torch.empty(x.shape[1]) if w is not None else None
    lib().kwo_rmsnorm_bwd(_p(x), _p(w), _p(dy), _p(dx), _p(dw), c_int(x.shape[0]), c_int(x.shape[1]), c_float(eps),
                          c_int(int(one_plus)))
    return dx, dw


def swiglu_fwd(h):
    h = _f(h)
    H = h.shape[1] // 2
    out = torch.empty(h.shape[0], H)
    lib().kwo_swiglu_fwd(_p(h), _p(out), c_int(h.shape[0]), c_int(H))
    return out


def swiglu_bwd(h, dout):
    h, dout = _f(h), _f(dout)
    dh = torch.empty_like(h)
    lib().kwo_swiglu_bwd(_p(h), _p(dout), _p(dh), c_int(h.shape[0]), c_int(h.shape[1] // 2))
    return dh


def rope(x, cos, sin, inverse=False):
    x, cos, sin = _f(x), _f(cos), _f(sin)
    T, H, D = x.shape
    out = torch.empty_like(x)
    lib().kwo_rope(_p(x), _p(cos), _p(sin), _p(out), c_int(T), c_int(H), c_int(D), c_int(cos.shape[1]),
                   c_float(-1.0 if inverse else 1.0))
    return out


def attention_varlen(q, k, v, cu_seqlens, window=None, sink_lse=None, scale=None):
    q, k, v, sink_lse = _f(q), _f(k), _f(v), _f(sink_lse)
    T, Hq, D = q.shape
    cu = cu_seqlens.detach().to("cpu", torch.int32).contiguous()
    out = torch.zeros_like(q)
    lse = torch.zeros(Hq, T)
    lib().kwo_attention_varlen(_p(q), _p(k), _p(v), _p(cu), c_int(cu.numel() - 1), c_int(T), c_int(Hq),
                               c_int(k.shape[1]), c_int(D), c_int(int(window or 0)), _p(sink_lse),
                               c_float(scale if scale is not None else D ** -0.5), _p(out), _p(lse))
    return out, lse


def mxfp8_quantize(x):
    """(M,K) -> (e4m3 bytes uint8 (M,K), exponent bytes uint8 (M,K/32), dequantised fp32 (M,K))."""
    x = _f(x)
    M, K = x.shape
    q = torch.empty(M, K, dtype=torch.uint8)
    e8 = torch.empty(M, K // 32, dtype=torch.uint8)
    deq = torch.empty(M, K)
    lib().kwo_mxfp8_quantize(_p(x), _p(q), _p(e8), _p(deq), c_int(M), c_int(K))
    return q, e8, deq


def linear_ce(x, W, labels):
    x, W = _f(x), _f(W)
    labels = labels.detach().to("cpu", torch.int64).contiguous()
    T = x.shape[0]
    ce, lse = torch.empty(T), torch.empty(T)
    lib().kwo_linear_ce(_p(x), _p(W), _p(labels), _p(ce), _p(lse), c_int(T), c_int(x.shape[1]), c_int(W.shape[0]))
    return ce, lse


SCORE_IDS = {"sigmoid": 0, "softmax": 1, "sqrtsoftplus": 2}


def router_topk(x, Wg, bias, k, score="sigmoid", norm_topk=True, scaling=1.0):
    x, Wg, bias = _f(x), _f(Wg), _f(bias)
    T, E = x.shape[0], Wg.shape[0]
    idx = torch.empty(T, k, dtype=torch.int32)
    w = torch.empty(T, k)
    counts = torch.empty(E, dtype=torch.int32)
    lib().kwo_router_topk(_p(x), _p(Wg), _p(bias), _p(idx), _p(w), _p(counts), c_int(T), c_int(x.shape[1]), c_int(E),
                          c_int(k), c_int(SCORE_IDS[score]), c_int(int(norm_topk)), c_float(scaling))
    return idx, w, counts


def routed_experts(x, idx, weight, w_in, w_out):
    x, weight, w_in, w_out = _f(x), _f(weight), _f(w_in), _f(w_out)
    idx = idx.detach().to("cpu", torch.int32).contiguous()
    T, D = x.shape
    E, H = w_out.shape[0], w_out.shape[2]
    y = torch.empty(T, D)
    lib().kwo_routed_experts(_p(x), _p(idx), _p(weight), _p(w_in), _p(w_out), _p(y), c_int(T), c_int(D), c_int(H),
                             c_int(E), c_int(idx.shape[1]))
    return y


def adamw(p, m, v, g, grad_scale, lr, beta1, beta2, eps, wd, step):
    """In place on CPU fp32 tensors p, m, v."""
    lib().kwo_adamw(_p(p), _p(m), _p(v), _p(_f(g)), c_ll(p.numel()), c_float(grad_scale), c_float(lr), c_float(beta1),
                    c_float(beta2), c_float(eps), c_float(wd), c_int(step))


def sr_round(x, bits16):
    x = _f(x)
    bits = bits16.detach().to("cpu", torch.int64).to(torch.int32).contiguous()
    out = torch.empty_like(x)
    lib().kwo_sr_round(_p(x), _p(bits), _p(out), c_ll(x.numel()))
    return out


def draw16(seed: int, i: int) -> int:
    return int(lib().kwo_draw16(seed, i))
