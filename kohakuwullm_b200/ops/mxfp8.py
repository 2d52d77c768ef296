"""MXFP8 (e4m3 + UE8M0 per-32 block scales) quantisation, block-scaled GEMM and the MXFP8 linear.

Recipe of one linear layer ``y = x W^T`` (reference: src/kohakuwullm/kernels/mxfp8/linear.py:49-126):

=========  =================================================  ==========================
product    operands                                           precision
=========  =================================================  ==========================
FPROP      ``x`` quantised along K  x  ``W`` quantised along K   MXFP8, fp32 accumulate
DGRAD      ``dy`` quantised along N x  ``W^T`` quantised along N  MXFP8, fp32 accumulate
WGRAD      ``dy^T x`` in bf16, accumulated into ``main_grad``    bf16 inputs, fp32 accumulate
=========  =================================================  ==========================

The two weight copies (``W`` along K and the transposed copy ``W^T`` along N) are cached on the
parameter and rebuilt by ``refresh_weight`` after every optimizer step. Activations are quantised on
the fly. Quantisation rule: ``exp = max(ceil(log2(amax/448)), -127)``, value ``x / 2^exp`` rounded to
e4m3 with saturation (src/kohakuwullm/kernels/mxfp8/quantize.py:39-56).

``quantize_reference`` / ``dequantize`` restate the rule in PyTorch (bit-exact oracle of the kernel);
scales are kept in the tensor-core layout described in ``csrc/mxfp8.cu`` and converted by
``sf_to_natural`` for inspection.
"""

from __future__ import annotations

import ctypes
import os

import torch

from kohakuwullm_b200.ops import native
from kohakuwullm_b200.ops.gemm import launch_wgrad, matmul

c_int, c_float = ctypes.c_int, ctypes.c_float
E4M3_MAX = 448.0


# ------------------------------------------------------------------------------------ reference
SQRT2_MANTISSA = 0x3504F3   # fraction bits of sqrt(2): a float at or above 2^E * sqrt(2) has log2 >= E + 0.5


def quantize_reference(x: torch.Tensor, exponent: str = "ceil"):
    """(M,K) -> (q float8_e4m3fn (M,K), exp uint8 (M,K/32)).

    ``exponent="ceil"`` is the rule above (the kernels' rule: the scaled block never exceeds 448, nothing
    saturates). ``"nearest"`` rounds ``log2(amax/448)`` to the nearest integer instead: half of the blocks get a
    scale one binade smaller (finer steps) and their largest elements saturate at 448. It exists for A/B runs of
    the two conventions (src/kohakuwullm/bench/vendor/mxfp8_rounding.py); no kernel uses it."""
    if exponent not in ("ceil", "nearest"):
        raise ValueError(f"unknown exponent rule {exponent!r}")
    M, K = x.shape
    xb = x.float().view(M, K // 32, 32)
    amax = xb.abs().amax(-1).clamp(min=1e-30)
    # exact from the float bits (log2 of a float can be off by one ulp near powers of two)
    bits = (amax / E4M3_MAX).view(torch.int32)
    frac = bits & 0x7FFFFF
    up = (frac != 0) if exponent == "ceil" else (frac >= SQRT2_MANTISSA)
    e = (((bits >> 23) & 0xFF) + up.to(torch.int32)).clamp(max=254)
    inv = torch.where(e >= 254, torch.full_like(e, 1), 254 - e)
    inv_scale = (inv << 23).view(torch.float32)
    q = (xb * inv_scale[..., None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).view(M, K)
    return q, e.to(torch.uint8)


def dequantize(q: torch.Tensor, e_natural: torch.Tensor) -> torch.Tensor:
    M, K = q.shape
    scale = torch.pow(2.0, e_natural.float() - 127.0)
    return (q.float().view(M, K // 32, 32) * scale[..., None]).view(M, K)


def sf_to_natural(sf: torch.Tensor, rows: int, K: int) -> torch.Tensor:
    """Tensor-core scale layout -> (rows, K/32) uint8."""
    nk = K // 128
    rt = (rows + 127) // 128
    chunks = sf.view(rt, nk, 32, 4, 4)             # [row_tile][k_chunk][r%32][r/32][k_block]
    nat = chunks.permute(0, 3, 2, 1, 4).reshape(rt * 128, nk * 4)
    return nat[:rows].contiguous()


# ------------------------------------------------------------------------------------ native ops
def sf_bytes(rows: int, K: int) -> int:
    return ((rows + 127) // 128) * (K // 128) * 512


def quantize(x: torch.Tensor, out_q: torch.Tensor | None = None, out_sf: torch.Tensor | None = None):
    """bf16 (M,K) -> (q uint8 (M,K), sf uint8 chunks); blocks along K."""
    L = native.require()
    M, K = x.shape
    q = out_q if out_q is not None else torch.empty(M, K, dtype=torch.uint8, device=x.device)
    sf = out_sf if out_sf is not None else torch.empty(sf_bytes(M, K), dtype=torch.uint8, device=x.device)
    rc = L.kwu_mxfp8_quantize(native.ptr(x), c_int(x.stride(0)), native.ptr(q), c_int(q.stride(0)),
                              native.ptr(sf), c_int(M), c_int(K), native.stream_ptr())
    native.check(rc, "mxfp8_quantize")
    return q, sf


def quantize_transposed(x: torch.Tensor, out_q=None, out_sf=None):
    """bf16 (R,C) -> (qT uint8 (C,R), sf chunks of a (C,R) operand); blocks along R."""
    L = native.require()
    R, C = x.shape
    q = out_q if out_q is not None else torch.empty(C, R, dtype=torch.uint8, device=x.device)
    sf = out_sf if out_sf is not None else torch.empty(sf_bytes(C, R), dtype=torch.uint8, device=x.device)
    rc = L.kwu_mxfp8_quantize_t(native.ptr(x), c_int(x.stride(0)), native.ptr(q), c_int(q.stride(0)),
                                native.ptr(sf), c_int(R), c_int(C), native.stream_ptr())
    native.check(rc, "mxfp8_quantize_t")
    return q, sf


def gemm(a_q, a_sf, b_q, b_sf, out=None, out_dtype=torch.bfloat16, accumulate=False, alpha=1.0, bn: int = 0):
    """``out (+)= alpha * A B^T`` with A (M,K), B (N,K) both e4m3 with per-32 scales along K. ``bn``: width of
    the output tiles; a value above 128 says that ``b_sf`` is in the tile-local layout for that width (made by
    ``quantize_weight`` / ``quantize_weight_transposed``), 0 or 128 the plain layout."""
    L = native.require()
    M, K = a_q.shape
    N = b_q.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=a_q.device)
    rc = L.kwu_gemm_mxfp8(native.ptr(a_q), native.ptr(a_sf), native.ptr(b_q), native.ptr(b_sf), native.ptr(out),
                          c_int(M), c_int(N), c_int(K), c_int(a_q.stride(0)), c_int(b_q.stride(0)),
                          c_int(out.stride(0)), c_int(int(out.dtype == torch.float32)), c_int(int(accumulate)),
                          c_float(alpha), c_int(bn), native.stream_ptr(), native.ptr(native.status_word()))
    native.check(rc, "gemm_mxfp8")
    return out


# ------------------------------------------------------------------------------------ weights: tile width
TILE_WIDTHS = (128, 144, 160, 176, 192, 208, 224, 240)


def pick_tile_width(n_cols: int, m_rows: int = 4096, sms: int = 148) -> int:
    """Width of the output tiles of ``A (m_rows, K) x W (n_cols, K)^T`` that minimises rounds x cost per round.

    The block-scaled GEMM is bound by shared-memory traffic: per 128-deep k-block a 128 x BN tile moves
    16 KB + BN * 128 B, so a round of tiles costs ``16 + BN / 8`` units whatever it computes, and a problem
    takes ``ceil(tiles / SMs)`` rounds. A wider tile is cheaper per column, and the right width fills whole
    waves (4096 x 1280: 320 tiles of 128 are 3 rounds, 288 tiles of 144 are 2). ``KWU_MX_BN`` forces a width."""
    forced = os.environ.get("KWU_MX_BN")
    if forced:
        return int(forced)
    tiles_m = max((m_rows + 127) // 128, 1)
    best, best_bn = None, 128
    for bn in TILE_WIDTHS:
        rounds = -(-(tiles_m * -(-n_cols // bn)) // sms)
        cost = rounds * (16 + bn / 8)
        if best is None or cost < best - 1e-9:
            best, best_bn = cost, bn
    return best_bn


_TUNED: dict[tuple[int, int, int, int], int] = {}


def tuned_tile_width(m_rows: int, n_cols: int, K: int, device) -> int:
    """Tile width for ``A (m_rows, K) x W (n_cols, K)^T``, MEASURED once per problem shape on this device: every
    supported width runs the real kernel on synthetic operands (10 back-to-back launches between two events,
    best of three) and the fastest wins; the result is cached. The analytic pick above ranks the widths by
    shared-memory traffic and wave count only and misses the fixed costs of a tile (pipeline fill, epilogue),
    which decide between near-equal candidates at short contraction lengths. Falls back to the analytic pick
    under stream capture, without a GPU, and unless ``KWU_MX_AUTOTUNE=1`` asks for the measurement (on the
    dense training shapes both picks gave the same step time). Every width gives bit-identical results, so
    ranks that pick differently still agree."""
    if os.environ.get("KWU_MX_BN"):
        return int(os.environ["KWU_MX_BN"])
    dev = torch.device(device)
    key = (dev.index or 0, m_rows, n_cols, K)
    if key in _TUNED:
        return _TUNED[key]
    if (os.environ.get("KWU_MX_AUTOTUNE", "0") != "1" or dev.type != "cuda" or not native.available()
            or torch.cuda.is_current_stream_capturing() or m_rows <= 0):
        return pick_tile_width(n_cols, m_rows)
    a_q = torch.randint(0, 120, (m_rows, K), dtype=torch.uint8, device=dev)
    a_sf = torch.full((sf_bytes(m_rows, K),), 127, dtype=torch.uint8, device=dev)
    b_q = torch.randint(0, 120, (n_cols, K), dtype=torch.uint8, device=dev)
    out = torch.empty(m_rows, n_cols, dtype=torch.bfloat16, device=dev)
    best_ms, best_bn = None, 128
    for bn in TILE_WIDTHS:
        b_sf = alloc_weight_sf(n_cols, K, bn, dev)
        run = lambda: gemm(a_q, a_sf, b_q, b_sf, out=out, bn=bn)  # noqa: E731
        run()
        run()
        samples = []
        for _ in range(3):
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record()
            for _ in range(10):
                run()
            s1.record()
            s1.synchronize()
            samples.append(s0.elapsed_time(s1) / 10)
        ms = min(samples)
        if best_ms is None or ms < best_ms * 0.99:   # a wider tile must win by more than timing noise
            best_ms, best_bn = ms, bn
    _TUNED[key] = best_bn
    return best_bn


def sf_bytes_tiled(rows: int, K: int, bn: int) -> int:
    if bn <= 128:
        return sf_bytes(rows, K)
    return -(-rows // bn) * (K // 128) * 1024


def alloc_weight_sf(rows: int, K: int, bn: int, device) -> torch.Tensor:
    """Scale buffer of a weight for tile width ``bn``; padding rows hold the neutral scale 2^0."""
    return torch.full((sf_bytes_tiled(rows, K, bn),), 127, dtype=torch.uint8, device=device)


def quantize_weight(w: torch.Tensor, out_q: torch.Tensor, out_sf: torch.Tensor, bn: int):
    """bf16 (N,K) -> e4m3 (N,K) + scales along K in the layout for ``bn``-wide tiles."""
    L = native.require()
    N, K = w.shape
    rc = L.kwu_mxfp8_quantize_w(native.ptr(w), c_int(w.stride(0)), native.ptr(out_q), c_int(out_q.stride(0)),
                                native.ptr(out_sf), c_int(N), c_int(K), c_int(bn), native.stream_ptr())
    native.check(rc, "mxfp8_quantize_w")
    return out_q, out_sf


def quantize_weight_transposed(w: torch.Tensor, out_q: torch.Tensor, out_sf: torch.Tensor, bn: int):
    """bf16 (R,C) -> e4m3 (C,R) + scales along R in the layout for ``bn``-wide tiles of the (C,R) operand."""
    L = native.require()
    R, C = w.shape
    rc = L.kwu_mxfp8_quantize_t_w(native.ptr(w), c_int(w.stride(0)), native.ptr(out_q), c_int(out_q.stride(0)),
                                  native.ptr(out_sf), c_int(R), c_int(C), c_int(bn), native.stream_ptr())
    native.check(rc, "mxfp8_quantize_t_w")
    return out_q, out_sf


# ------------------------------------------------------------------------------------ producer-made copies
# A producer kernel (RMSNorm, SwiGLU, their backward passes) can write the fp8 copy of its output in the same
# pass. It registers the copy here under the output's address; the MXFP8 linear that consumes the tensor takes
# it instead of running the quantise kernel. Entries are single-use, are only made when the model wiring says
# that the consumer is an MXFP8 linear, and are dropped at the start of every model forward.
_PREQUANTIZED: dict[int, tuple] = {}


def alloc_quantized(rows: int, cols: int, device):
    return (torch.empty(rows, cols, dtype=torch.uint8, device=device),
            torch.empty(sf_bytes(rows, cols), dtype=torch.uint8, device=device))


def can_emit(rows: int, cols: int) -> bool:
    return rows > 0 and rows % 128 == 0 and cols % 128 == 0


def stash_quantized(t: torch.Tensor, q: torch.Tensor, sf: torch.Tensor) -> None:
    _PREQUANTIZED[t.data_ptr()] = (q, sf, t.numel(), q.shape)


def take_quantized(t: torch.Tensor):
    """The producer-made fp8 copy of ``t`` (2-D, contiguous), or None."""
    entry = _PREQUANTIZED.pop(t.data_ptr(), None)
    if entry is None:
        return None
    q, sf, numel, shape = entry
    if numel != t.numel() or tuple(shape) != tuple(t.shape):
        return None
    return q, sf


def clear_prequantized() -> None:
    _PREQUANTIZED.clear()


# ------------------------------------------------------------------------------------ linear
class QuantizedWeight:
    """The two MXFP8 copies of one weight matrix (N,K): ``W`` along K (the B operand of FPROP, N output
    columns) and ``W^T`` along N (the B operand of DGRAD, K output columns). Each copy's scales are laid out for
    the tile width picked for its product (``rows_hint`` = the activation row count the layer runs at)."""

    def __init__(self, weight: torch.Tensor, rows_hint: int = 4096):
        N, K = weight.shape
        dev = weight.device
        self.bn = tuned_tile_width(rows_hint, N, K, dev)       # FPROP: x (rows, K) x W (N, K)^T
        self.bn_t = tuned_tile_width(rows_hint, K, N, dev)     # DGRAD: dy (rows, N) x W^T (K, N)^T
        self.q = torch.empty(N, K, dtype=torch.uint8, device=dev)
        self.sf = alloc_weight_sf(N, K, self.bn, dev)
        self.qt = torch.empty(K, N, dtype=torch.uint8, device=dev)
        self.sft = alloc_weight_sf(K, N, self.bn_t, dev)
        self.refresh(weight)

    @torch.no_grad()
    def refresh(self, weight: torch.Tensor) -> None:
        quantize_weight(weight, self.q, self.sf, self.bn)
        quantize_weight_transposed(weight, self.qt, self.sft, self.bn_t)


class _MXFP8Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, qw: QuantizedWeight):
        xq, xsf = take_quantized(x) or quantize(x)
        y = gemm(xq, xsf, qw.q, qw.sf, out_dtype=x.dtype, bn=qw.bn)
        ctx.save_for_backward(x, w)
        ctx.qw = qw
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        qw = ctx.qw
        dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dyq, dysf = take_quantized(dy) or quantize(dy)
            dx = gemm(dyq, dysf, qw.qt, qw.sft, out_dtype=x.dtype, bn=qw.bn_t)
        if ctx.needs_input_grad[1]:
            main_grad = getattr(w, "main_grad", None)
            if main_grad is not None:
                launch_wgrad(lambda: matmul(dy, x, a_mn=True, b_mn=True, out=main_grad, accumulate=True), dy, x)
            else:
                dw = matmul(dy, x, a_mn=True, b_mn=True, out_dtype=w.dtype)
        return dx, dw, None


def supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    """MXFP8 needs bf16 CUDA operands with both feature dimensions multiples of 128."""
    return (native.available() and x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and w.shape[0] % 128 == 0 and w.shape[1] % 128 == 0)


def mxfp8_linear(x: torch.Tensor, w: torch.Tensor, qw: QuantizedWeight) -> torch.Tensor:
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    return _MXFP8Linear.apply(x2, w, qw).reshape(*lead, w.shape[0])


def mxfp8_linear_reference(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """Quantise-dequantise emulation of the forward product in fp32 (oracle for tests and CPU)."""
    xq, xe = quantize_reference(x.reshape(-1, x.shape[-1]))
    wq, we = quantize_reference(w)
    y = dequantize(xq, xe) @ dequantize(wq, we).t()
    return y.to(x.dtype).reshape(*x.shape[:-1], w.shape[0])


# ------------------------------------------------------------------------------------ grouped (experts)
class GroupedQuantizedWeight:
    """MXFP8 copies of a stacked expert weight (E, N, K): ``W[e]`` along K, stacked as (E*N, K), and
    ``W[e]^T`` along N, stacked as (E*K, N). N and K are multiples of 128, so every expert's block of
    rows starts on a scale-chunk boundary."""

    def __init__(self, weight: torch.Tensor):
        E, N, K = weight.shape
        dev = weight.device
        self.shape = (E, N, K)
        self.q = torch.empty(E * N, K, dtype=torch.uint8, device=dev)
        self.sf = torch.empty(sf_bytes(E * N, K), dtype=torch.uint8, device=dev)
        self.qt = torch.empty(E * K, N, dtype=torch.uint8, device=dev)
        self.sft = torch.empty(E * sf_bytes(K, N), dtype=torch.uint8, device=dev)
        self.refresh(weight)

    @torch.no_grad()
    def refresh(self, weight: torch.Tensor) -> None:
        L = native.require()
        E, N, K = self.shape
        w2 = weight.detach().reshape(E * N, K)
        quantize(w2, self.q, self.sf)
        rc = L.kwu_mxfp8_quantize_t_batched(native.ptr(w2), c_int(K), native.ptr(self.qt), c_int(N),
                                            native.ptr(self.sft), c_int(N), c_int(K), c_int(E), native.stream_ptr())
        native.check(rc, "mxfp8_quantize_t_batched")


def grouped_gemm(a_q, a_sf, b_q, b_sf, n_per_expert: int, n_experts: int, tiles: torch.Tensor, out_dtype=torch.bfloat16,
                 out=None, row_ptrs=None):
    """``out[rows of expert e] = A[rows] B[e]^T`` over expert-sorted, 128-row-aligned A rows."""
    L = native.require()
    M, K = a_q.shape
    if out is None:
        out = torch.empty(M, n_per_expert, dtype=out_dtype, device=a_q.device)
    rc = L.kwu_gemm_mxfp8_grouped(native.ptr(a_q), native.ptr(a_sf), native.ptr(b_q), native.ptr(b_sf), native.ptr(out),
                                  c_int(M), c_int(n_per_expert), c_int(K), c_int(a_q.stride(0)), c_int(b_q.stride(0)),
                                  c_int(out.stride(0)), c_int(n_experts), native.ptr(tiles), c_int(tiles.shape[0]),
                                  native.ptr(row_ptrs), native.stream_ptr(), native.ptr(native.status_word()))
    native.check(rc, "gemm_mxfp8_grouped")
    return out


class _MXFP8GroupedLinear(torch.autograd.Function):
    """Grouped expert linear in the MXFP8 recipe: FPROP and DGRAD block-scaled fp8, WGRAD bf16 into fp32
    (``main_grad`` when the trainer provides it). ``plan`` carries the tile table and expert offsets."""

    @staticmethod
    def forward(ctx, rows, W, qw: GroupedQuantizedWeight, plan, out=None, dgrad_out=None, out_row_ptrs=None,
                dgrad_row_ptrs=None):
        E, N, K = W.shape
        xq, xsf = take_quantized(rows) or quantize(rows)
        out = grouped_gemm(xq, xsf, qw.q, qw.sf, N, E, plan.tiles, out_dtype=rows.dtype, out=out, row_ptrs=out_row_ptrs)
        ctx.save_for_backward(rows, W)
        ctx.qw, ctx.plan, ctx.dgrad_out, ctx.dgrad_row_ptrs = qw, plan, dgrad_out, dgrad_row_ptrs
        return out

    @staticmethod
    def backward(ctx, dout):
        L = native.require()
        rows, W = ctx.saved_tensors
        qw, plan = ctx.qw, ctx.plan
        E, N, K = W.shape
        dout = dout.contiguous()
        drows = dW = None
        if ctx.needs_input_grad[0]:
            dq, dsf = take_quantized(dout) or quantize(dout)
            drows = grouped_gemm(dq, dsf, qw.qt, qw.sft, K, E, plan.tiles, out_dtype=rows.dtype, out=ctx.dgrad_out,
                                 row_ptrs=ctx.dgrad_row_ptrs)
        if ctx.needs_input_grad[1]:
            main_grad = getattr(W, "main_grad", None)
            target = main_grad if main_grad is not None else torch.zeros(E, N, K, dtype=torch.float32, device=W.device)
            rc = L.kwu_gemm_bf16_grouped_wgrad(native.ptr(dout), native.ptr(rows), native.ptr(target),
                                               c_int(plan.max_rows), c_int(N), c_int(K), c_int(dout.stride(0)),
                                               c_int(rows.stride(0)), c_int(E), native.ptr(plan.offsets), c_int(1),
                                               c_int(1), native.stream_ptr(), native.ptr(native.status_word()))
            native.check(rc, "grouped_gemm_wgrad")
            if main_grad is None:
                dW = target.to(W.dtype)
        return drows, dW, None, None, None, None, None, None


def grouped_supported(W: torch.Tensor) -> bool:
    return (native.available() and W.is_cuda and W.dtype == torch.bfloat16 and W.dim() == 3
            and W.shape[1] % 128 == 0 and W.shape[2] % 128 == 0)
