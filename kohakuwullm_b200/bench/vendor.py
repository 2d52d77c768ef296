"""Vendor cross-checks on the same bytes: the block-scaled MXFP8 product through cuBLASLt (``F.scaled_mm`` with
``BlockWise1x32`` scales in the ``SWIZZLE_32_4_4`` layout) beside this library's tcgen05 kernel, and the dense
bf16 rate the card reaches in this process (the ceiling a row is judged against is measured, not carried).

The scale layout of ``ops/mxfp8`` IS the vendor swizzle: one 512-byte chunk per 128-row x 128-column tile, byte
``(r % 32) * 16 + (r / 32) * 4 + j`` inside it, chunks ordered row tile by k chunk. So the very same ``q`` and
``sf`` buffers go to both implementations, and agreement pins the scale layout, the exponent convention and
the operand byte order against an independent implementation.
Reference: verification layer 3 of docs/internals/mxfp8.md:726-772; src/kohakuwullm/bench/vendor/vendor_moe.py."""

from __future__ import annotations

import torch


def vendor_available() -> bool:
    import torch.nn.functional as F

    return hasattr(F, "scaled_mm") and hasattr(F, "ScalingType") and hasattr(torch, "float8_e8m0fnu")


def vendor_mxfp8_mm(a_q: torch.Tensor, a_sf: torch.Tensor, b_q: torch.Tensor, b_sf: torch.Tensor,
                    out_dtype=torch.bfloat16) -> torch.Tensor:
    """``A (M,K) x B (N,K)^T`` through the vendor library. M, N multiples of 128 and K of 128 (whole chunks)."""
    import torch.nn.functional as F

    a = a_q.view(torch.float8_e4m3fn)
    b = b_q.view(torch.float8_e4m3fn).t()            # (K, N) column-major, as the library wants its B
    sa = a_sf.view(torch.float8_e8m0fnu)
    sb = b_sf.view(torch.float8_e8m0fnu)
    return F.scaled_mm(a, b, sa, F.ScalingType.BlockWise1x32, sb, F.ScalingType.BlockWise1x32,
                       swizzle_a=F.SwizzleType.SWIZZLE_32_4_4, swizzle_b=F.SwizzleType.SWIZZLE_32_4_4,
                       output_dtype=out_dtype)


def compare_with_vendor(M: int = 512, N: int = 768, K: int = 1024, seed: int = 0) -> dict:
    """Own kernel vs vendor on identical bytes: share of bit-equal outputs and the largest difference in units of
    the output's last place."""
    from kohakuwullm_b200.bench.timing import ulp_error
    from kohakuwullm_b200.ops import mxfp8 as mx

    g = torch.Generator(device="cuda").manual_seed(seed)
    a = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    b = torch.randn(N, K, device="cuda", generator=g).bfloat16()
    aq, asf = mx.quantize(a)
    bq, bsf = mx.quantize(b)
    ours = mx.gemm(aq, asf, bq, bsf)
    theirs = vendor_mxfp8_mm(aq, asf, bq, bsf)
    exact = mx.dequantize(aq.view(torch.float8_e4m3fn), mx.sf_to_natural(asf, M, K)).double() @ \
        mx.dequantize(bq.view(torch.float8_e4m3fn), mx.sf_to_natural(bsf, N, K)).double().t()
    return {"bit_equal_share": float((ours == theirs).float().mean()),
            "ours_vs_vendor_max_ulp": ulp_error(ours, theirs.double())["max_ulp"],
            "ours_vs_fp64_max_ulp": ulp_error(ours, exact)["max_ulp"],
            "vendor_vs_fp64_max_ulp": ulp_error(theirs, exact)["max_ulp"]}


def dense_ceilings(n: int = 8192, repeats: int = 10) -> dict:
    """bf16 ``torch.matmul`` rate (TFLOP/s) of this card in this process."""
    from kohakuwullm_b200.bench.timing import bench_samples

    a = torch.randn(n, n, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(n, n, device="cuda", dtype=torch.bfloat16)
    ms = min(bench_samples(lambda: torch.matmul(a, b), repeats=repeats, flush=False))
    return {"bf16": 2.0 * n ** 3 / ms / 1e9}
