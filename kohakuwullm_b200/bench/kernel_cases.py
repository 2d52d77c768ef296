"""Per-kernel micro-benchmarks with roofline fractions against the measured peaks of this machine.

    python -m kohakuwullm_b200.bench.kernel_cases                 # all cases, one JSON line each
    python -m kohakuwullm_b200.bench.kernel_cases --only flash    # a single family (used under ncu)

Every case is timed with CUDA events on the launching stream after warm-up, with an L2 flush before each
sample (``bench_samples``). FLOP / byte counts are the algorithmic ones. Shapes are those of the dense
546M benchmark config (4096-token packs, d 1280, FFN 3584, 20/4 heads of 64, vocab 65536).
"""

from __future__ import annotations

import argparse
import json
import statistics

import torch

from kohakuwullm_b200.bench.timing import bench_samples, module_metrics


def _report(name, samples, **kw):
    ms = statistics.median(samples)
    out = {"case": name, **module_metrics(ms, **kw)}
    print(json.dumps(out), flush=True)


def case_gemm(reps):
    from kohakuwullm_b200.ops.gemm import matmul

    for (M, N, K, amn, bmn, tag) in [(8192, 8192, 8192, False, False, "square"), (4096, 1792, 1280, False, False, "qkv_fwd"),
                                     (4096, 7168, 1280, False, False, "w_in_fwd"), (4096, 1280, 3584, False, False, "w_out_fwd"),
                                     (4096, 1280, 7168, False, True, "w_in_dgrad"), (7168, 1280, 4096, True, True, "w_in_wgrad")]:
        a = torch.randn((K, M) if amn else (M, K), device="cuda").to(torch.bfloat16)
        b = torch.randn((K, N) if bmn else (N, K), device="cuda").to(torch.bfloat16)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        s = bench_samples(lambda: matmul(a, b, a_mn=amn, b_mn=bmn, out=out), repeats=reps)
        _report(f"gemm_bf16/{tag}_{M}x{N}x{K}", s, flops=2.0 * M * N * K, bytes_moved=2.0 * (M * K + N * K + M * N))


def case_wgrad(reps):
    """Weight-gradient products the way a training step runs them: both operands token-major, fp32 ``C +=``."""
    from kohakuwullm_b200.ops.gemm import matmul

    K = 4096
    for (M, N, tag) in [(1792, 1280, "qkv"), (1280, 1280, "wo"), (7168, 1280, "w_in"), (1280, 3584, "w_out")]:
        a = torch.randn(K, M, device="cuda").to(torch.bfloat16)
        b = torch.randn(K, N, device="cuda").to(torch.bfloat16)
        out = torch.zeros(M, N, device="cuda", dtype=torch.float32)
        s = bench_samples(lambda: matmul(a, b, a_mn=True, b_mn=True, out=out, accumulate=True), repeats=reps)
        _report(f"wgrad_fp32_accumulate/{tag}_{M}x{N}x{K}", s, flops=2.0 * M * N * K,
                bytes_moved=2.0 * K * (M + N) + 8.0 * M * N)


def case_mxfp8(reps):
    from kohakuwullm_b200.ops import mxfp8 as mx

    for (M, N, K, tag) in [(8192, 8192, 8192, "square"), (4096, 1792, 1280, "qkv_fwd"), (4096, 7168, 1280, "w_in_fwd"),
                           (4096, 1280, 3584, "w_out_fwd"), (4096, 1280, 7168, "w_in_dgrad"), (4096, 1280, 1280, "o_fwd")]:
        a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        b = torch.randn(N, K, device="cuda").to(torch.bfloat16)
        aq, asf = mx.quantize(a)
        bq, bsf = mx.quantize(b)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        s = bench_samples(lambda: mx.gemm(aq, asf, bq, bsf, out=out), repeats=reps)
        _report(f"gemm_mxfp8/{tag}_{M}x{N}x{K}", s, flops=2.0 * M * N * K, bytes_moved=1.0 * (M * K + N * K) + 2.0 * M * N)
        # the same product as a linear layer runs it: weight scales laid out for the tile width picked for (M, N)
        bn = mx.pick_tile_width(N, M)
        if bn != 128:
            q2 = torch.empty(N, K, dtype=torch.uint8, device="cuda")
            sf2 = mx.alloc_weight_sf(N, K, bn, "cuda")
            mx.quantize_weight(b, q2, sf2, bn)
            s = bench_samples(lambda: mx.gemm(aq, asf, q2, sf2, out=out, bn=bn), repeats=reps)
            _report(f"gemm_mxfp8_w{bn}/{tag}_{M}x{N}x{K}", s, flops=2.0 * M * N * K,
                    bytes_moved=1.0 * (M * K + N * K) + 2.0 * M * N)
    x = torch.randn(16384, 3584, device="cuda").to(torch.bfloat16)
    q = torch.empty(16384, 3584, dtype=torch.uint8, device="cuda")
    sf = torch.empty(mx.sf_bytes(16384, 3584), dtype=torch.uint8, device="cuda")
    s = bench_samples(lambda: mx.quantize(x, q, sf), repeats=reps)
    _report("mxfp8_quantize/16384x3584", s, bytes_moved=x.numel() * 3.0 + sf.numel())
    w = torch.randn(7168, 1280, device="cuda").to(torch.bfloat16)
    s = bench_samples(lambda: mx.quantize_transposed(w), repeats=reps)
    _report("mxfp8_quantize_t/7168x1280", s, bytes_moved=w.numel() * 3.0)


def case_flash(reps):
    from kohakuwullm_b200.models.flops import attention_pairs
    from kohakuwullm_b200.models.seqinfo import SeqInfo
    from kohakuwullm_b200.ops.attention import attention_plan, varlen_attention

    for lengths, window, tag in [([2500, 1596], None, "causal_4096"), ([16384], 1024, "window1024_16384"), ([16384], None, "causal_16384")]:
        info = SeqInfo.from_lengths(lengths, device="cuda")
        T, Hq, Hkv = info.total_tokens, 20, 4
        q = torch.randn(T, Hq, 64, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        k = torch.randn(T, Hkv, 64, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        v = torch.randn(T, Hkv, 64, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        do = torch.randn(T, Hq, 64, device="cuda", dtype=torch.bfloat16)
        plan = attention_plan(info.cu_seqlens, T)
        pairs = sum(attention_pairs(n, window) for n in lengths)
        fwd_flops = 4.0 * Hq * 64 * pairs
        with torch.no_grad():
            s = bench_samples(lambda: varlen_attention(q, k, v, info.cu_seqlens, window=window, plan=plan), repeats=reps)
        _report(f"flash_fwd/{tag}", s, flops=fwd_flops)
        out = varlen_attention(q, k, v, info.cu_seqlens, window=window, plan=plan)

        def bwd():
            q.grad = k.grad = v.grad = None
            out.backward(do, retain_graph=True)

        s = bench_samples(bwd, repeats=reps)
        _report(f"flash_bwd/{tag}", s, flops=2.5 * fwd_flops)


def case_elementwise(reps):
    from kohakuwullm_b200.ops.elementwise import qknorm_rope, rmsnorm, swiglu

    rows, cols = 32768, 1280
    x = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    res = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(cols, device="cuda", requires_grad=True)
    with torch.no_grad():
        s = bench_samples(lambda: rmsnorm(x, w, residual=res), repeats=reps)
    _report(f"rmsnorm_add_fwd/{rows}x{cols}", s, bytes_moved=rows * cols * 2.0 * 4)
    y, h = rmsnorm(x, w, residual=res)
    dy = torch.randn_like(y)

    def bwd():
        x.grad = w.grad = None
        torch.autograd.backward([y, h], [dy, dy], retain_graph=True)

    s = bench_samples(bwd, repeats=reps)
    _report(f"rmsnorm_add_bwd/{rows}x{cols}", s, bytes_moved=rows * cols * 2.0 * 4)
    hh = torch.randn(16384, 2 * 3584, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    with torch.no_grad():
        s = bench_samples(lambda: swiglu(hh), repeats=reps)
    _report("swiglu_fwd/16384x3584", s, bytes_moved=16384 * 3584 * 2.0 * 3)
    qkv = torch.randn(16384, 28 * 64, device="cuda", dtype=torch.bfloat16)
    ang = torch.rand(16384, 32, device="cuda")
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    qw = torch.ones(64, device="cuda")
    with torch.no_grad():
        s = bench_samples(lambda: qknorm_rope(qkv[:, :1280].view(16384, 20, 64), qw, cos, sin), repeats=reps)
    _report("qknorm_rope_fwd/16384x20x64", s, bytes_moved=16384 * 1280 * 2.0 * 2)


def case_qk(reps):
    """QK-norm + rotary for the q and k heads of a fused qkv buffer in one launch, forward and backward (the
    backward also writes the MXFP8 copy of the whole d(qkv) row), at the training shape."""
    import ctypes

    from kohakuwullm_b200.ops import mxfp8 as mx
    from kohakuwullm_b200.ops import native

    L = native.require()
    ci, cf = ctypes.c_int, ctypes.c_float
    T, Hq, Hkv, D = 4096, 20, 4, 64
    cols = (Hq + 2 * Hkv) * D
    qkv = torch.randn(T, cols, device="cuda").bfloat16()
    wq, wk = torch.ones(D, device="cuda"), torch.ones(D, device="cuda")
    ang = torch.rand(T, 32, device="cuda") * 6.28
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    q, k = torch.empty(T, Hq, D, device="cuda", dtype=torch.bfloat16), torch.empty(T, Hkv, D, device="cuda", dtype=torch.bfloat16)
    dq, dk = torch.randn_like(q), torch.randn_like(k)
    dqkv = torch.zeros(T, cols, device="cuda", dtype=torch.bfloat16)
    dwq, dwk = torch.zeros(D, device="cuda"), torch.zeros(D, device="cuda")
    q8, sf = mx.alloc_quantized(T, cols, "cuda")
    st = native.stream_ptr()

    def fwd():
        L.kwu_qknorm_rope_fwd_qk(native.ptr(qkv), ci(cols), native.ptr(q), native.ptr(k), native.ptr(wq), native.ptr(wk),
                                 native.ptr(cos), native.ptr(sin), ci(T), ci(Hq), ci(Hkv), ci(32), cf(1e-6), ci(1), st)

    def bwd():
        L.kwu_qknorm_rope_bwd_qk(native.ptr(qkv), ci(cols), native.ptr(dq), native.ptr(dk), native.ptr(dqkv), ci(cols),
                                 native.ptr(wq), native.ptr(wk), native.ptr(dwq), native.ptr(dwk), native.ptr(cos),
                                 native.ptr(sin), ci(T), ci(Hq), ci(Hkv), ci(32), cf(1e-6), ci(1), native.ptr(q8), ci(cols),
                                 native.ptr(sf), st)

    qk_bytes = T * (Hq + Hkv) * D * 2.0
    s = bench_samples(fwd, repeats=reps)
    _report(f"qknorm_rope_fwd_qk/{T}x{Hq}+{Hkv}x{D}", s, bytes_moved=2 * qk_bytes)
    s = bench_samples(bwd, repeats=reps)
    _report(f"qknorm_rope_bwd_qk_mx/{T}x{Hq}+{Hkv}x{D}", s, bytes_moved=3 * qk_bytes + T * cols * 1.0 + T * Hkv * D * 2.0)


def case_loss(reps):
    from kohakuwullm_b200.ops.loss import linear_cross_entropy

    T, D, V = 4096, 1280, 65536
    h = (torch.randn(T, D, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
    w = (torch.randn(V, D, device="cuda") * 0.02).to(torch.bfloat16).requires_grad_()
    labels = torch.randint(0, V, (T,), device="cuda")
    with torch.no_grad():
        s = bench_samples(lambda: linear_cross_entropy(h, w, labels), repeats=reps)
    _report(f"linear_ce_fwd/{T}x{D}x{V}", s, flops=2.0 * T * D * V)

    def fb():
        h.grad = w.grad = None
        ce, lse = linear_cross_entropy(h, w, labels)
        (ce.sum() + 1e-4 * (lse ** 2).sum()).backward()

    s = bench_samples(fb, repeats=reps)
    _report(f"linear_ce_fwd_bwd/{T}x{D}x{V}", s, flops=8.0 * T * D * V)


def case_optim(reps):
    from kohakuwullm_b200.parallel.flat import FlatParameters
    from kohakuwullm_b200.training.optim.fused_adamw import FlatAdamW

    for rows in (8192, 57344):     # 134M elements, and 940M: the size of a whole 1B-parameter model's buffers (17 GB)
        lin = torch.nn.Linear(16384, rows, bias=False, device="cuda", dtype=torch.bfloat16)
        flat = FlatParameters(lin)
        opt = FlatAdamW(flat)
        n = lin.weight.numel()
        s = bench_samples(lambda: opt.step(), repeats=reps)
        _report(f"adamw_flat/{n}", s, bytes_moved=n * (4 * 4 * 2 + 2.0))   # grad r+zero, master/m/v r+w, bf16 w
        import ctypes

        from kohakuwullm_b200.ops import native

        L = native.require()
        grad = flat.grad_buffers()[0] if hasattr(flat, "grad_buffers") else torch.zeros(n, device="cuda")
        partial, out = torch.empty(L.kwu_sumsq_blocks(), device="cuda"), torch.zeros(1, device="cuda")
        s = bench_samples(lambda: L.kwu_sumsq_flat(native.ptr(grad), ctypes.c_longlong(grad.numel()), native.ptr(partial),
                                                   native.ptr(out), ctypes.c_int(0), native.stream_ptr()), repeats=reps)
        _report(f"sumsq_flat/{grad.numel()}", s, bytes_moved=grad.numel() * 4.0)
        del opt, flat, lin, grad


CASES = {"gemm": case_gemm, "wgrad": case_wgrad, "mxfp8": case_mxfp8, "flash": case_flash, "elementwise": case_elementwise, "qk": case_qk, "loss": case_loss,
         "optim": case_optim}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default=None, choices=sorted(CASES))
    ap.add_argument("--reps", type=int, default=10)
    args = ap.parse_args(argv)
    for name, fn in CASES.items():
        if args.only in (None, name):
            fn(args.reps)
    from kohakuwullm_b200.ops import native

    torch.cuda.synchronize()
    native.check_status()


if __name__ == "__main__":
    main()
