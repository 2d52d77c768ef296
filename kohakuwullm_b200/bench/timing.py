"""Benchmark harness: CUDA-event timing with an L2 flush between samples, CUDA-graph replay timing, host
enqueue cost, error metrics in ULP, and roofline fractions against the MEASURED peaks of this machine
(``MEASURED_PEAKS.json`` at the repository root; fall-back figures otherwise).
Reference: src/kohakuwullm/bench/core/timing.py:21-385."""

from __future__ import annotations

import json
import statistics
import time
from pathlib import Path
from typing import Callable

import torch

L2_FLUSH_BYTES = 256 * 1024 * 1024
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
NVLINK_PEER_GBS = 770.0       # measured peer copy, per direction per GPU
HOST_SHARE_LIMIT = 0.5        # a sample whose host enqueue time exceeds this share of device time is launch-bound
CEILING_SLACK = 1.02

_flush_buf: dict = {}


def measured_peaks() -> dict:
    path = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    try:
        data = json.loads(path.read_text())
        return {**FALLBACK_PEAKS, **{k: data[k] for k in FALLBACK_PEAKS if k in data}, "source": "measured"}
    except (OSError, ValueError):
        return {**FALLBACK_PEAKS, "source": "fallback"}


def flush_l2(device=None) -> None:
    """Overwrite a buffer twice the size of the 126 MB L2 so the next sample starts cold."""
    dev = torch.device(device or "cuda")
    buf = _flush_buf.get(dev)
    if buf is None:
        buf = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=dev)
        _flush_buf[dev] = buf
    buf.zero_()


def bench_samples(fn: Callable, *, warmup: int = 3, repeats: int = 20, flush: bool = True) -> list[float]:
    """Per-call device milliseconds (CUDA events on the launching stream, synchronised on both sides)."""
    for _ in range(max(warmup, 3)):
        fn()
    samples = []
    for _ in range(repeats):
        if flush:
            flush_l2()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        # keep the GPU busy for ~0.1 ms so that the host enqueues start event, work and end event before
        # the device reaches them: the interval then holds device time only, not host launch latency
        torch.cuda._sleep(200_000)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        samples.append(s.elapsed_time(e))
    return samples


def timing_profile(samples: list[float]) -> dict:
    q = statistics.quantiles(samples, n=10) if len(samples) >= 10 else [min(samples)] * 9
    return {"median_ms": statistics.median(samples), "p10_ms": q[0], "p90_ms": q[-1], "min_ms": min(samples), "n": len(samples)}


def bench_ms(fn: Callable, **kw) -> float:
    return statistics.median(bench_samples(fn, **kw))


def graph_ms(fn: Callable, replays: int = 20, warmup: int = 3) -> float:
    """Device time of ``fn`` replayed from a CUDA graph (launch overhead removed)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(warmup):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    g.replay()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(replays):
        g.replay()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / replays


def cpu_enqueue_ms(fn: Callable, repeats: int = 20) -> float:
    """Host time to ENQUEUE the work (no synchronisation inside the timed region)."""
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(repeats):
        fn()
    dt = (time.perf_counter() - t0) * 1e3 / repeats
    torch.cuda.synchronize()
    return dt


def bench_peak_memory(fn: Callable) -> float:
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    base = torch.cuda.memory_allocated()
    fn()
    torch.cuda.synchronize()
    return (torch.cuda.max_memory_allocated() - base) / 2 ** 30


def ulp_error(got: torch.Tensor, want: torch.Tensor) -> dict:
    """Error of ``got`` against a higher-precision ``want`` in units in the last place of got's dtype."""
    dtype = got.dtype
    ref = want.to(torch.float64)
    spacing = torch.abs(torch.nextafter(ref.to(dtype), torch.full_like(ref, float("inf")).to(dtype)).double() - ref.to(dtype).double())
    spacing = spacing.clamp(min=torch.finfo(dtype).tiny)
    ulp = (got.double() - ref).abs() / spacing
    return {"max_ulp": float(ulp.max()), "mean_ulp": float(ulp.mean())}


def rel_error(got: torch.Tensor, want: torch.Tensor) -> float:
    return float((got.double() - want.double()).norm() / want.double().norm().clamp(min=1e-30))


def stream_bandwidths(n_bytes: int = 2 ** 30, repeats: int = 10) -> dict:
    """STREAM-style copy and triad (GB/s) on the current device."""
    n = n_bytes // 4
    a, b, c = (torch.empty(n, dtype=torch.float32, device="cuda").normal_() for _ in range(3))
    copy = min(bench_samples(lambda: a.copy_(b), repeats=repeats, flush=False))
    triad = min(bench_samples(lambda: torch.add(b, c, alpha=2.0, out=a), repeats=repeats, flush=False))
    return {"copy_gbs": 2 * n * 4 / copy / 1e6, "triad_gbs": 3 * n * 4 / triad / 1e6}


def module_metrics(ms: float, *, flops: float = 0.0, bytes_moved: float = 0.0, sustained: bool = False) -> dict:
    """Achieved throughput and its fraction of the measured roofline ("of measured" / "of fallback")."""
    peaks = measured_peaks()
    tf_peak = peaks["bf16_tflops_sustained" if sustained else "bf16_tflops"]
    out = {"ms": ms, "peaks": peaks["source"]}
    if flops:
        out["tflops"] = flops / ms / 1e9
        out["frac_of_tensor_peak"] = out["tflops"] / tf_peak
    if bytes_moved:
        out["gbs"] = bytes_moved / ms / 1e6
        out["frac_of_hbm_peak"] = out["gbs"] / peaks["hbm_gbs"]
    return out


def device_op_counts(fn: Callable) -> dict:
    """Device kernels launched by one call of ``fn`` and their summed device time, per kernel name."""
    from torch.profiler import ProfilerActivity, profile

    fn()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        fn()
        torch.cuda.synchronize()
    out = {}
    for ev in prof.key_averages():
        if ev.device_time_total > 0:
            out[ev.key] = {"count": ev.count, "device_us": ev.device_time_total}
    return out


def gpu_is_busy(threshold_ms: float = 1.5, probe_ms_expected: float = 0.2) -> bool:
    """Contention probe: a fixed small kernel that takes far longer than expected means the GPU is shared."""
    x = torch.empty(2 ** 24, device="cuda")
    t = min(bench_samples(lambda: x.add_(1.0), repeats=5, flush=False))
    return t > max(threshold_ms, 5 * probe_ms_expected)
