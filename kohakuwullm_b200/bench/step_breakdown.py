"""Whole-step time breakdown by kernel family.

    python -m kohakuwullm_b200.bench.step_breakdown [--preset B200-dense-546M] [--micro-tokens 4096]
                                                     [--grad-accum 4] [--json out.json]

One optimizer step of the preset runs EAGER (CUDA graphs off) with a CUDA-event pair around every call
into the native library; the pairs are summed per (entry point, phase) and grouped into families
(MXFP8 GEMM forward / dgrad, bf16 weight gradients, quantise passes, attention forward / backward,
norm + SwiGLU + RoPE, loss head, optimizer + weight refresh). What the events do not cover (ATen fill /
copy kernels, gaps between launches while the host catches up) is reported as ``other / gaps`` = step
device time minus the covered sum. The same step is then timed with graphs on, as the trainer runs it,
so the table ends with the launch-gap cost that graph replay removes and the idle time that remains.

Per-op accounting of the reference: src/kohakuwullm/bench/core/timing.py:150-187,313-383.
"""

from __future__ import annotations

import argparse
import ctypes
import json
from collections import defaultdict

import torch

from kohakuwullm_b200.ops import native

FAMILIES = [
    ("mxfp8 gemm fwd", lambda n, ph: n in ("kwu_gemm_mxfp8", "kwu_gemm_mxfp8_grouped") and ph == "fwd"),
    ("mxfp8 gemm dgrad", lambda n, ph: n in ("kwu_gemm_mxfp8", "kwu_gemm_mxfp8_grouped") and ph == "bwd"),
    ("bf16 gemm fwd", lambda n, ph: n in ("kwu_gemm_bf16", "kwu_gemm_bf16_grouped_rows") and ph == "fwd"),
    ("bf16 gemm bwd (wgrad, dgrad)", lambda n, ph: n in ("kwu_gemm_bf16", "kwu_gemm_bf16_grouped_rows",
                                                          "kwu_gemm_bf16_grouped_wgrad") and ph == "bwd"),
    ("quantise passes", lambda n, ph: n.startswith("kwu_mxfp8_quant") and ph in ("fwd", "bwd")),
    ("flash fwd (+plan)", lambda n, ph: n in ("kwu_flash_fwd", "kwu_attn_plan")),
    ("flash bwd", lambda n, ph: n == "kwu_flash_bwd"),
    ("qk-norm + rope", lambda n, ph: n.startswith("kwu_qknorm_rope")),
    ("rmsnorm", lambda n, ph: n.startswith("kwu_rmsnorm")),
    ("swiglu", lambda n, ph: n.startswith("kwu_swiglu")),
    ("loss head (lse, dlogits, combine)", lambda n, ph: n in ("kwu_gemm_lse", "kwu_gemm_dlogits", "kwu_ce_combine")),
    ("embedding", lambda n, ph: n.startswith("kwu_embedding")),
    ("moe (router, dispatch, combine)", lambda n, ph: n.startswith("kwu_moe") or n.startswith("kwu_ep")),
    ("optimizer (sumsq, clip, adamw)", lambda n, ph: n in ("kwu_sumsq_flat", "kwu_clip_coef", "kwu_adamw_flat",
                                                         "kwu_adamw16", "kwu_ddp_reduce_shard",
                                                         "kwu_ddp_adamw_allgather")),
    ("mxfp8 weight refresh", lambda n, ph: n.startswith("kwu_mxfp8_quant") and ph == "opt"),
]


class TimedLibrary:
    """Stands in for the ctypes handle: every ``kwu_*`` call that takes a stream is bracketed by events."""

    HOST_ONLY = ("kwu_last_error", "kwu_launch_count", "kwu_sumsq_blocks", "kwu_mxfp8_sf_bytes", "kwu_ce_tiles_n",
                 "kwu_flash_bwd_scratch_floats", "kwu_decode_scratch_floats", "kwu_rmsnorm_bwd_blocks",
                 "kwu_moe_max_rows", "kwu_ddp_blocks", "kwu_ep_flag_ints", "kwu_ep_table_ints", "kwu_sr_chunk_bytes",
                 "kwu_gemm_debug_override")

    SHAPE_ARGS = {"kwu_gemm_mxfp8": (5, 6, 7), "kwu_gemm_bf16": (3, 4, 5)}

    def __init__(self, handle: ctypes.CDLL):
        self._h = handle
        self.phase = "fwd"
        self.records: list[tuple[str, str, torch.cuda.Event, torch.cuda.Event]] = []
        self.enabled = False

    def __getattr__(self, name):
        fn = getattr(self._h, name)
        if name in self.HOST_ONLY or not name.startswith("kwu_"):
            return fn

        def timed(*args):
            if not self.enabled:
                return fn(*args)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            rc = fn(*args)
            e1.record()
            label = name
            pos = self.SHAPE_ARGS.get(name)
            if pos is not None:  # GEMMs are listed per (M, N, K)
                label = name + ":" + "x".join(str(getattr(args[i], "value", args[i])) for i in pos)
            self.records.append((label, self.phase, e0, e1))
            return rc

        return timed

    def table(self) -> dict:
        per = defaultdict(lambda: [0, 0.0])
        for name, ph, e0, e1 in self.records:
            per[(name, ph)][0] += 1
            per[(name, ph)][1] += e0.elapsed_time(e1)
        return per


def event_pair_overhead_ms(n: int = 400) -> float:
    """Device time between two events recorded back to back with nothing in between, while the GPU is
    busy (as it is inside a step): what every bracketed call pays on top of its kernels."""
    x = torch.empty(1 << 22, device="cuda")
    pairs = []
    for _ in range(n):
        x.add_(1.0)                      # keeps the stream busy so that the events queue behind real work
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        e1.record()
        pairs.append((e0, e1))
    torch.cuda.synchronize()
    vals = sorted(a.elapsed_time(b) for a, b in pairs)
    return vals[len(vals) // 2]


def family_of(name: str, phase: str) -> str:
    for fam, pred in FAMILIES:
        if pred(name, phase):
            return fam
    return f"{name} ({phase})"


def run(preset: str, micro_tokens: int, grad_accum: int, mxfp8: bool | None, depth: int | None, len_min: int,
        len_max: int, steps: int = 3) -> dict:
    from kohakuwullm_b200.data.synthetic import make_packs
    from kohakuwullm_b200.models import LMBackbone, get_preset
    from kohakuwullm_b200.training.engine import TrainEngine

    dev = torch.device("cuda", torch.cuda.current_device())
    torch.manual_seed(1234)
    overrides = {}
    if mxfp8 is not None:
        overrides["mxfp8"] = mxfp8
    if depth is not None:
        overrides["depth"] = depth
    cfg = get_preset(preset, **overrides)
    with torch.device(dev):
        model = LMBackbone(cfg)
    engine = TrainEngine(model, lr=1e-4, param_dtype=torch.bfloat16, cuda_graphs=False)
    packs = [p.to(dev) for p in make_packs(grad_accum, micro_tokens, len_min, len_max, cfg.vocab_size, seed=17)]

    handle = native.lib()
    timed = TimedLibrary(handle)
    original = native.lib
    orig_backward = torch.Tensor.backward
    orig_opt = engine.optimizer.step
    orig_norm = engine._grad_norm_and_coef
    native.lib = lambda: timed  # ops fetch the handle through native.lib() / native.require() on every call
    try:
        for _ in range(3):
            engine.step(packs)
        torch.cuda.synchronize()
        # phases are told apart by hooks: forward until loss.backward(), optimizer after the last micro-batch
        def backward(self, *a, **k):
            timed.phase = "bwd"
            out = orig_backward(self, *a, **k)
            timed.phase = "fwd"
            return out

        def opt_step(*a, **k):
            timed.phase = "opt"
            return orig_opt(*a, **k)

        def norm_and_coef(*a, **k):
            timed.phase = "opt"
            return orig_norm(*a, **k)

        torch.Tensor.backward = backward
        engine.optimizer.step = opt_step
        engine._grad_norm_and_coef = norm_and_coef
        timed.enabled = True
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        for _ in range(steps):
            timed.phase = "fwd"
            engine.step(packs)
        e.record()
        torch.cuda.synchronize()
        eager_ms = s.elapsed_time(e) / steps
        timed.enabled = False
        per = timed.table()
    finally:
        torch.Tensor.backward = orig_backward
        native.lib = original
        engine.optimizer.step = orig_opt
        engine._grad_norm_and_coef = orig_norm

    # an event pair is not free: the gap it adds (measured with nothing between the two records) is taken
    # off every bracketed call, so that 3000 small launches do not look 15 ms heavier than they are
    pair_ms = event_pair_overhead_ms()
    fams = defaultdict(lambda: [0, 0.0])
    calls = {}
    for (name, ph), (n, ms) in per.items():
        f = family_of(name.split(":")[0], ph)
        net = max(ms - n * pair_ms, 0.0)
        fams[f][0] += n / steps
        fams[f][1] += net / steps
        calls[f"{name}/{ph}"] = {"launches_per_step": n / steps, "ms_per_step": net / steps,
                                 "us_per_call": 1e3 * net / max(n, 1)}
    covered = sum(v[1] for v in fams.values())

    # the step as the trainer runs it: micro-batches replayed from CUDA graphs
    engine.cuda_graphs = True
    for _ in range(3):
        engine.step(packs)
    torch.cuda.synchronize()
    s.record()
    for _ in range(steps):
        engine.step(packs)
    e.record()
    torch.cuda.synchronize()
    graph_ms = s.elapsed_time(e) / steps
    tokens = micro_tokens * grad_accum
    return {
        "preset": preset, "micro_tokens": micro_tokens, "grad_accum": grad_accum,
        "eager_ms_per_step": eager_ms, "graph_ms_per_step": graph_ms, "covered_ms": covered,
        "event_pair_overhead_us": 1e3 * pair_ms,
        "other_and_gaps_ms_eager": eager_ms - covered,
        "idle_and_aten_ms_graph": graph_ms - covered,
        "tokens_per_s_graph": tokens / graph_ms * 1e3,
        "families": {k: {"launches_per_step": v[0], "ms_per_step": v[1], "share_of_graph_step": v[1] / graph_ms}
                     for k, v in sorted(fams.items(), key=lambda kv: -kv[1][1])},
        "calls": dict(sorted(calls.items(), key=lambda kv: -kv[1]["ms_per_step"])),
    }


def render(res: dict) -> str:
    lines = [f"step breakdown: {res['preset']}, {res['grad_accum']} x {res['micro_tokens']} tokens",
             f"eager step {res['eager_ms_per_step']:.2f} ms; graph-replayed step {res['graph_ms_per_step']:.2f} ms "
             f"({res['tokens_per_s_graph'] / 1e3:.1f}k tokens/s); event-covered kernels {res['covered_ms']:.2f} ms "
             f"after taking {res['event_pair_overhead_us']:.1f} us per bracketed call off (the measured cost of an "
             f"empty event pair)",
             "", "| family | launches/step | ms/step | share of the graph-replayed step |", "|---|---|---|---|"]
    for k, v in res["families"].items():
        lines.append(f"| {k} | {v['launches_per_step']:.0f} | {v['ms_per_step']:.3f} | {100 * v['share_of_graph_step']:.1f} % |")
    lines.append(f"| ATen fill/copy kernels + idle gaps (graph step - covered) | | {res['idle_and_aten_ms_graph']:.3f} | "
                 f"{100 * res['idle_and_aten_ms_graph'] / res['graph_ms_per_step']:.1f} % |")
    lines += ["", "| entry point / phase | launches/step | ms/step | us/call |", "|---|---|---|---|"]
    for k, v in res["calls"].items():
        lines.append(f"| {k} | {v['launches_per_step']:.0f} | {v['ms_per_step']:.3f} | {v['us_per_call']:.1f} |")
    return "\n".join(lines)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", default="B200-dense-546M")
    ap.add_argument("--micro-tokens", type=int, default=4096)
    ap.add_argument("--grad-accum", type=int, default=4)
    ap.add_argument("--len-min", type=int, default=64)
    ap.add_argument("--len-max", type=int, default=4096)
    ap.add_argument("--depth", type=int, default=None)
    ap.add_argument("--no-mxfp8", action="store_true")
    ap.add_argument("--json", default=None)
    args = ap.parse_args()
    res = run(args.preset, args.micro_tokens, args.grad_accum, False if args.no_mxfp8 else None, args.depth,
              args.len_min, args.len_max)
    print(render(res))
    if args.json:
        with open(args.json, "w") as f:
            json.dump(res, f, indent=1)


if __name__ == "__main__":
    main()
