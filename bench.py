"""Headline benchmark: training tokens/s of the dense ~546M config on N B200s of one node.

    python bench.py --gpus 1 --steps 8 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 8 --warmup 3
    python bench.py --impl reference ...      # the unmodified reference from baseline/_ref

Config (the dense DDP config this framework is measured on): d_model 1280, 24 layers, 20 query / 4 KV
heads of 64, QK-norm, RoPE theta 5e5, SwiGLU 3584, vocab 65536 untied; per GPU 4 micro-batches of
one 4096-token pack (documents uniform in [64, 4096], random ids), token-exact accumulation, fused
AdamW, DDP. Data are synthetic, weights random-init.

The step is timed twice:
  value  device time (CUDA events, barrier + synchronize on both sides, max over ranks) of K steps
         whose packs are already resident on the device;
  e2e    the same K steps through ``TrainEngine.step`` with every pack copied host->device from pinned
         memory inside the timed region and the loss read back to the host every step.
Rank 0 prints one JSON line.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

MICRO_TOKENS = 4096
GRAD_ACCUM = 4
LEN_MIN, LEN_MAX = 64, 4096
PRESET = "B200-dense-546M"
METRIC = "train_tokens_per_sec"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.device_index}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def _dist_setup(n_gpus: int):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if world != n_gpus:
        raise SystemExit(f"--gpus {n_gpus} but WORLD_SIZE={world}: launch with torch.distributed.run for N>1")
    return rank, world, local


def _timed(fn, steps: int, world: int):
    """Device time of ``steps`` calls of fn (ms total), max over ranks."""
    import torch
    import torch.distributed as dist

    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    wall0 = time.perf_counter()
    start.record()
    for _ in range(steps):
        fn()
    end.record()
    torch.cuda.synchronize()
    wall = (time.perf_counter() - wall0) * 1e3
    if world > 1:
        dist.barrier()
    ms = max(start.elapsed_time(end), 0.0)
    t = torch.tensor([ms, wall], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0]), float(t[1])


def run_ours(args):
    import torch

    from kohakuwullm_b200.data.synthetic import make_packs
    from kohakuwullm_b200.models import LMBackbone, get_preset
    from kohakuwullm_b200.ops import native
    from kohakuwullm_b200.training.engine import TrainEngine

    rank, world, local = _dist_setup(args.gpus)
    dev = torch.device("cuda", local)
    torch.manual_seed(1234)
    overrides = {}
    if args.no_mxfp8:
        overrides["mxfp8"] = False
    cfg = get_preset(PRESET, **overrides)
    with torch.device(dev):
        model = LMBackbone(cfg)
    mode = args.grad_sync
    if mode == "auto":
        mode = "fused" if world > 1 else "nccl"
    try:
        engine = TrainEngine(model, lr=1e-4, param_dtype=torch.bfloat16, grad_sync=mode)
    except Exception as exc:  # noqa: BLE001  symmetric memory unavailable: keep the run alive on NCCL
        if mode != "fused" or args.grad_sync == "fused":
            raise
        print(f"[bench] fused gradient sync unavailable ({type(exc).__name__}: {exc}); using NCCL", file=sys.stderr)
        mode = "nccl"
        engine = TrainEngine(model, lr=1e-4, param_dtype=torch.bfloat16, grad_sync=mode)
    args.grad_sync = mode

    host_packs = [p.pin_memory() for p in make_packs(GRAD_ACCUM, MICRO_TOKENS, LEN_MIN, LEN_MAX, cfg.vocab_size, seed=17 + rank)]
    dev_packs = [p.to(dev) for p in host_packs]
    losses = []

    def step_device():
        engine.step(dev_packs)

    def step_e2e():
        out = engine.step(host_packs)
        losses.append(float(out["loss"]))  # device->host read of the step result

    for _ in range(args.warmup):
        step_e2e()
    torch.cuda.synchronize()
    native.check_status()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = engine.native_launch_total()
    ms_dev, _ = _timed(step_device, args.steps, world)
    launches = engine.native_launch_total() - launches0
    ms_e2e, wall_e2e = _timed(step_e2e, args.steps, world)
    clocks = sampler.stop() if rank == 0 else {}
    native.check_status()

    evidence = _multi_gpu_evidence(engine, cfg, dev, rank, world, host_packs, args) if world > 1 else {}

    tokens_per_step = MICRO_TOKENS * GRAD_ACCUM * world
    value = tokens_per_step * args.steps / (ms_dev / 1e3)
    e2e_value = tokens_per_step * args.steps / (max(ms_e2e, wall_e2e) / 1e3)
    h2d = sum(p.nbytes() for p in host_packs) + 4  # + the token-count scalar
    if rank == 0:
        baseline = _published_baseline()
        print(json.dumps({
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_dev / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": (value / baseline) if baseline else None,
            "dtype": "bf16" if args.no_mxfp8 else "bf16+mxfp8", "data": "synthetic", "impl": "kohakuwullm_b200",
            "config": {"model": "dense-546M (d1280 L24 h20/kv4 ffn3584 v65536)",
                       "global_batch": tokens_per_step, "seq_len": MICRO_TOKENS, "grad_accum": GRAD_ACCUM,
                       "parallelism": f"dp{world}", "grad_sync": args.grad_sync,
                       "l2": "working set per step (>10 GB of weights, activations and optimizer state) is far larger than the 126 MB L2"},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": max(ms_e2e, wall_e2e) / args.steps,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
            "gpu_launches": int(launches),
            "final_loss": losses[-1] if losses else None,
            **evidence,
        }))
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


def _multi_gpu_evidence(engine, cfg, dev, rank, world, host_packs, args) -> dict:
    """Correctness evidence a multi-GPU run carries with its number (the single-GPU test run cannot):

    ``params_equal_across_ranks``  after all the steps above every rank holds bit-identical parameters (an fp64 sum
                                   and an XOR-free integer digest of the raw bytes, all-gathered and compared);
    ``nccl_check``                 two FRESH engines of the same seed, one on the fused peer-memory gradient step and
                                   one on NCCL all-reduce + unsharded AdamW, run the same packs for a few steps: the
                                   per-step losses of the two paths side by side and their largest difference.
    """
    import torch
    import torch.distributed as dist

    from kohakuwullm_b200.models import LMBackbone
    from kohakuwullm_b200.training.engine import TrainEngine

    out: dict = {}
    digests = []
    for g in engine.flat.groups.values():
        raw = g.data.view(torch.uint8).to(torch.int64)
        weights = torch.arange(1, raw.numel() + 1, device=dev, dtype=torch.int64) % 8191
        digests.append(torch.stack([(raw * weights).sum(), raw.sum()]))
    digest = torch.cat(digests)
    gathered = [torch.empty_like(digest) for _ in range(world)]
    dist.all_gather(gathered, digest)
    out["params_equal_across_ranks"] = bool(all(torch.equal(gathered[0], g) for g in gathered))
    if args.grad_sync != "fused" or args.skip_nccl_check:
        return out
    curves = {}
    for mode in ("fused", "nccl"):
        torch.manual_seed(1234)
        with torch.device(dev):
            model = LMBackbone(cfg)
        eng = TrainEngine(model, lr=1e-4, param_dtype=torch.bfloat16, grad_sync=mode)
        curve = [float(eng.step(host_packs)["loss"]) for _ in range(args.check_steps)]
        curves[mode] = curve
        del eng, model
        torch.cuda.empty_cache()
    diff = max(abs(a - b) for a, b in zip(curves["fused"], curves["nccl"]))
    out["nccl_check"] = {"steps": args.check_steps, "fused_loss": curves["fused"], "nccl_loss": curves["nccl"],
                         "max_abs_diff": diff, "agree": bool(diff < 5e-2)}
    return out


def _published_baseline():
    """The reference publishes no B200 number for this config (BASELINE.json ``published`` is empty)."""
    try:
        data = json.loads((ROOT / "BASELINE.json").read_text())
        pub = data.get("published") or {}
        return float(pub[METRIC]) if METRIC in pub else None
    except (OSError, ValueError, TypeError):
        return None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--grad-sync", default="auto", choices=["auto", "nccl", "fused"],
                    help="auto: fused NVLink peer-memory kernels when N>1 (NCCL all-reduce if they cannot be set up)")
    ap.add_argument("--ref-attn", default="triton", help="attention backend of the reference arm")
    ap.add_argument("--no-mxfp8", action="store_true", help="bf16 linears instead of MXFP8 (diagnostic only)")
    ap.add_argument("--check-steps", type=int, default=4, help="steps of the fused-vs-NCCL loss comparison (N > 1)")
    ap.add_argument("--skip-nccl-check", action="store_true", help="N > 1: skip the fused-vs-NCCL loss comparison")
    ap.add_argument("--ref-dtype", default="fp32", choices=["fp32", "bf16"],
                    help="reference arm: parameter dtype (fp32 + fused AdamW is its default arm; bf16 = adamw16)")
    ap.add_argument("--ref-compile", action="store_true",
                    help="reference arm: per-block torch.compile in reduce-overhead mode (its harness's --compile)")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        from baseline.reference_arm import run_reference

        run_reference(args, MICRO_TOKENS, GRAD_ACCUM, LEN_MIN, LEN_MAX, METRIC, ClockSampler, _timed, _dist_setup)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
