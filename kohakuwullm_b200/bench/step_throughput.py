"""Step throughput of any preset at a fixed optimizer-step token budget.

    python -m kohakuwullm_b200.bench.step_throughput --preset B200-moe-991M --micro-tokens 4096 --accum 4
    torchrun --nproc-per-node 4 -m kohakuwullm_b200.bench.step_throughput --preset B200-moe-991M --pipeline

Data-parallel mode runs ``TrainEngine`` (token-exact accumulation, fused gradient sync on N>1); with
``--pipeline`` the ranks form a pipeline whose split is measured at start-up (``measure_costs`` on rank 0,
broadcast, ``plan_for``) and driven by the 1F1B schedule. Packs are synthetic (documents uniform or
log-uniform in ``[len-min, len-max]``, random ids). Timing: CUDA events around ``--steps`` steps after
``--warmup`` steps, barrier + synchronize on both sides, max over ranks.
Reference: scripts/bench/e2e/step_throughput.py:100-374.
"""

from __future__ import annotations

import argparse
import json
import os
import time

import torch
import torch.distributed as dist

from kohakuwullm_b200.data.synthetic import make_packs
from kohakuwullm_b200.models import LMBackbone, get_preset


def _timed(fn, steps, world):
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(steps):
        fn()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e)], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", default="B200-dense-546M")
    ap.add_argument("--micro-tokens", type=int, default=4096)
    ap.add_argument("--accum", type=int, default=4)
    ap.add_argument("--len-min", type=int, default=64)
    ap.add_argument("--len-max", type=int, default=4096)
    ap.add_argument("--log-uniform", action="store_true")
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--pipeline", action="store_true")
    ap.add_argument("--schedule", default="1f1b")
    ap.add_argument("--no-mxfp8", action="store_true")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--expert-parallel", action="store_true", help="split MoE experts over the ranks (EP + DP)")
    ap.add_argument("--grad-sync", default=None, choices=["nccl", "fused"])
    ap.add_argument("--router-bias-std", type=float, default=0.0,
                    help="seeded N(0, std) selection bias on every router: a skewed expert load")
    ap.add_argument("--ep-capacity", type=float, default=2.0, help="expert-parallel receive capacity factor")
    ap.add_argument("--no-head-only-stage", action="store_true",
                    help="pipeline: every stage must hold at least one block (default: the last may hold the head only)")
    ap.add_argument("--stage-report", action="store_true",
                    help="pipeline: per-stage busy time (CUDA events around every stage forward / backward), the "
                         "bubble share of the step and the cost of one boundary hop")
    ap.add_argument("--set", action="append", default=[], help="config override KEY=VALUE (python literal)")
    args = ap.parse_args(argv)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if args.pipeline:
            dist.init_process_group("nccl")  # lazy: per-pair communicators for P2P
        else:
            dist.init_process_group("nccl", device_id=dev)
    overrides = {}
    for kv in args.set:
        k, v = kv.split("=", 1)
        try:
            overrides[k] = eval(v, {}, {})  # noqa: S307  operator-supplied literals
        except Exception:  # noqa: BLE001
            overrides[k] = v
    if args.no_mxfp8:
        overrides["mxfp8"] = False
    cfg = get_preset(args.preset, **overrides)
    torch.manual_seed(1234)

    if args.pipeline and world > 1:
        from kohakuwullm_b200.pipe.trainer import PipelineTrainer
        from kohakuwullm_b200.training.parallel.autotune import broadcast_costs, measure_costs
        from kohakuwullm_b200.training.parallel.pipeline import plan_for
        from kohakuwullm_b200.training.parallel.uwupipe import LMPipelineModule

        costs = measure_costs(cfg, args.micro_tokens, dev) if rank == 0 else None
        costs = broadcast_costs(costs, cfg.depth, dev)
        # a head as wide as this vocabulary costs more than two blocks: the planner may give it a stage of its own
        plans = plan_for(cfg, world, args.micro_tokens, costs=costs, allow_empty_last=not args.no_head_only_stage)
        module = LMPipelineModule(cfg, micro_tokens=args.micro_tokens, lr=1e-4)
        trainer = PipelineTrainer(module, plans, rank=rank, world=world, device=dev, n_micro=args.accum,
                                  schedule=args.schedule)
        packs = make_packs(args.accum, args.micro_tokens, args.len_min, args.len_max, cfg.vocab_size, seed=17,
                           log_uniform=args.log_uniform)
        step = lambda: trainer.loop.step(packs)  # noqa: E731
        split = [p.num_layers for p in plans]
        tokens_per_step = args.micro_tokens * args.accum
    else:
        from kohakuwullm_b200.training.engine import TrainEngine

        with torch.device(dev):
            model = LMBackbone(cfg)
        if args.router_bias_std > 0:
            gen = torch.Generator(device=dev).manual_seed(4242)     # the same skew on every rank
            for m in model.modules():
                if hasattr(m, "expert_bias"):
                    m.expert_bias.copy_(torch.randn(m.expert_bias.shape, generator=gen, device=dev) * args.router_bias_std)
                    m.bias_update_rate = 0.0                          # keep the skew for the whole measurement
        engine = TrainEngine(model, lr=1e-4, param_dtype=torch.bfloat16, ep_capacity_factor=args.ep_capacity,
                             grad_sync=args.grad_sync or ("fused" if world > 1 else "nccl"),
                             cuda_graphs=not args.no_graphs, expert_parallel=args.expert_parallel)
        packs = [p.to(dev) for p in make_packs(args.accum, args.micro_tokens, args.len_min, args.len_max,
                                               cfg.vocab_size, seed=17 + rank, log_uniform=args.log_uniform)]
        step = lambda: engine.step(packs)  # noqa: E731
        split = None
        tokens_per_step = args.micro_tokens * args.accum * world

    for _ in range(args.warmup):
        out = step()
    ms = _timed(step, args.steps, world)
    from kohakuwullm_b200.ops import native

    native.check_status()
    report = {}
    if args.stage_report and args.pipeline and world > 1 and hasattr(trainer.schedule, "busy_ms"):
        from kohakuwullm_b200.pipe.latency import hop_cost

        trainer.schedule.profile = True
        for _ in range(2):
            step()
        busy = trainer.schedule.busy_ms()
        trainer.schedule.profile = False
        mine = torch.tensor([busy["forward"] / 2, busy["backward"] / 2], device=dev)
        every = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(every, mine)
        hop = hop_cost(args.micro_tokens * cfg.dim * 2, dev)
        per = ms / args.steps
        fwd = [round(float(t[0]), 2) for t in every]
        bwd = [round(float(t[1]), 2) for t in every]
        report = {"stage_forward_ms": fwd, "stage_backward_ms": bwd,
                  "stage_busy_share": [round((a + b) / per, 3) for a, b in zip(fwd, bwd)],
                  "bubble_share_of_slowest_stage": round(1.0 - max(a + b for a, b in zip(fwd, bwd)) / per, 3),
                  "hop_us": round(hop["seconds"] * 1e6, 1), "hop_gb_per_s": round(hop["gb_per_s"], 1)}
    if rank == 0:
        loss = out["loss"] if isinstance(out, dict) else out.loss
        print(json.dumps({**report, "preset": args.preset, "n_gpus": world, "mode": "pipeline" if args.pipeline and world > 1 else ("ep+dp" if args.expert_parallel and world > 1 else "dp"),
                          "split": split, "tokens_per_step": tokens_per_step, "ms_per_step": ms / args.steps,
                          "tokens_per_s": tokens_per_step * args.steps / (ms / 1e3), "loss": float(loss),
                          "peak_mem_gib": torch.cuda.max_memory_allocated() / 2 ** 30}))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
