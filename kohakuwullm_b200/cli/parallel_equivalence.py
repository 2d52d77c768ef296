"""Parallel-equivalence harness: the same tokens, trained for a few steps under different parallel
layouts, must give the same losses (up to summation order).

    torchrun --nproc-per-node 2 -m kohakuwullm_b200.cli.parallel_equivalence --mode ddp
    torchrun --nproc-per-node 2 -m kohakuwullm_b200.cli.parallel_equivalence --mode ep --preset B200-moe-991M
    torchrun --nproc-per-node 2 -m kohakuwullm_b200.cli.parallel_equivalence --mode pipeline

Every rank first runs the single-process baseline on the WHOLE step batch (same seed, same weights),
then the group runs the parallel layout on its shares of that batch; rank 0 prints one JSON line with
both loss curves and their largest difference, and exits non-zero when it exceeds ``--tol``.
Works on CPU (gloo) and GPU (nccl). Reference: scripts/dist/parallel_equivalence.py:177-218.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist


def _build(args, device):
    from kohakuwullm_b200.models import LMBackbone, get_preset

    overrides = dict(depth=args.depth, vocab_size=args.vocab)
    if device.type == "cpu":
        overrides.update(mxfp8=False)
    cfg = get_preset(args.preset, **overrides)
    torch.manual_seed(args.seed)
    with torch.device(device):
        model = LMBackbone(cfg)
    return cfg, model


def _packs(args, cfg, step):
    from kohakuwullm_b200.data.synthetic import make_packs

    return make_packs(args.micro_batches, args.micro_tokens, 16, max(32, args.micro_tokens // 4), cfg.vocab_size,
                      seed=args.seed + step)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="ddp", choices=["ddp", "ddp-fused", "ep", "pipeline"])
    ap.add_argument("--preset", default="B200-smoke")
    ap.add_argument("--depth", type=int, default=4)
    ap.add_argument("--vocab", type=int, default=4096)
    ap.add_argument("--micro-tokens", type=int, default=1024)
    ap.add_argument("--micro-batches", type=int, default=4, help="micro-batches per step over the whole group")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--seed", type=int, default=11)
    ap.add_argument("--tol", type=float, default=5e-3)
    args = ap.parse_args(argv)

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    cuda = torch.cuda.is_available()
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0))) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(device)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29555")
    if world > 1:
        dist.init_process_group("nccl" if cuda else "gloo", rank=rank, world_size=world,
                                **({"device_id": device} if cuda else {}))
    if args.micro_batches % world:
        raise SystemExit("--micro-batches must be a multiple of the world size")
    from kohakuwullm_b200.training.engine import TrainEngine

    dtype = torch.bfloat16 if cuda else None
    # ---- baseline: one process, the whole batch (built without the process group so nothing is reduced)
    cfg, model = _build(args, device)
    base = TrainEngine(model, lr=1e-3, param_dtype=dtype, group=None, grad_sync="nccl", cuda_graphs=False)
    base.world, base.sync.world = 1, 1
    base_loss = [float(base.step(_packs(args, cfg, s))["loss"]) for s in range(args.steps)]
    del base, model

    # ---- parallel layout
    cfg, model = _build(args, device)
    if args.mode == "pipeline":
        from kohakuwullm_b200.pipe.trainer import PipelineTrainer
        from kohakuwullm_b200.training.parallel.pipeline import plan_for
        from kohakuwullm_b200.training.parallel.uwupipe import LMPipelineModule

        plans = plan_for(cfg, world, args.micro_tokens)
        module = LMPipelineModule(cfg, micro_tokens=args.micro_tokens, lr=1e-3, seed=args.seed)
        trainer = PipelineTrainer(module, plans, rank=rank, world=world, device=device, n_micro=args.micro_batches)
        par_loss = [float(trainer.loop.step(_packs(args, cfg, s)).loss) for s in range(args.steps)]
    else:
        eng = TrainEngine(model, lr=1e-3, param_dtype=dtype, cuda_graphs=False,
                          grad_sync="fused" if args.mode == "ddp-fused" else "nccl",
                          expert_parallel=(args.mode == "ep"))
        par_loss = [float(eng.step(_packs(args, cfg, s)[rank::world])["loss"]) for s in range(args.steps)]
    worst = max(abs(a - b) for a, b in zip(base_loss, par_loss))
    if cuda:
        from kohakuwullm_b200.ops import native

        torch.cuda.synchronize()
        native.check_status()
    if rank == 0:
        print(json.dumps({"mode": args.mode, "world": world, "baseline_loss": base_loss, "parallel_loss": par_loss,
                          "max_abs_diff": worst, "tol": args.tol, "ok": worst <= args.tol}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0 if worst <= args.tol else 1


if __name__ == "__main__":
    sys.exit(main())
