"""Time the data-parallel gradient step in isolation: fused reduce-scatter + AdamW + all-gather over peer
memory against NCCL all-reduce + unsharded fused AdamW, on a flat parameter set of the flagship's size.

    torchrun --nproc-per-node 8 -m kohakuwullm_b200.bench.ddp_sync --params 546e6

Device-timed (CUDA events, max over ranks), rank 0 prints one JSON line per arm with the bytes that must
cross NVLink per GPU and direction and the fraction of the link roofline:
  reduce-scatter: every rank reads the other W-1 ranks' fp32 gradients of its own 1/W shard;
  all-gather:     every rank's updated bf16 shard is stored into the other W-1 ranks.
Incoming bytes per GPU = (W-1)/W * N * (4 + 2). Roofline time = that / link bandwidth (770 GB/s measured
peer copy on this machine class by default, ``--link-gbs`` to change).
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist
from torch import nn


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--params", type=float, default=546e6)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--link-gbs", type=float, default=770.0)
    args = ap.parse_args(argv)
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from kohakuwullm_b200.parallel.ddp import GradSync
    from kohakuwullm_b200.parallel.flat import FlatParameters
    from kohakuwullm_b200.training.optim.fused_adamw import FlatAdamW

    n = int(args.params)
    rows = n // 4096

    def build():
        torch.manual_seed(0)
        m = nn.Linear(4096, rows, bias=False, device=dev, dtype=torch.bfloat16)
        return m

    def timed(fn):
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(args.steps):
            fn()
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) / args.steps], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    inv = torch.tensor([1.0 / 65536.0], device=dev)
    bytes_in = (world - 1) / world * rows * 4096 * (4 + 2)
    roof_ms = bytes_in / (args.link_gbs * 1e9) * 1e3
    results = []
    # ---- NCCL all-reduce + unsharded AdamW
    m = build()
    flat = FlatParameters(m)
    sync = GradSync(flat)
    opt = FlatAdamW(flat, lr=1e-4)
    coef = torch.ones(1, device=dev)

    def nccl_step():
        for g in flat.groups.values():
            g.main_grad.fill_(1e-3)
        sync.reduce()
        opt.step(grad_scale=coef, zero_grad=True)

    ms = timed(nccl_step)
    results.append({"arm": "nccl all-reduce + AdamW", "ms": ms})
    del m, flat, sync, opt
    torch.cuda.empty_cache()
    # ---- fused
    if world > 1:
        from kohakuwullm_b200.ops import native
        from kohakuwullm_b200.parallel.fused_ddp import FusedGradSync
        from kohakuwullm_b200.parallel.symm import SymmetricPool

        m = build()
        pool = SymmetricPool()
        flat = FlatParameters(m, allocator=pool.empty)
        fsync = FusedGradSync(flat, pool)
        opt = FlatAdamW(flat, lr=1e-4, shard=(rank, world))

        def fused_step():
            for g in flat.groups.values():
                g.main_grad.fill_(1e-3)
            fsync.step(opt, inv, 1.0)

        ms = timed(fused_step)
        torch.cuda.synchronize()
        native.check_status()
        results.append({"arm": "fused reduce-scatter + AdamW + all-gather", "ms": ms})
    # the gradient fill is part of both arms: time it alone and take it off
    m = build()
    flat = FlatParameters(m)
    fill = timed(lambda: [g.main_grad.fill_(1e-3) for g in flat.groups.values()])
    if rank == 0:
        for r in results:
            net = r["ms"] - fill
            print(json.dumps({**r, "n_gpus": world, "params": rows * 4096, "grad_fill_ms": fill, "net_ms": net,
                              "nvlink_bytes_in_per_gpu": bytes_in, "link_roofline_ms": roof_ms,
                              "fraction_of_link_roofline": (roof_ms / net) if net > 0 and world > 1 else None}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
