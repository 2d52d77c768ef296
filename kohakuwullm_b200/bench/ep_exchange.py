"""Time the expert-parallel token exchange in isolation: dispatch (token rows into the owners' receive buffers) and
return (result rows back to the source ranks and the weighted sum per token), without the expert GEMMs between them.

    torchrun --nproc-per-node 8 -m kohakuwullm_b200.bench.ep_exchange --tokens 8192 --dim 1024 --experts 64 --top-k 6

Routing is uniform over the experts (seeded, a different draw per rank), so a fraction (W-1)/W of every rank's
(token, expert) pairs lives on another rank. Device-timed (CUDA events on the launching stream, max over ranks). Per GPU
and direction the bytes that must cross NVLink are

    dispatch:  pairs_remote x dim x 2   (bf16 rows stored into the owners)
    return:    pairs_remote x dim x 2   (bf16 result rows read back from the owners)

and the roofline time of each phase is that divided by the link bandwidth (770 GB/s measured peer copy on this
machine class by default, ``--link-gbs`` to change). Rank 0 prints one JSON line with the achieved fractions, and, for
comparison, the same exchange done with ``all_to_all_single`` on NCCL over pre-sorted rows.
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--dim", type=int, default=1024)
    ap.add_argument("--experts", type=int, default=64)
    ap.add_argument("--top-k", type=int, default=6)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--link-gbs", type=float, default=770.0)
    args = ap.parse_args(argv)
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29534")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from kohakuwullm_b200.ops import native
    from kohakuwullm_b200.parallel.ep import ExpertParallel

    T, D, E, k = args.tokens, args.dim, args.experts, args.top_k
    El = E // world
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    x = torch.randn(T, D, device=dev, generator=g).bfloat16()
    idx = torch.stack([torch.randperm(E, device=dev, generator=g)[:k] for _ in range(T)]).to(torch.int32)
    w = torch.full((T * k,), 1.0 / k, device=dev)
    counts = torch.bincount(idx.reshape(-1).long(), minlength=E).to(torch.int32)
    remote = int(((idx // El) != rank).sum())
    ep = ExpertParallel(capacity_factor=2.0)

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
        ms = torch.tensor([s.elapsed_time(e) / args.steps], device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms)

    plan = ep.plan(idx, counts, D)
    state = {}

    def dispatch():
        plan.cursors.zero_()
        ep._push_rows(x, plan)
        state["rows"] = ep._take_received(plan, D)

    def giveback():
        if ep._publish_rows(state["rows"], plan):
            ep._sum_pairs(plan, w, T, D, keep=False)
        else:
            ep._pull(plan, w, T, D, keep=False)

    t_plan = timed(lambda: ep.plan(idx, counts, D))
    plan = ep.plan(idx, counts, D)
    t_disp = timed(dispatch)
    dispatch()
    t_back = timed(giveback)
    native.check_status()

    # NCCL reference: rows pre-sorted by owner, split sizes known: all_to_all_single there and back
    owner = (idx.reshape(-1) // El).long()
    order = torch.argsort(owner, stable=True)
    send = x.repeat_interleave(k, 0)[order].contiguous()
    in_split = torch.bincount(owner, minlength=world).tolist()
    out_split_t = torch.tensor(in_split, device=dev)
    gathered = [torch.zeros_like(out_split_t) for _ in range(world)]
    dist.all_gather(gathered, out_split_t)
    out_split = [int(t[rank]) for t in gathered]
    recv = torch.empty(sum(out_split), D, dtype=torch.bfloat16, device=dev)
    back = torch.empty_like(send)
    t_nccl_there = timed(lambda: dist.all_to_all_single(recv, send, out_split, in_split))
    t_nccl_back = timed(lambda: dist.all_to_all_single(back, recv, in_split, out_split))

    nbytes = remote * D * 2.0
    worst = torch.tensor([nbytes], device=dev)
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    roof_ms = float(worst) / (args.link_gbs * 1e9) * 1e3
    if rank == 0:
        print(json.dumps({"n_gpus": world, "tokens": T, "dim": D, "experts": E, "top_k": k, "pairs": T * k,
                          "remote_pairs_max": int(float(worst) / (D * 2)), "bytes_per_direction": float(worst),
                          "roofline_ms_per_phase": roof_ms,
                          "plan_ms": t_plan, "dispatch_ms": t_disp, "return_ms": t_back,
                          "dispatch_frac_of_link_roofline": roof_ms / t_disp, "return_frac_of_link_roofline": roof_ms / t_back,
                          "nccl_all_to_all_there_ms": t_nccl_there, "nccl_all_to_all_back_ms": t_nccl_back,
                          "note": "dispatch = scatter rows + flag barrier + copy into private rows with zeroed padding; "
                                  "return = publish + flag barrier + weighted gather-sum per token; the NCCL arms move "
                                  "pre-sorted rows only (no sort, no gather-sum)"}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
