"""Multi-stream stage boundaries on the pipeline engine: three shapes, each checked for the gradient it is about.

    python -m kohakuwullm_b200.cli.pipe_streams --case aux      # spawns 3 gloo ranks on this machine
    python -m kohakuwullm_b200.cli.pipe_streams --case context
    python -m kohakuwullm_b200.cli.pipe_streams --case skip
    torchrun --nproc-per-node 4 -m kohakuwullm_b200.cli.pipe_streams --case all

* ``aux``      every stage adds a term of its own (an auxiliary loss) to an ACCUMULATOR stream that the last
               stage folds into the loss; each stage's term must reach its parameters with gradient 1, as an
               independent ``.backward()`` of that term would give.
* ``context``  every stage reads the same conditioning tensor (text context of a diffusion transformer), made
               on stage 0 and carried along as a stream; its producer must receive the SUM of all stages' uses.
* ``skip``     an early activation is carried past the middle stages to the last one (U-Net skip); the middle
               stages do not touch it, so on them the stream's gradient is only what comes back from downstream.

Nothing here knows about language models: the stages are three-line MLPs, the boundaries are real (tensors cross
ranks through the schedule's send / receive). Every case compares the gradients of every stage's parameters with
the same model run in one process and ends in a PASS / FAIL line.
Reference: scripts/kohakuwupipe/streams_demo.py, streams_probe.py, train_toy.py.
"""

from __future__ import annotations

import argparse
import os
import sys

import torch
import torch.distributed as dist
from torch import nn

from kohakuwullm_b200.pipe import streams
from kohakuwullm_b200.pipe.schedules import NativeSchedule

DIM, ROWS, MICRO = 16, 6, 4
CASES = ("aux", "context", "skip")


class ToyStage(nn.Module):
    def __init__(self, index: int, n_stages: int, case: str):
        super().__init__()
        torch.manual_seed(100 + index)
        self.index, self.n, self.case = index, n_stages, case
        self.lin = nn.Linear(DIM, DIM)
        if case == "context":
            self.read = nn.Linear(DIM, DIM)           # how this stage uses the context
            if index == 0:
                self.make = nn.Linear(DIM, DIM)       # stage 0 produces it
        if case == "skip" and index == n_stages - 1:
            self.merge = nn.Linear(DIM, DIM)

    def forward(self, x, *extra):
        """First stage: ``x`` is the micro-batch. Returns (hidden, stream) except on the last stage, which
        returns what the loss needs."""
        first, last = self.index == 0, self.index == self.n - 1
        if self.case == "aux":
            acc = streams.accumulator(x.device) if first else extra[0]
            h = torch.tanh(self.lin(x))
            acc = streams.accumulate(acc, 0.01 * h.pow(2).mean())
            return (h, acc)
        if self.case == "context":
            ctx = torch.tanh(self.make(x)) if first else extra[0]
            h = torch.tanh(self.lin(x) + self.read(ctx))
            return (h, ctx)
        skip = torch.tanh(self.lin(x)) if first else extra[0]
        h = skip if first else torch.tanh(self.lin(x))
        if last:
            h = h + self.merge(skip)
        return (h, skip)


def loss_of(case: str, outs, target) -> torch.Tensor:
    h, stream = outs
    main = (h - target).pow(2).sum()
    return main + streams.reduce_accumulator(stream) if case == "aux" else main


def batches(seed: int = 7):
    g = torch.Generator().manual_seed(seed)
    xs = [torch.randn(ROWS, DIM, generator=g) for _ in range(MICRO)]
    ys = [torch.randn(ROWS, DIM, generator=g) for _ in range(MICRO)]
    return xs, ys


def reference_grads(case: str, n_stages: int) -> list[dict]:
    stages = [ToyStage(i, n_stages, case) for i in range(n_stages)]
    xs, ys = batches()
    for x, y in zip(xs, ys):
        cur = (x,)
        for st in stages:
            cur = st(*cur)
        loss_of(case, cur, y).backward()
    return [{k: p.grad.clone() for k, p in st.named_parameters()} for st in stages]


def run_case(case: str, rank: int, world: int) -> bool:
    stage = ToyStage(rank, world, case)
    xs, ys = batches()
    example = (torch.zeros(ROWS, DIM), torch.zeros(1) if case == "aux" else torch.zeros(ROWS, DIM))

    def stage_fn(mb, *inputs):
        return stage(xs[mb]) if rank == 0 else stage(*inputs)

    sched = NativeSchedule(stage_fn, stage_index=rank, num_stages=world, n_micro=MICRO,
                           loss_fn=(lambda outs, mb: loss_of(case, outs, ys[mb])) if rank == world - 1 else None,
                           boundary=() if rank == 0 else example, out_boundary=() if rank == world - 1 else example,
                           kind="1f1b")
    sched.step()
    want = reference_grads(case, world)[rank]
    worst = 0.0
    for k, p in stage.named_parameters():
        if p.grad is None:
            worst = float("inf")
            continue
        worst = max(worst, float((p.grad - want[k]).abs().max() / want[k].abs().max().clamp(min=1e-12)))
    flags = [None] * world
    dist.all_gather_object(flags, worst)
    ok = all(f < 1e-5 for f in flags)
    if rank == 0:
        print(f"{case}: {'PASS' if ok else 'FAIL'} (largest relative gradient error per stage: "
              f"{', '.join(f'{f:.1e}' for f in flags)})", flush=True)
    return ok


def _worker(rank: int, world: int, port: int, cases) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ok = all([run_case(c, rank, world) for c in cases])
    dist.barrier()
    dist.destroy_process_group()
    if not ok:
        raise SystemExit(1)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--case", default="all", choices=CASES + ("all",))
    ap.add_argument("--stages", type=int, default=3, help="ranks to spawn when not started under torchrun")
    ap.add_argument("--port", type=int, default=29631)
    a = ap.parse_args(argv)
    cases = CASES if a.case == "all" else (a.case,)
    if "RANK" in os.environ:                       # started under torchrun: use the ranks that exist
        dist.init_process_group("gloo")
        ok = all([run_case(c, dist.get_rank(), dist.get_world_size()) for c in cases])
        dist.barrier()
        dist.destroy_process_group()
        return 0 if ok else 1
    import torch.multiprocessing as mp

    mp.spawn(_worker, args=(a.stages, a.port, cases), nprocs=a.stages, join=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
