"""Seam measurements for pipeline planning: the cost of one hop between neighbouring ranks.

``hop_cost`` sends a tensor of ``nbytes`` around the ring (rank r -> r+1) ``repeats`` times and reports
the median time per hop and the resulting bandwidth; ``SyntheticStage`` is a stage that burns a fixed
amount of matmul time, for schedule experiments without a model.
Reference: src/kohakuwupipe/bench/latency.py:22-120.
"""

from __future__ import annotations

import statistics
import time

import torch
import torch.distributed as dist


def hop_cost(nbytes: int, device, repeats: int = 20, warmup: int = 3, group=None) -> dict:
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    n = max(nbytes // 2, 1)
    send = torch.ones(n, dtype=torch.bfloat16, device=device)
    recv = torch.empty_like(send)
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    samples = []
    for i in range(warmup + repeats):
        if device.type == "cuda":
            torch.cuda.synchronize(device)
        dist.barrier(group=group)
        t0 = time.perf_counter()
        ops = [dist.P2POp(dist.isend, send, nxt, group), dist.P2POp(dist.irecv, recv, prv, group)]
        for w in dist.batch_isend_irecv(ops):
            w.wait()
        if device.type == "cuda":
            torch.cuda.synchronize(device)
        if i >= warmup:
            samples.append(time.perf_counter() - t0)
    sec = statistics.median(samples)
    return {"bytes": n * 2, "seconds": sec, "gb_per_s": n * 2 / sec / 1e9}


class SyntheticStage(torch.nn.Module):
    """Identity on the hidden state after ``flops`` of matmul work (forward) and twice that (backward)."""

    def __init__(self, dim: int, layers: int):
        super().__init__()
        self.weights = torch.nn.ParameterList(torch.nn.Parameter(torch.eye(dim)) for _ in range(layers))

    def forward(self, x):
        for w in self.weights:
            x = x @ w
        return x


def overlap(compute_s: float, hop_s: float) -> float:
    """Fraction of a hop hidden behind one micro-batch of compute."""
    return 1.0 if hop_s <= 0 else min(1.0, compute_s / hop_s)


def roofline(nbytes: int, link_gb_per_s: float = 770.0) -> float:
    """Seconds a boundary of ``nbytes`` needs at the measured NVLink peer-copy bandwidth."""
    return nbytes / (link_gb_per_s * 1e9)
