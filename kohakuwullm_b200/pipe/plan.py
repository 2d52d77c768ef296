"""Stage planning: split ``depth`` layers into contiguous pipeline stages by cost.

``partition`` is an exact dynamic program over contiguous cuts. It minimises, lexicographically,
(1) the cost of the most expensive stage and (2) the sum of squared per-stage parameter counts (so
among equally fast splits memory is spread evenly). The first stage also carries the embedding, the
last one the head; ``allow_empty_last`` lets the last stage hold the head only. ``partition_v`` plans
``2 * ranks`` chunks folded in a V (rank r runs chunks r and 2R-1-r; rank 0 holds embedding and head)
by binary search on the per-rank cost ceiling. Reference: src/kohakuwupipe/parallel/plan.py:10-257.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence


@dataclass(frozen=True)
class StagePlan:
    index: int
    num_stages: int
    start_layer: int
    end_layer: int
    cost: float = 0.0

    @property
    def num_layers(self) -> int:
        return self.end_layer - self.start_layer

    @property
    def is_first(self) -> bool:
        return self.index == 0

    @property
    def is_last(self) -> bool:
        return self.index == self.num_stages - 1

    def owns(self, layer: int) -> bool:
        return self.start_layer <= layer < self.end_layer


def _prefix(xs: Sequence[float]) -> list[float]:
    out = [0.0]
    for x in xs:
        out.append(out[-1] + x)
    return out


def partition(layer_costs: Sequence[float], num_stages: int, *, embed_cost: float = 0.0, head_cost: float = 0.0,
              layer_params: Sequence[float] | None = None, embed_params: float = 0.0, head_params: float = 0.0,
              allow_empty_last: bool = False) -> list[tuple[int, int]]:
    """Contiguous ``[start, end)`` ranges, one per stage."""
    n = len(layer_costs)
    if num_stages < 1:
        raise ValueError("num_stages must be >= 1")
    min_layers = num_stages - (1 if allow_empty_last else 0)
    if n < min_layers:
        raise ValueError(f"{n} layers cannot fill {num_stages} stages")
    params = list(layer_params) if layer_params is not None else [1.0] * n
    pc, pp = _prefix(layer_costs), _prefix(params)

    def stage(s: int, a: int, b: int) -> tuple[float, float]:
        cost, par = pc[b] - pc[a], pp[b] - pp[a]
        if s == 0:
            cost, par = cost + embed_cost, par + embed_params
        if s == num_stages - 1:
            cost, par = cost + head_cost, par + head_params
        return cost, par

    INF = (float("inf"), float("inf"))
    # best[s][b]: best (max cost, sum par^2) using stages 0..s for layers [0, b)
    best = [[INF] * (n + 1) for _ in range(num_stages)]
    cut = [[0] * (n + 1) for _ in range(num_stages)]
    for b in range(n + 1):
        if b >= 1 or (num_stages == 1 and allow_empty_last):
            c, p = stage(0, 0, b)
            best[0][b] = (c, p * p)
    for s in range(1, num_stages):
        last = s == num_stages - 1
        for b in range(s, n + 1):
            for a in range(s, b + 1):
                if a == b and not (last and allow_empty_last):
                    continue
                prev = best[s - 1][a]
                if prev == INF:
                    continue
                c, p = stage(s, a, b)
                cand = (max(prev[0], c), prev[1] + p * p)
                if cand < best[s][b]:
                    best[s][b] = cand
                    cut[s][b] = a
    if best[num_stages - 1][n] == INF:
        raise ValueError("no feasible partition")
    bounds, b = [], n
    for s in range(num_stages - 1, 0, -1):
        a = cut[s][b]
        bounds.append((a, b))
        b = a
    bounds.append((0, b))
    return bounds[::-1]


def partition_v(layer_costs: Sequence[float], num_ranks: int, *, embed_cost: float = 0.0,
                head_cost: float = 0.0) -> list[tuple[int, int]]:
    """``2 * num_ranks`` contiguous chunks; chunk c runs on rank ``c`` (going down) or ``2R-1-c`` (coming
    back up). Minimises the largest per-rank cost by binary search on the ceiling."""
    n, chunks = len(layer_costs), 2 * num_ranks
    if n < chunks:
        raise ValueError(f"{n} layers cannot fill {chunks} V-chunks")

    def rank_of(c: int) -> int:
        return c if c < num_ranks else chunks - 1 - c

    def feasible(ceiling: float):
        load = [0.0] * num_ranks
        load[0] = embed_cost + head_cost
        bounds, start = [], 0
        for c in range(chunks):
            r = rank_of(c)
            remaining_chunks = chunks - c - 1
            end = start + 1  # every chunk takes at least one layer
            acc = layer_costs[start]
            if load[r] + acc > ceiling:
                return None
            while end < n - remaining_chunks and load[r] + acc + layer_costs[end] <= ceiling:
                acc += layer_costs[end]
                end += 1
            if c == chunks - 1:
                if end < n:
                    extra = sum(layer_costs[end:])
                    if load[r] + acc + extra > ceiling:
                        return None
                    end = n
            load[r] += acc if c < chunks - 1 else sum(layer_costs[start:end])
            bounds.append((start, end))
            start = end
        return bounds if start == n else None

    lo, hi = max(layer_costs), sum(layer_costs) + embed_cost + head_cost
    best = feasible(hi)
    for _ in range(60):
        mid = (lo + hi) / 2
        got = feasible(mid)
        if got is not None:
            best, hi = got, mid
        else:
            lo = mid
    if best is None:
        raise ValueError("no feasible V partition")
    return best


def plan_stages(layer_costs: Sequence[float], num_stages: int, style: str = "loop", **kw) -> list[StagePlan]:
    if style == "v":
        bounds = partition_v(layer_costs, num_stages // 2, embed_cost=kw.get("embed_cost", 0.0),
                             head_cost=kw.get("head_cost", 0.0))
    else:
        bounds = partition(layer_costs, num_stages, **kw)
    pc = _prefix(layer_costs)
    plans = []
    for i, (a, b) in enumerate(bounds):
        cost = pc[b] - pc[a]
        if i == 0:
            cost += kw.get("embed_cost", 0.0)
        if i == len(bounds) - 1:
            cost += kw.get("head_cost", 0.0)
        plans.append(StagePlan(i, len(bounds), a, b, cost))
    return plans


def plan_from_layers(layers_per_stage: Sequence[int]) -> list[StagePlan]:
    """Explicit split, e.g. ``[5, 4, 4, 3]``."""
    plans, start = [], 0
    for i, n in enumerate(layers_per_stage):
        plans.append(StagePlan(i, len(layers_per_stage), start, start + n, float(n)))
        start += n
    return plans


def describe(plans: Sequence[StagePlan]) -> str:
    worst = max((p.cost for p in plans), default=0.0) or 1.0
    rows = [f"stage {p.index}: layers [{p.start_layer}, {p.end_layer})  n={p.num_layers}  "
            f"cost={p.cost:.3f} ({100 * p.cost / worst:.0f}% of max)" for p in plans]
    return "\n".join(rows)
