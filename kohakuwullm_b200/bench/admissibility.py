"""May a measurement be quoted? Sample loops that carry their own contention verdict, the split of a
wall-clock time into host enqueue and device work, and the notes a result row gets when one of its arms was
measured on a shared card or is dominated by host time. Reference: src/kohakuwullm/bench/analysis/admissibility.py:1-61."""

from __future__ import annotations

import os
import statistics

from kohakuwullm_b200.bench import contention
from kohakuwullm_b200.bench.timing import HOST_SHARE_LIMIT, bench_samples, cpu_enqueue_ms, graph_ms


def median_and_contention(fn, iters: int | None = None, flush: bool = True) -> tuple[float, float, bool]:
    """Median device ms, contended fraction and whether that verdict has power, from ONE sample loop."""
    need = contention.contended_fraction_min_iters()
    iters = iters or need
    if iters < need:
        raise ValueError(f"iters={iters} cannot resolve a {contention.CONTENDED_LIMIT:.0%} contended-fraction limit; "
                         f"needs {need}")
    samples = bench_samples(fn, repeats=iters, flush=flush)
    med = statistics.median(samples)
    return med, contention.contended_fraction(samples), contention.spread_has_power(med)


def net_and_graph(fn, graph_iters: int = 30) -> dict:
    """Device time net of host enqueue, graph-replay time, and the host share of the eager time."""
    wall, frac, power = median_and_contention(fn)
    host = cpu_enqueue_ms(fn)
    return {"wall_ms": wall, "host_ms": host, "net_ms": wall - host, "graph_ms": graph_ms(fn, replays=graph_iters),
            "host_share": host / wall if wall else float("nan"), "contended_fraction": frac, "has_power": power}


def contention_notes(row: dict, keys: tuple[str, ...], certifiable: bool) -> list[str]:
    if not certifiable:
        return ["too short to certify exclusivity; not a clean verdict"]
    return [f"{k}={row[k]:.2%}: card was shared, discard this row" for k in keys if row[k] > contention.CONTENDED_LIMIT]


def suspect_speedup(row: dict, keys: tuple[str, ...]) -> str:
    """Why a row's RATIO is not evidence although its own number may be: a shared baseline arm, or a baseline
    whose time is mostly host enqueue (its 'net' time is then a difference of two noisy numbers)."""
    notes = []
    for k in keys:
        if k.startswith("contended") and row[k] > contention.CONTENDED_LIMIT:
            notes.append(f"{k}={row[k]:.2%}: baseline arm was shared")
        if k.startswith("host_share") and row[k] > HOST_SHARE_LIMIT:
            notes.append(f"{k}={row[k]:.0%}: baseline net time is not evidence")
    return "; ".join(notes)


def visible_devices() -> str:
    return os.environ.get("CUDA_VISIBLE_DEVICES", "<unset: device 0 of the process>")
