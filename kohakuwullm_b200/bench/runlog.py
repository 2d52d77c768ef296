"""Per-step CSV of a training run: written with one device->host transfer per flush, read back as arrays, and
judged: step time is quoted only from the part of the run after the first ``TIMING_HEAD`` steps (compilation,
allocator warm-up), needs ``MIN_TIMING_STEPS`` steps, and carries the contention verdict of its own samples.
Reference: src/kohakuwullm/bench/analysis/runlog.py:1-194."""

from __future__ import annotations

import csv
import statistics

from kohakuwullm_b200.bench import contention

COLUMNS = ("step", "tokens", "trained", "loss", "grad_norm", "lr", "elapsed")
HEADER = ",".join(COLUMNS)
TIMING_HEAD = 100
MIN_TIMING_STEPS = 200


def write_step_rows(handle, pending: list[tuple], elapsed_now: float) -> tuple:
    """``pending``: rows in ``COLUMNS`` order (``tokens``: cumulative tokens seen; ``trained``: trained tokens of
    that step) whose loss (a SUM over the step's trained tokens) and grad norm are still device tensors. All of them come to the host in one stacked transfer; the last row's timestamp becomes
    ``elapsed_now`` (the only moment the host knows the device has caught up). Returns that row's
    ``(loss per token, grad_norm, elapsed)``."""
    import torch

    if not pending:
        return (0.0, 0.0, elapsed_now)
    as_t = lambda v: v.detach().float().reshape(()) if torch.is_tensor(v) else torch.tensor(float(v))  # noqa: E731
    scalars = torch.stack([as_t(r[3]) for r in pending] + [as_t(r[4]) for r in pending]).tolist()
    half = len(pending)
    last = (0.0, 0.0, elapsed_now)
    for i, row in enumerate(pending):
        step, tokens, trained, _, _, lr, elapsed = row
        per_token = scalars[i] / max(trained, 1)
        gnorm = scalars[half + i]
        if i == half - 1:
            elapsed = elapsed_now
            last = (per_token, gnorm, elapsed_now)
        handle.write(f"{step},{tokens},{trained},{per_token:.8f},{gnorm:.6f},{lr:.8e},{elapsed:.3f}\n")
    handle.flush()
    return last


def load_run(path: str) -> dict[str, list]:
    with open(path) as fh:
        rows = list(csv.DictReader(fh))
    if not rows:
        raise ValueError(f"{path} has no rows")
    missing = [c for c in COLUMNS if c not in rows[0]]
    if missing:
        raise ValueError(f"{path} lacks columns {missing}")
    out: dict[str, list] = {c: [] for c in COLUMNS}
    for r in rows:
        for c in COLUMNS:
            out[c].append(int(r[c]) if c in ("step", "tokens", "trained") else float(r[c]))
    return out


def step_times(run: dict[str, list]) -> list[float]:
    """Seconds per step from the elapsed column, head excluded. Rows flushed together share a timestamp, so the
    time of a flush interval is spread evenly over its steps."""
    steps, elapsed = run["step"], run["elapsed"]
    out: list[float] = []
    i = 0
    while i < len(steps) - 1:
        j = i + 1
        while j < len(steps) - 1 and elapsed[j] == elapsed[i]:
            j += 1
        span, n = elapsed[j] - elapsed[i], steps[j] - steps[i]
        if n > 0 and span > 0 and steps[j] > TIMING_HEAD:
            out.extend([span / n] * n)
        i = j
    return out


def clock_verdict(run: dict[str, list]) -> dict:
    times = step_times(run)
    if len(times) < MIN_TIMING_STEPS:
        return {"admissible": False, "why": f"only {len(times)} timed steps after the first {TIMING_HEAD}; "
                                            f"{MIN_TIMING_STEPS} are needed", "n": len(times)}
    med = statistics.median(times)
    frac = contention.contended_fraction(times)
    tokens = run["tokens"]
    per_step = (tokens[-1] - tokens[0]) / max(len(tokens) - 1, 1)
    return {"admissible": frac <= contention.CONTENDED_LIMIT, "median_s": med, "contended_fraction": frac,
            "tokens_per_s": per_step / med if med else float("nan"), "n": len(times),
            "why": "" if frac <= contention.CONTENDED_LIMIT else f"{frac:.2%} of steps ran over 1.1x the median: shared card"}
