"""Learning-rate schedules as plain functions of the step (the role AnySchedule plays in the reference).

A spec is a dict; ``build_schedule(spec)`` returns ``f(step) -> multiplier`` (``lr = base_lr * f(step)``).

Single schedules, ``{"mode": ..., "warmup": n, "end": total, "value": 1.0, "min_value": 0.0, ...}``: the first
``warmup`` steps ramp linearly up to ``value``, then the mode takes over until ``end`` and holds its last value:

=============  =========================================================================================
``constant``   ``value``
``linear``     straight line from ``value`` to ``min_value`` at ``end``
``cosine``     half cosine from ``value`` to ``min_value`` at ``end``
``wsd``        ``value`` until ``decay_start``, then a straight line to ``min_value`` at ``end``
``power``      ``value * (max(step, s0) / s0) ** b``: flat for ``s0`` steps, then a power law (``b = -0.5`` is the
               inverse-square-root decay); never below ``min_value``
``exponential`` ``value * 0.5 ** (step / half_life)``, never below ``min_value``
=============  =========================================================================================

Compositions, ``{"phases": [spec, ...]}`` (``{"mode": "composer", "schedules": [...], "end": total}`` is read the
same way): phase i runs from the previous phase's ``end`` to its own. A phase's ``end`` is an absolute step, or a
fraction of the composition's ``end`` when it is a float in (0, 1]. Inside a phase the step counts from the phase's
start, and the phase's output is multiplied by the value the previous phase ended on, so the curve is continuous
(a power-law phase followed by a cosine tail starts the tail where the power law stopped).
"""

from __future__ import annotations

import math
from typing import Callable

MODES = ("constant", "linear", "cosine", "wsd", "power", "exponential")


def _single(spec: dict) -> Callable[[int], float]:
    mode = spec.get("mode", "cosine")
    if mode not in MODES:
        raise ValueError(f"unknown schedule mode {mode!r}; known: {', '.join(MODES)}")
    warmup = int(spec.get("warmup", 0) or 0)
    end = int(spec.get("end", 0) or 0)
    lo = float(spec.get("min_value", 0.0))
    hi = float(spec.get("value", 1.0))
    decay_start = int(spec.get("decay_start", end))  # wsd: constant until here, then decay to end
    s0 = max(float(spec.get("s0", 1.0)), 1.0)
    b = float(spec.get("b", -0.5))
    half_life = max(float(spec.get("half_life", 1.0)), 1e-9)

    def f(step: int) -> float:
        if warmup and step < warmup:
            return hi * (step + 1) / warmup
        if mode == "power":
            return max(lo, hi * (max(float(min(step, end) if end else step), s0) / s0) ** b)
        if mode == "exponential":
            return max(lo, hi * 0.5 ** ((min(step, end) if end else step) / half_life))
        if mode == "constant" or end <= warmup:
            return hi
        if mode == "wsd":
            if step < decay_start:
                return hi
            t = min(1.0, (step - decay_start) / max(end - decay_start, 1))
            return lo + (hi - lo) * (1 - t)
        t = min(1.0, (step - warmup) / max(end - warmup, 1))
        if mode == "linear":
            return lo + (hi - lo) * (1 - t)
        return lo + (hi - lo) * 0.5 * (1 + math.cos(math.pi * t))

    return f


def _phase_ends(phases: list[dict], total: int | None) -> list[int]:
    ends = []
    for p in phases:
        e = p.get("end")
        if isinstance(e, float) and 0.0 < e <= 1.0:
            if not total or total <= 0:
                raise ValueError("a fractional phase end needs the composition's own 'end'")
            e = int(round(e * total))
        frac = isinstance(p.get("end"), float) and 0.0 < p["end"] <= 1.0
        last = ends[-1] if ends else 0
        if e is None or int(e) < last or (int(e) == last and not frac):
            raise ValueError(f"phase ends must be given and increase, got {[q.get('end') for q in phases]}")
        ends.append(int(e))        # a fractional end may round onto the previous one in a very short run: an empty phase
    return ends


def build_schedule(spec: dict | None) -> Callable[[int], float]:
    if not spec:
        return lambda step: 1.0
    phases = spec.get("phases", spec.get("schedules") if spec.get("mode") == "composer" else None)
    if phases is None:
        return _single(spec)
    phases = [dict(p) for p in phases]
    if not phases:
        return lambda step: 1.0
    total = spec.get("end")
    ends = _phase_ends(phases, int(total) if isinstance(total, (int, float)) and total and total > 0 else None)
    starts = [0] + ends[:-1]
    keep = [i for i, (a, b) in enumerate(zip(starts, ends)) if b > a]          # phases that rounding left empty drop out
    phases, starts, ends = [phases[i] for i in keep], [starts[i] for i in keep], [ends[i] for i in keep]
    fns = [_single({**p, "end": e - s}) for p, s, e in zip(phases, starts, ends)]
    carry = [1.0]                       # value the previous phases ended on
    for fn, s, e in zip(fns[:-1], starts, ends):
        carry.append(carry[-1] * fn(e - s))

    def f(step: int) -> float:
        for i, e in enumerate(ends):
            if step < e or i == len(ends) - 1:
                return carry[i] * fns[i](step - starts[i])
        raise AssertionError("unreachable")

    return f


class GroupLRSchedule:
    """A scheduler object for the training loops (``step`` / ``state_dict`` / ``load_state_dict``): after every
    optimizer step each parameter group's rate becomes its OWN base rate times ``fn(step)``, so groups with
    different base rates (Muon, embedding, muP groups) keep their ratios. Works on anything with ``param_groups``."""

    def __init__(self, optimizer, fn: Callable[[int], float]):
        self.optimizer, self.fn, self.step_count = optimizer, fn, 0
        self.base = [g["lr"] for g in optimizer.param_groups]
        self._apply()

    def _apply(self) -> None:
        f = float(self.fn(self.step_count))
        for g, base in zip(self.optimizer.param_groups, self.base):
            g["lr"] = base * f

    def step(self) -> None:
        self.step_count += 1
        self._apply()

    def state_dict(self) -> dict:
        return {"step": self.step_count, "base": list(self.base)}

    def load_state_dict(self, state: dict) -> None:
        self.step_count = int(state.get("step", 0))
        if state.get("base") and len(state["base"]) == len(self.base):
            self.base = list(state["base"])
        self._apply()
