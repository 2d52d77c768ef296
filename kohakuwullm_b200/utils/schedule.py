"""Learning-rate schedules as plain functions of the step (the role AnySchedule plays in the reference).

A spec is ``{"mode": "cosine"|"linear"|"constant"|"wsd", "warmup": n, "end": total, "min_value": f, ...}`` or a
composition ``{"phases": [spec, ...]}`` where each phase runs until its own ``end``. ``build_schedule``
returns ``f(step) -> multiplier``; ``LambdaLR``-style use: ``lr = base_lr * f(step)``."""

from __future__ import annotations

import math
from typing import Callable


def _single(spec: dict) -> Callable[[int], float]:
    mode = spec.get("mode", "cosine")
    warmup = int(spec.get("warmup", 0) or 0)
    end = int(spec.get("end", 0) or 0)
    lo = float(spec.get("min_value", 0.0))
    hi = float(spec.get("value", 1.0))
    decay_start = int(spec.get("decay_start", end))  # wsd: constant until here, then decay to end

    def f(step: int) -> float:
        if warmup and step < warmup:
            return hi * (step + 1) / warmup
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


def build_schedule(spec: dict | None) -> Callable[[int], float]:
    if not spec:
        return lambda step: 1.0
    if "phases" in spec:
        phases = [(int(p["end"]), _single(p)) for p in spec["phases"]]

        def f(step: int) -> float:
            start = 0
            for end, fn in phases:
                if step < end or end == phases[-1][0]:
                    return fn(step - start) if start else fn(step)
                start = end
            return phases[-1][1](step)

        return f
    return _single(spec)


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
