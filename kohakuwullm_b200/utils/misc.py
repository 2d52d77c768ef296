"""Small host-side helpers (imports, parameter counting, number formatting).

Counterpart of the reference's src/kohakuwullm/utils.py:9-81.
"""

from __future__ import annotations

import importlib
from typing import Any


def import_class(path: str) -> Any:
    """Import ``pkg.module.Name`` or ``pkg.module:Name``."""
    if ":" in path:
        module_name, attr = path.split(":", 1)
    else:
        module_name, _, attr = path.rpartition(".")
    if not module_name:
        raise ImportError(f"{path!r} is not a dotted path")
    module = importlib.import_module(module_name)
    obj = module
    for part in attr.split("."):
        obj = getattr(obj, part)
    return obj


def count_parameters(module, trainable_only: bool = False) -> int:
    return sum(p.numel() for p in module.parameters() if p.requires_grad or not trainable_only)


def count_active_parameters(module) -> int:
    """Parameters touched per token.

    A sub-module that processes only part of its weights per token (a routed expert bank)
    declares it by implementing ``active_parameters() -> int``; everything else counts in full.
    """
    total = 0
    claimed: set[int] = set()
    for sub in module.modules():
        fn = getattr(sub, "active_parameters", None)
        if callable(fn) and not any(id(p) in claimed for p in sub.parameters()):
            total += int(fn())
            claimed.update(id(p) for p in sub.parameters())
    total += sum(p.numel() for p in module.parameters() if id(p) not in claimed)
    return total


def human_count(n: float) -> str:
    n = float(n)
    for unit, div in (("T", 1e12), ("B", 1e9), ("M", 1e6), ("K", 1e3)):
        if abs(n) >= div:
            return f"{n / div:.2f}{unit}"
    return f"{n:.0f}"


def autofill_schedule_steps(schedule: dict | None, total_steps: int, warmup_steps: int | None = None) -> dict | None:
    """Fill ``end`` / ``warmup`` of a schedule spec that left them open (``None`` or ``-1``).

    For a composed schedule (``{"phases": [...]}``) the warm-up goes to the first phase and the
    end to the last one.
    """
    if schedule is None:
        return None
    out = dict(schedule)

    def _open(v):
        return v is None or v == -1

    key = "phases" if "phases" in out else ("schedules" if out.get("mode") == "composer" and "schedules" in out else None)
    if key:
        phases = [dict(p) for p in out[key]]
        if _open(out.get("end")):
            out["end"] = total_steps            # what fractional phase ends refer to
        if phases:
            if warmup_steps is not None and "warmup" in phases[0] and _open(phases[0]["warmup"]):
                phases[0]["warmup"] = warmup_steps
            if _open(phases[-1].get("end")):
                phases[-1]["end"] = total_steps
        out[key] = phases
        return out
    if _open(out.get("end")):
        out["end"] = total_steps
    if warmup_steps is not None and "warmup" in out and _open(out["warmup"]):
        out["warmup"] = warmup_steps
    return out
