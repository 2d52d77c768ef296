"""Metric sinks for the trainers' callbacks: a callable ``reporter(row, step)`` on rank 0, no-op elsewhere.

* ``WandbReporter``   a Weights & Biases run (``mode="offline"`` by default: these machines have no network; an
                      offline run directory can be synced later). Scalars go to ``run.log``; generated samples go
                      to a ``wandb.Table`` with the columns step / name / prompt / sample / text and never to the
                      console log.
* ``JsonlReporter``   one JSON object per report in a file (what the offline analysis tools read).
* ``ConsoleReporter`` the structured logger, every ``interval`` steps.
* ``MultiReporter``   fans a report out to several sinks.

Every sink adds ``ppl = exp(min(loss, 20))`` when the row has a float ``train/loss`` or ``loss`` (the trainers
report the loss; perplexity is the language model's own metric).
Reference: scripts/train/lm_pipe.py:262-322 (the run, the reporter pair); scripts/train/lm.py:402 (WandbLogger).
"""

from __future__ import annotations

import json
import math
import os
import time
from typing import Any, Sequence

from kohakuwullm_b200.utils.logging import get_logger

log = get_logger("metrics")


def _is_rank0() -> bool:
    try:
        import torch.distributed as dist

        return not (dist.is_available() and dist.is_initialized()) or dist.get_rank() == 0
    except Exception:  # noqa: BLE001
        return True


def _plain(v: Any) -> Any:
    """Device scalars and numpy numbers -> Python numbers (one host read per value, on the reporting interval)."""
    if hasattr(v, "item") and getattr(v, "numel", lambda: 1)() == 1:
        return v.item()
    return v


def with_perplexity(row: dict) -> dict:
    for key in ("train/loss", "loss"):
        val = row.get(key)
        if isinstance(val, float) and math.isfinite(val):
            return dict(row, **{key.replace("loss", "ppl"): math.exp(min(val, 20.0))})
    return row


class Reporter:
    """Base: ``__call__(row, step)`` for scalars, ``samples(step, rows)`` for generated text, ``finish()``."""

    def __call__(self, row: dict, step: int | None = None) -> None:
        if not _is_rank0():
            return
        step = int(row.get("step", 0)) if step is None else int(step)
        clean = with_perplexity({k: _plain(v) for k, v in row.items() if k != "step"})
        self.write(clean, step)

    def write(self, row: dict, step: int) -> None:
        raise NotImplementedError

    def samples(self, step: int, rows: Sequence[tuple]) -> None:
        """``rows``: (name, prompt, sample index, text)."""

    def finish(self) -> None:
        pass


class WandbReporter(Reporter):
    def __init__(self, project: str, name: str | None = None, config: dict | None = None, mode: str = "offline",
                 run_id: str | None = None, directory: str | None = None):
        self.run = None
        if not _is_rank0():
            return
        import wandb

        if directory:
            os.makedirs(directory, exist_ok=True)
        self.run = wandb.init(project=project, name=name, config=config or {}, mode=mode, id=run_id or None,
                              resume="must" if run_id else None, dir=directory)

    @property
    def run_id(self) -> str | None:
        return getattr(self.run, "id", None)

    def write(self, row: dict, step: int) -> None:
        if self.run is not None:
            self.run.log(row, step=step)

    def samples(self, step: int, rows: Sequence[tuple]) -> None:
        if self.run is None:
            return
        import wandb

        table = wandb.Table(columns=["step", "name", "prompt", "sample", "text"])
        for name, prompt, index, text in rows:
            table.add_data(step, name, prompt, index, text)
        self.run.log({"samples": table}, step=step)

    def finish(self) -> None:
        if self.run is not None:
            self.run.finish()
            self.run = None


class JsonlReporter(Reporter):
    def __init__(self, path: str):
        self.path = path
        if _is_rank0():
            os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        self._t0 = time.time()

    def write(self, row: dict, step: int) -> None:
        with open(self.path, "a") as fh:
            fh.write(json.dumps({"step": step, "t": round(time.time() - self._t0, 3), **row}, default=str) + "\n")

    def samples(self, step: int, rows: Sequence[tuple]) -> None:
        if _is_rank0():
            with open(self.path, "a") as fh:
                fh.write(json.dumps({"step": step, "samples": [list(r) for r in rows]}, default=str) + "\n")


class ConsoleReporter(Reporter):
    def __init__(self, interval: int = 100):
        self.interval = max(int(interval), 1)

    def write(self, row: dict, step: int) -> None:
        if step % self.interval == 0:
            log.info("metrics", step=step, **{k: v for k, v in row.items() if isinstance(v, (int, float, str))})


class MultiReporter(Reporter):
    def __init__(self, *sinks: Reporter):
        self.sinks = [s for s in sinks if s is not None]

    def __call__(self, row: dict, step: int | None = None) -> None:
        for s in self.sinks:
            s(row, step)

    def samples(self, step: int, rows: Sequence[tuple]) -> None:
        for s in self.sinks:
            s.samples(step, rows)

    def finish(self) -> None:
        for s in self.sinks:
            s.finish()


def build_reporter(wandb_project: str | None = None, name: str | None = None, config: dict | None = None,
                   jsonl: str | None = None, console_interval: int = 0, wandb_mode: str = "offline",
                   run_id: str | None = None, directory: str | None = None) -> Reporter | None:
    """The sinks a training script asks for, as one reporter (None when it asks for none)."""
    sinks: list[Reporter] = []
    if wandb_project:
        sinks.append(WandbReporter(wandb_project, name, config, wandb_mode, run_id, directory))
    if jsonl:
        sinks.append(JsonlReporter(jsonl))
    if console_interval > 0:
        sinks.append(ConsoleReporter(console_interval))
    if not sinks:
        return None
    return sinks[0] if len(sinks) == 1 else MultiReporter(*sinks)
