"""Stock callbacks of the pipeline trainer. None of them reads a device tensor except on its own
interval, so the step loop stays free of host synchronisation.
Reference: src/kohakuwupipe/training/callbacks.py:20-253.
"""

from __future__ import annotations

import math
import os
import time

import torch

from kohakuwullm_b200.pipe.hooks import Callback
from kohakuwullm_b200.utils.logging import get_logger

log = get_logger("pipe")


class Throughput(Callback):
    """Tokens/s over a trailing window; synchronises the device only when it reports."""

    def __init__(self, interval: int = 10, window: int = 50, reporter=None):
        self.interval, self.window, self.reporter = interval, window, reporter
        self._marks: list[tuple[float, int]] = []
        self.last: float | None = None

    def on_train_batch_end(self, loop, out, batch, step):
        if step % self.interval:
            return
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        self._marks.append((time.perf_counter(), loop.tokens_seen))
        self._marks = self._marks[-max(2, self.window // self.interval + 1):]
        if len(self._marks) >= 2:
            (t0, n0), (t1, n1) = self._marks[0], self._marks[-1]
            self.last = (n1 - n0) / max(t1 - t0, 1e-9)
            log.info("throughput", step=step, tokens_per_s=self.last, b_tokens_per_day=self.last * 86400 / 1e9)
            if self.reporter:
                self.reporter({"throughput/tokens_per_s": self.last}, step)


class LossLog(Callback):
    """Loss, its EMA and the learning rate, read from the device every ``interval`` steps."""

    def __init__(self, interval: int = 10, ema: float = 0.98, reporter=None):
        self.interval, self.beta, self.reporter = interval, ema, reporter
        self.ema: float | None = None
        self.history: list[tuple[int, float]] = []

    def on_train_batch_end(self, loop, out, batch, step):
        if step % self.interval:
            return
        loss = float(out.loss)
        if math.isfinite(loss):
            self.ema = loss if self.ema is None else self.beta * self.ema + (1 - self.beta) * loss
        self.history.append((step, loss))
        lr = loop.optimizer.param_groups[0]["lr"] if hasattr(loop.optimizer, "param_groups") else float("nan")
        extra = {k: float(v) for k, v in out.extra.items()}
        log.info("train", step=step, loss=loss, loss_ema=self.ema, lr=lr, skipped=out.skipped, **extra)
        if self.reporter:
            self.reporter({"train/loss": loss, "train/loss_ema": self.ema, "train/lr": lr}, step)

    def state_dict(self):
        return {"ema": self.ema}

    def load_state_dict(self, state):
        self.ema = state.get("ema")


class ProgressBar(Callback):
    def __init__(self, total: int | None = None):
        self.total, self.bar = total, None

    def on_train_start(self, loop):
        if loop.rank == 0:
            from tqdm import tqdm

            self.bar = tqdm(total=self.total, initial=loop.global_step, dynamic_ncols=True)

    def on_train_batch_end(self, loop, out, batch, step):
        if self.bar is not None:
            self.bar.update(1)

    def on_train_end(self, loop):
        if self.bar is not None:
            self.bar.close()


class Checkpoint(Callback):
    """``step-N.ckpt`` every ``every`` steps plus ``last.ckpt``; saving goes through the trainer so every
    rank takes part in the gather."""

    def __init__(self, trainer, directory: str, every: int = 1000, keep_last: bool = True):
        self.trainer, self.directory, self.every, self.keep_last = trainer, directory, every, keep_last

    def on_train_batch_end(self, loop, out, batch, step):
        if self.every and step % self.every == 0:
            self.trainer.save_checkpoint(os.path.join(self.directory, f"step-{step}.ckpt"))
            if self.keep_last:
                self.trainer.save_checkpoint(os.path.join(self.directory, "last.ckpt"))

    def on_exception(self, loop, exc):
        log.error("exception", kind=type(exc).__name__, message=str(exc)[:200], step=loop.global_step)
