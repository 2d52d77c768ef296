"""Callbacks of ``LMTrainer``: global-step progress bar, throughput / MFU report, sample previews.
Reference: src/kohakuwullm/training/loop/callbacks.py:13-268."""

from __future__ import annotations

import time

import torch

from kohakuwullm_b200.pipe.hooks import Callback
from kohakuwullm_b200.utils.logging import get_logger

log = get_logger("train")

# dense bf16 tensor peak per GPU, TFLOP/s (used for MFU / HFU); B200 is the nominal dense figure
PEAK_TFLOPS = {"B200": 2250.0, "H100": 989.0, "A100": 312.0, "RTX 5090": 270.0, "RTX 4090": 165.2}


def device_peak_tflops(name: str | None = None) -> float:
    if name is None and torch.cuda.is_available():
        name = torch.cuda.get_device_name()
    for key, val in PEAK_TFLOPS.items():
        if name and key in name:
            return val
    return 0.0


class StepProgressBar(Callback):
    """tqdm bar driven by optimizer steps (not by loader batches)."""

    def __init__(self, total: int | None = None):
        self.total, self.bar = total, None

    def on_train_start(self, trainer):
        if trainer.rank == 0:
            from tqdm import tqdm

            self.bar = tqdm(total=self.total, initial=trainer.global_step, dynamic_ncols=True, desc="train")

    def on_train_batch_end(self, trainer, out, batch, step):
        if self.bar is not None:
            self.bar.update(1)
            if step % 10 == 0 and "loss_host" in out:
                self.bar.set_postfix(loss=f"{out['loss_host']:.4f}")

    def on_train_end(self, trainer):
        if self.bar is not None:
            self.bar.close()


class ThroughputCallback(Callback):
    """Interval and cumulative tokens/s, billions of tokens per day, MFU / HFU against the device peak."""

    def __init__(self, interval: int = 20, peak_tflops: float | None = None, reporter=None):
        self.interval, self.reporter = interval, reporter
        self.peak = (peak_tflops if peak_tflops is not None else device_peak_tflops()) * 1e12
        self._last = None

    def on_train_batch_end(self, trainer, out, batch, step):
        if step % self.interval:
            return
        snap = trainer.snapshot(sync=True)
        if self._last is not None:
            d = snap - self._last
            world = trainer.world
            fields = {"tokens_per_s": d.tokens_per_s, "b_tokens_per_day": d.b_tokens_per_day,
                      "mfu": d.mfu(self.peak * world), "hfu": d.hfu(self.peak * world), "cumulative_tokens_per_s": snap.tokens_per_s}
            log.info("throughput", step=step, **fields)
            if self.reporter:
                self.reporter({f"throughput/{k}": v for k, v in fields.items()}, step)
        self._last = snap


class SampleLogCallback(Callback):
    """Every ``interval`` steps decode a few prompts and log the text (rank 0; collective for pipelines)."""

    def __init__(self, prompts, tokenizer, interval: int = 500, max_new_tokens: int = 64, reporter=None, **sampling):
        self.prompts, self.tok, self.interval, self.max_new, self.reporter = prompts, tokenizer, interval, max_new_tokens, reporter
        self.sampling = sampling or {"temperature": 0.8, "top_p": 0.95}
        self.enabled = True

    def on_train_batch_end(self, trainer, out, batch, step):
        # with the experts split over the ranks a forward is a collective: every rank decodes, rank 0 reports
        collective = bool(getattr(getattr(trainer, "engine", None), "ep_sharded", False))
        if not self.enabled or step % self.interval or (trainer.rank != 0 and not collective):
            return
        try:
            texts = []
            for prompt in self.prompts:
                ids = torch.tensor([self.tok.encode(prompt)], device=trainer.device)
                gen = trainer.generate(ids, self.max_new, **self.sampling)
                texts.append(self.tok.decode(gen[0].tolist()))
            if trainer.rank != 0:
                return
            for p, t in zip(self.prompts, texts):
                log.info("sample", step=step, prompt=p[:40].replace("\n", "\\n"), text=t[:200].replace("\n", "\\n"))
            if self.reporter:
                # a reporter with a ``samples`` method gets a table (step, name, prompt, sample, text); a plain
                # callable gets the texts
                if hasattr(self.reporter, "samples"):
                    self.reporter.samples(step, [("preview", p, i, t) for i, (p, t) in enumerate(zip(self.prompts, texts))])
                else:
                    self.reporter({"samples": texts}, step)
        except NotImplementedError:
            self.enabled = False  # this parallel layout cannot be driven for previews


class ValidationCallback(Callback):
    """Every ``interval`` steps run ``trainer.validate`` over ``max_batches`` batches of a freshly built loader (so every
    validation sees the same held-out batches) and log / report ``val/loss``, ``val/ppl``, ``val/tokens``."""

    def __init__(self, make_loader, interval: int = 500, max_batches: int = 8, reporter=None):
        self.make_loader, self.interval, self.max_batches, self.reporter = make_loader, interval, max_batches, reporter
        self.last: dict = {}

    def on_train_batch_end(self, trainer, out, batch, step):
        if self.interval <= 0 or step % self.interval:
            return
        self.last = trainer.validate(self.make_loader(), self.max_batches)
        if not self.last.get("val/tokens"):
            if trainer.rank == 0 and not getattr(self, "_warned_empty", False):
                log.warning("validation", step=step, message="the held-out split is empty: nothing to validate on")
                self._warned_empty = True
            return
        if trainer.rank == 0:
            log.info("validation", step=step, **self.last)
            if self.reporter:
                self.reporter(dict(self.last), step)
