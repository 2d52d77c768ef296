"""Rank-aware structured logging: ``log.info("event", key=value, ...)``.

Only rank 0 prints unless ``KWP_LOG_ALL_RANKS=1``. Reference: src/kohakuwupipe/utils/logging.py:30-119.
"""

from __future__ import annotations

import logging
import os
import sys
import time

_configured = False
_muted = False     # this rank prints nothing (every rank but 0, unless all ranks are asked for)


def _rank() -> int:
    return int(os.environ.get("RANK", "0"))


def configure(level: str | int = "INFO", stream=None, all_ranks: bool | None = None) -> None:
    global _configured, _muted
    root = logging.getLogger("kohakuwullm_b200")
    root.handlers.clear()
    handler = logging.StreamHandler(stream or sys.stderr)
    handler.setFormatter(logging.Formatter("%(message)s"))
    root.addHandler(handler)
    root.setLevel(level)
    root.propagate = False
    if all_ranks is None:
        all_ranks = os.environ.get("KWP_LOG_ALL_RANKS", "0") == "1"
    # a flag of our own: ``Logger.disabled`` on the parent does not stop records that child loggers hand up
    _muted = (not all_ranks) and _rank() != 0
    _configured = True


class StructuredLogger:
    def __init__(self, name: str):
        self._log = logging.getLogger(f"kohakuwullm_b200.{name}")

    def _emit(self, level: int, event: str, fields: dict) -> None:
        if not _configured:
            configure()
        if _muted and level < logging.ERROR:      # errors are worth seeing from any rank
            return
        stamp = time.strftime("%H:%M:%S")
        body = " ".join(f"{k}={_fmt(v)}" for k, v in fields.items())
        self._log.log(level, f"{stamp} [r{_rank()}] {event} {body}".rstrip())

    def info(self, event: str, **fields):
        self._emit(logging.INFO, event, fields)

    def warning(self, event: str, **fields):
        self._emit(logging.WARNING, event, fields)

    def error(self, event: str, **fields):
        self._emit(logging.ERROR, event, fields)

    def debug(self, event: str, **fields):
        self._emit(logging.DEBUG, event, fields)


def _fmt(v) -> str:
    if isinstance(v, float):
        return f"{v:.6g}"
    return str(v)


def get_logger(name: str) -> StructuredLogger:
    return StructuredLogger(name)
