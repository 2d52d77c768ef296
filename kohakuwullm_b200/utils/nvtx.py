"""NVTX ranges around the phases of a training step (off unless ``KWU_NVTX=1`` or ``enable()``).

``with nvtx.range("name"):`` costs one attribute test when disabled. The ranges show up in any
NVTX-aware timeline tool; nothing here depends on one being installed. Reference: the ``record_function``
ranges of src/kohakuwullm/bench/profile (module attribution) play the same role.
"""

from __future__ import annotations

import contextlib
import os

_enabled = os.environ.get("KWU_NVTX", "0") not in ("", "0", "false", "False")


def enable(on: bool = True) -> None:
    global _enabled
    _enabled = on


def enabled() -> bool:
    return _enabled


@contextlib.contextmanager
def range(name: str):  # noqa: A001  (mirrors torch.cuda.nvtx.range)
    if not _enabled:
        yield
        return
    import torch

    if not torch.cuda.is_available():
        yield
        return
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()
