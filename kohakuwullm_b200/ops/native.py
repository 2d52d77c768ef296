"""ctypes binding of the in-tree sm_100a library ``_kwu_native.so``.

The library is plain ``extern "C"``: every entry point takes raw device pointers, sizes, a CUDA
stream handle and (for tensor-core kernels) the address of an int32 status word. Keeping torch
out of the native build makes a full rebuild take seconds and lets callers without torch use
the same symbols.

On a machine with a GPU the library is mandatory: :func:`lib` raises if it is missing rather
than letting an op fall back silently to eager PyTorch.
"""

from __future__ import annotations

import ctypes
import functools
import os
from pathlib import Path

import torch

_PKG = Path(__file__).resolve().parent.parent
LIB_PATH = _PKG / "_kwu_native.so"

ERROR_NAMES = {
    0: "ok",
    1: "timeout waiting for a TMA stage (full barrier)",
    2: "timeout waiting for a free smem stage (empty barrier)",
    3: "timeout waiting for an accumulator (full)",
    4: "timeout waiting for an accumulator (empty)",
    5: "timeout waiting for a flag",
    6: "timeout (misc)",
    7: "bad argument",
    8: "expert-parallel receive buffer overflow (raise the capacity factor)",
}


class NativeError(RuntimeError):
    pass


@functools.lru_cache(maxsize=1)
def lib() -> ctypes.CDLL:
    if not LIB_PATH.exists():
        if os.environ.get("KWU_BUILD_ON_IMPORT", "1") == "1":
            from kohakuwullm_b200.build import build

            build()
        else:
            raise NativeError(
                f"{LIB_PATH} is missing; run `python -m kohakuwullm_b200.build` (needs nvcc)"
            )
    handle = ctypes.CDLL(str(LIB_PATH))
    handle.kwu_last_error.restype = ctypes.c_char_p
    handle.kwu_launch_count.restype = ctypes.c_longlong
    if hasattr(handle, "kwu_flash_bwd_scratch_floats"):
        handle.kwu_flash_bwd_scratch_floats.restype = ctypes.c_longlong
    return handle


def available() -> bool:
    """True when the native kernels can run here (CUDA device of compute capability 10.x)."""
    if not torch.cuda.is_available():
        return False
    major, _ = torch.cuda.get_device_capability()
    return major == 10


def require() -> ctypes.CDLL:
    if not torch.cuda.is_available():
        raise NativeError("native kernels need a CUDA device")
    return lib()


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = lib().kwu_last_error().decode()
        raise NativeError(f"{what} failed (code {rc}): {msg}")


def stream_ptr() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


_status: dict[int, torch.Tensor] = {}


def status_word() -> torch.Tensor:
    """Per-device int32 word that kernels set when a bounded wait gives up."""
    dev = torch.cuda.current_device()
    if dev not in _status:
        _status[dev] = torch.zeros(1, dtype=torch.int32, device=f"cuda:{dev}")
        handle = lib()
        if hasattr(handle, "kwu_set_status_word"):
            with torch.cuda.device(dev):
                handle.kwu_set_status_word(ctypes.c_void_p(_status[dev].data_ptr()))
    return _status[dev]


class _StatusMirror:
    """Pinned host copy of one device's status word, refreshed by asynchronous copies."""

    def __init__(self, dev: int):
        self.host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.event = torch.cuda.Event()
        self.pending = False


_mirrors: dict[int, _StatusMirror] = {}


def poll_status() -> None:
    """Sync-free status check for training loops: raises if a kernel of an EARLIER step reported an error.

    Each call reads the pinned host mirror if the copy started by the previous call has completed, then
    starts the next 4-byte device->host copy on the current stream. An error is therefore seen one or two
    calls after the failing kernel ran, without the host ever waiting for the device."""
    if not torch.cuda.is_available():
        return
    dev = torch.cuda.current_device()
    word = _status.get(dev)
    if word is None:
        return
    mirror = _mirrors.get(dev)
    if mirror is None:
        mirror = _mirrors[dev] = _StatusMirror(dev)
    if mirror.pending and mirror.event.query():
        mirror.pending = False
        code = int(mirror.host[0])
        if code:
            word.zero_()
            raise NativeError(f"device {dev}: kernel reported '{ERROR_NAMES.get(code, code)}'")
    if not mirror.pending:
        mirror.host.copy_(word, non_blocking=True)
        mirror.event.record()
        mirror.pending = True


def check_status(sync: bool = True) -> None:
    """Read the status word (a host sync) and raise if any kernel reported a time-out."""
    if not _status:
        return
    for dev, word in _status.items():
        code = int(word.item()) if sync else 0
        if code:
            word.zero_()
            raise NativeError(f"device {dev}: kernel reported '{ERROR_NAMES.get(code, code)}'")
