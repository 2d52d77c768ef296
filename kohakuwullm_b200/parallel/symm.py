"""Peer-mapped (symmetric) device memory over NVLink.

``SymmetricPool`` allocates tensors through ``torch.distributed._symmetric_memory`` and, after
``rendezvous``, exposes for each of them the device addresses of EVERY rank's copy, which is what the
fused communication kernels take. Only plain peer loads/stores are used by this framework; NVLink
multicast binding is switched off before the first allocation (a rank that dies while its memory is
bound to a multicast object can fault its peers' GPUs).
"""

from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")


class SymmetricTensor:
    def __init__(self, tensor: torch.Tensor):
        self.tensor = tensor
        self.handle = None
        self.ptrs: list[int] = []

    def rendezvous(self, group) -> "SymmetricTensor":
        import torch.distributed._symmetric_memory as symm_mem

        self.handle = symm_mem.rendezvous(self.tensor, group=group)
        base = [int(p) for p in self.handle.buffer_ptrs]
        # the tensor may sit at an offset inside the handle's allocation
        local = base[self.handle.rank]
        delta = self.tensor.data_ptr() - local
        self.ptrs = [p + delta for p in base]
        return self

    def ptr_table(self):
        """ctypes array of the ``world`` device addresses (own rank included)."""
        return (ctypes.c_longlong * len(self.ptrs))(*self.ptrs)


class SymmetricPool:
    def __init__(self, group=None):
        self.group = group if group is not None else dist.group.WORLD
        self.items: list[SymmetricTensor] = []

    def empty(self, numel: int, dtype: torch.dtype, device) -> torch.Tensor:
        import torch.distributed._symmetric_memory as symm_mem

        t = symm_mem.empty(numel, dtype=dtype, device=device)
        self.items.append(SymmetricTensor(t))
        return t

    def rendezvous_all(self) -> None:
        for item in self.items:
            if item.handle is None:
                item.rendezvous(self.group)

    def find(self, tensor: torch.Tensor) -> SymmetricTensor:
        for item in self.items:
            if item.tensor.data_ptr() == tensor.data_ptr():
                return item
        raise KeyError("tensor was not allocated from this pool")
