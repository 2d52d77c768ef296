"""Flat parameter / gradient storage.

Every parameter of a model becomes a view into one contiguous buffer per dtype group
(``"lp"``: 16-bit matrices, ``"fp32"``: everything kept in fp32; parameters flagged ``ep_local`` go to
``"lp_ep"`` / ``"fp32_ep"``, which data-parallel reductions skip), and gets a ``main_grad`` attribute:
a view into an fp32 gradient buffer of the same layout. This is what makes the whole-model fused
optimizer (one launch), the bucketed gradient collectives (contiguous ranges, no packing) and the
GEMM-epilogue gradient accumulation possible. Tensors are padded to ``align`` elements so every
parameter starts on a 256-byte boundary (TMA needs 16).

Gradient flow: the tcgen05 linear backward adds weight gradients straight into ``main_grad``; every
other parameter gets a post-accumulate hook that moves ``.grad`` into ``main_grad`` and frees it.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch
from torch import nn


@dataclass
class FlatGroup:
    key: str
    dtype: torch.dtype
    names: list[str] = field(default_factory=list)
    params: list[nn.Parameter] = field(default_factory=list)
    offsets: list[int] = field(default_factory=list)
    numels: list[int] = field(default_factory=list)
    total: int = 0
    data: torch.Tensor | None = None
    main_grad: torch.Tensor | None = None

    def span(self, i: int) -> tuple[int, int]:
        return self.offsets[i], self.offsets[i] + self.numels[i]


class FlatParameters:
    def __init__(self, module: nn.Module, align: int = 128, pad_total_to: int = 1024,
                 install_hooks: bool = True, allocator=None):
        """``allocator(numel, dtype, device) -> 1-D tensor`` lets a caller place the buffers in special
        memory (e.g. peer-mapped symmetric memory); the default is ordinary device memory."""
        alloc = allocator or (lambda n, dt, dev: torch.zeros(n, dtype=dt, device=dev))
        self.module = module
        self.groups: dict[str, FlatGroup] = {}
        seen: set[int] = set()
        for name, p in module.named_parameters():
            if id(p) in seen or not p.requires_grad:
                continue
            seen.add(id(p))
            key = "fp32" if p.dtype == torch.float32 else "lp"
            if getattr(p, "ep_local", False):
                key += "_ep"  # expert-parallel shards: rank-local, never reduced over the data-parallel group
            g = self.groups.setdefault(key, FlatGroup(key, p.dtype))
            if p.dtype != g.dtype:
                raise ValueError(f"mixed low-precision dtypes: {p.dtype} vs {g.dtype} ({name})")
            g.names.append(name)
            g.params.append(p)
            g.offsets.append(g.total)
            g.numels.append(p.numel())
            g.total += -(-p.numel() // align) * align
        for g in self.groups.values():
            g.total = -(-g.total // pad_total_to) * pad_total_to
            device = g.params[0].device
            g.data = alloc(g.total, g.dtype, device)
            g.main_grad = alloc(g.total, torch.float32, device)
            g.data.zero_()
            g.main_grad.zero_()
            for i, p in enumerate(g.params):
                s, e = g.span(i)
                view = g.data[s:e].view(p.shape)
                view.copy_(p.data)
                p.data = view
                p.main_grad = g.main_grad[s:e].view(p.shape)
                p.grad_in_main = False
        self._hooks = []
        if install_hooks:
            self.install_hooks()

    def install_hooks(self) -> None:
        def hook(p: nn.Parameter) -> None:
            if p.grad is not None:
                p.main_grad.add_(p.grad)
                p.grad = None

        for g in self.groups.values():
            for p in g.params:
                self._hooks.append(p.register_post_accumulate_grad_hook(hook))

    def zero_grad(self) -> None:
        for g in self.groups.values():
            g.main_grad.zero_()
            for p in g.params:
                p.grad = None

    def named_parameters(self):
        for g in self.groups.values():
            yield from zip(g.names, g.params)

    def grad_buffers(self) -> list[torch.Tensor]:
        return [g.main_grad for g in self.groups.values()]

    def replicated_keys(self) -> list[str]:
        return [k for k in self.groups if not k.endswith("_ep")]

    def local_keys(self) -> list[str]:
        """Groups holding expert-parallel shards (different tensors on every rank)."""
        return [k for k in self.groups if k.endswith("_ep")]
