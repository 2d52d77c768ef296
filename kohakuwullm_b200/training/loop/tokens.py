"""Cumulative token / FLOP counters as an immutable snapshot; subtraction gives an interval.
Reference: src/kohakuwullm/training/loop/tokens.py:15-77."""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class TokenSnapshot:
    seen: int = 0            # tokens fed to the model
    trained: int = 0         # tokens with a target
    model_flops: float = 0.0
    hardware_flops: float = 0.0
    elapsed: float = 0.0     # seconds of training time

    def __sub__(self, other: "TokenSnapshot") -> "TokenSnapshot":
        return TokenSnapshot(self.seen - other.seen, self.trained - other.trained,
                             self.model_flops - other.model_flops, self.hardware_flops - other.hardware_flops,
                             self.elapsed - other.elapsed)

    def __add__(self, other: "TokenSnapshot") -> "TokenSnapshot":
        return TokenSnapshot(self.seen + other.seen, self.trained + other.trained,
                             self.model_flops + other.model_flops, self.hardware_flops + other.hardware_flops,
                             self.elapsed + other.elapsed)

    @property
    def tokens_per_s(self) -> float:
        return self.seen / self.elapsed if self.elapsed > 0 else 0.0

    @property
    def b_tokens_per_day(self) -> float:
        return self.tokens_per_s * 86400 / 1e9

    def mfu(self, peak_flops: float) -> float:
        return self.model_flops / (self.elapsed * peak_flops) if self.elapsed > 0 and peak_flops > 0 else 0.0

    def hfu(self, peak_flops: float) -> float:
        return self.hardware_flops / (self.elapsed * peak_flops) if self.elapsed > 0 and peak_flops > 0 else 0.0


def all_reduce_int(value: int, device, group=None) -> int:
    """Exact integer sum over the group (int64 on the device, one host read)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return int(value)
    t = torch.tensor([int(value)], dtype=torch.int64, device=device if dist.get_backend(group) == "nccl" else "cpu")
    dist.all_reduce(t, group=group)
    return int(t.item())


def all_reduce_(snap: TokenSnapshot, device, group=None) -> TokenSnapshot:
    """Sum the counters over the group (tokens as int64, FLOPs as fp64); elapsed is kept local."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return snap
    dev = device if dist.get_backend(group) == "nccl" else "cpu"
    ints = torch.tensor([snap.seen, snap.trained], dtype=torch.int64, device=dev)
    flops = torch.tensor([snap.model_flops, snap.hardware_flops], dtype=torch.float64, device=dev)
    dist.all_reduce(ints, group=group)
    dist.all_reduce(flops, group=group)
    return TokenSnapshot(int(ints[0]), int(ints[1]), float(flops[0]), float(flops[1]), snap.elapsed)
