"""Key/value cache for incremental decoding (padded layout only).

One (B, max_len, kv_heads, head_dim) K and V buffer per layer, allocated lazily from the first
append. ``static=True`` preallocates ``max_len`` rows and returns the whole buffer with a validity mask
(fixed shapes, CUDA-graph friendly); the dynamic cache returns only the filled prefix. All layers share
one ``length``, advanced by ``advance`` after the last layer of a step. Reference:
src/kohakuwullm/models/cache.py:14-199.
"""

from __future__ import annotations

import torch

from kohakuwullm_b200.models.seqinfo import SeqInfo


class KVCache:
    def __init__(self, num_layers: int, max_len: int, static: bool = True):
        self.num_layers, self.max_len, self.static = num_layers, max_len, static
        self.k: list[torch.Tensor | None] = [None] * num_layers
        self.v: list[torch.Tensor | None] = [None] * num_layers
        self.length = 0
        self._pending = 0

    @classmethod
    def from_config(cls, config, max_len: int, static: bool = True, num_layers: int | None = None):
        return cls(num_layers if num_layers is not None else config.depth, max_len, static)

    def seq_info(self, tokens: torch.Tensor) -> SeqInfo:
        """Layout of the next ``tokens`` (B,S): positions continue after the cached prefix."""
        b, s = tokens.shape
        return SeqInfo.padded(b, s, device=tokens.device, offset=self.length)

    def append(self, layer: int, k: torch.Tensor, v: torch.Tensor, q_pos: torch.Tensor):
        """Store this step's keys/values; returns ``(k_all, v_all, key_positions, key_valid)``."""
        B, S = k.shape[:2]
        end = self.length + S
        if end > self.max_len:
            raise RuntimeError(f"KV cache overflow: {end} > max_len {self.max_len}")
        if self.k[layer] is None:
            shape = (B, self.max_len, *k.shape[2:])
            self.k[layer] = torch.zeros(shape, dtype=k.dtype, device=k.device)
            self.v[layer] = torch.zeros(shape, dtype=v.dtype, device=v.device)
        self.k[layer][:, self.length:end] = k
        self.v[layer][:, self.length:end] = v
        self._pending = S
        used = self.max_len if self.static else end
        pos = torch.arange(used, device=k.device)[None, :].expand(B, used)
        valid = pos < end
        return self.k[layer][:, :used], self.v[layer][:, :used], pos, valid

    def advance(self) -> None:
        self.length += self._pending
        self._pending = 0

    def reset(self) -> None:
        self.length = 0
        self._pending = 0
