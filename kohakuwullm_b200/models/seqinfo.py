"""Sequence layout carried next to the tokens.

Packed layout: ``tokens`` is (T,), ``cu_seqlens`` (N+1,) int32 marks document boundaries,
``position_ids`` (T,) restarts at every document. Padded layout: ``tokens`` is (B,S),
``cu_seqlens`` is ``None`` and ``position_ids`` is (B,S). The backbone is a pure function of
``(tokens, seq_info)``. Reference: src/kohakuwullm/models/components/seqinfo.py:11-85.
"""

from __future__ import annotations

from dataclasses import dataclass, replace

import torch


@dataclass
class SeqInfo:
    cu_seqlens: torch.Tensor | None
    position_ids: torch.Tensor
    max_seqlen: int
    num_seqs: int
    # host copy of the document lengths (kept so FLOP accounting and splitters never sync)
    lengths: tuple[int, ...] | None = None

    @property
    def packed(self) -> bool:
        return self.cu_seqlens is not None

    @property
    def seqlens(self) -> torch.Tensor:
        if self.cu_seqlens is None:
            b, s = self.position_ids.shape
            return torch.full((b,), s, dtype=torch.int32, device=self.position_ids.device)
        return self.cu_seqlens[1:] - self.cu_seqlens[:-1]

    @property
    def total_tokens(self) -> int:
        return int(self.position_ids.numel())

    @classmethod
    def from_lengths(cls, lengths, device=None) -> "SeqInfo":
        lens = [int(x) for x in lengths]
        if any(n <= 0 for n in lens):
            raise ValueError("document lengths must be positive")
        lt = torch.tensor(lens, dtype=torch.int32)
        cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
        cu[1:] = torch.cumsum(lt, 0)
        total = int(cu[-1])
        # position = index - start of its own document
        starts = torch.repeat_interleave(cu[:-1].long(), lt.long())
        pos = torch.arange(total, dtype=torch.long) - starts
        info = cls(cu, pos, max(lens) if lens else 0, len(lens), tuple(lens))
        return info.to(device) if device is not None else info

    @classmethod
    def padded(cls, batch: int, seqlen: int, device=None, offset: int | torch.Tensor = 0) -> "SeqInfo":
        pos = torch.arange(seqlen, dtype=torch.long, device=device).unsqueeze(0).expand(batch, seqlen)
        if isinstance(offset, torch.Tensor):
            pos = pos + offset.to(pos.device).reshape(-1, 1)
        elif offset:
            pos = pos + int(offset)
        return cls(None, pos, seqlen, batch, None)

    def to(self, device, non_blocking: bool = False) -> "SeqInfo":
        cu = None if self.cu_seqlens is None else self.cu_seqlens.to(device, non_blocking=non_blocking)
        return replace(self, cu_seqlens=cu, position_ids=self.position_ids.to(device, non_blocking=non_blocking))

    def pin_memory(self) -> "SeqInfo":
        cu = None if self.cu_seqlens is None else self.cu_seqlens.pin_memory()
        return replace(self, cu_seqlens=cu, position_ids=self.position_ids.pin_memory())
