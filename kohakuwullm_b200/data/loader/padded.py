"""Padded (B,S) batches: the layout used by evaluation and by the KV-cache generation path.
Reference: src/kohakuwullm/data/loader/padded.py:14-102."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from kohakuwullm_b200.data.packing import IGNORE, shift_labels
from kohakuwullm_b200.models.seqinfo import SeqInfo


@dataclass
class PaddedBatch:
    tokens: torch.Tensor      # (B, S)
    labels: torch.Tensor      # (B, S), -100 on padding and on untrained positions
    lengths: torch.Tensor     # (B,)
    seq_info: SeqInfo

    def to(self, device, non_blocking=True):
        return PaddedBatch(self.tokens.to(device, non_blocking=non_blocking),
                           self.labels.to(device, non_blocking=non_blocking),
                           self.lengths.to(device, non_blocking=non_blocking), self.seq_info.to(device, non_blocking))


def collate_padded(samples, pad_id: int = 0, pad_to_multiple: int | None = None) -> PaddedBatch:
    docs = []
    for s in samples:
        ids, mask = s if isinstance(s, tuple) else (s, None)
        ids = torch.as_tensor(ids, dtype=torch.long)
        if ids.numel() > 1:
            docs.append((ids, shift_labels(ids, None if mask is None else torch.as_tensor(mask, dtype=torch.bool))))
    if not docs:
        raise ValueError("empty batch")
    S = max(d[0].numel() for d in docs)
    if pad_to_multiple:
        S = -(-S // pad_to_multiple) * pad_to_multiple
    B = len(docs)
    tokens = torch.full((B, S), pad_id, dtype=torch.long)
    labels = torch.full((B, S), IGNORE, dtype=torch.long)
    for i, (ids, lab) in enumerate(docs):
        tokens[i, : ids.numel()] = ids
        labels[i, : ids.numel()] = lab
    lengths = torch.tensor([d[0].numel() for d in docs])
    return PaddedBatch(tokens, labels, lengths, SeqInfo.padded(B, S))


def split_padded(batch: PaddedBatch, parts: int) -> list[PaddedBatch]:
    """Split along the batch axis into at most ``parts`` pieces of near-equal row count."""
    B = batch.tokens.shape[0]
    parts = min(parts, B)
    out, start = [], 0
    for p in range(parts):
        n = B // parts + (1 if p < B % parts else 0)
        sl = slice(start, start + n)
        out.append(PaddedBatch(batch.tokens[sl], batch.labels[sl], batch.lengths[sl],
                               SeqInfo.padded(n, batch.tokens.shape[1], device=batch.tokens.device)))
        start += n
    return out
