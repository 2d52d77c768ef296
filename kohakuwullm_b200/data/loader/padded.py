"""Padded (B,S) batches: the layout used by evaluation and by the KV-cache generation path; the training engine
takes them as well (eager launches, explicit-mask attention: for ablations and readable debugging, the loss per token
is the same as for the packed layout).
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

    @property
    def num_tokens(self) -> int:
        return int(self.tokens.numel())

    def trained_tokens(self) -> int:
        """Positions with a target (padding and masked spans carry -100)."""
        return int((self.labels != IGNORE).sum())

    def to(self, device, non_blocking=True):
        return PaddedBatch(self.tokens.to(device, non_blocking=non_blocking),
                           self.labels.to(device, non_blocking=non_blocking),
                           self.lengths.to(device, non_blocking=non_blocking), self.seq_info.to(device, non_blocking))


def collate_padded(samples, pad_id: int = 0, pad_to_multiple: int | None = None,
                   max_length: int | None = None) -> PaddedBatch:
    """Rows are documents (``ids`` or ``(ids, trained_mask)``), cut to ``max_length`` tokens, padded on the right."""
    docs = []
    for s in samples:
        ids, mask = s if isinstance(s, tuple) else (s, None)
        ids = torch.as_tensor(ids, dtype=torch.long)
        if max_length and ids.numel() > max_length:
            ids = ids[:max_length]
            mask = None if mask is None else torch.as_tensor(mask)[:max_length]
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
