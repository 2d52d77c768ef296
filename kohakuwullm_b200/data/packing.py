"""Packed variable-length batches.

A ``PackedBatch`` is one flat token stream with per-document boundaries: ``tokens`` (T,), ``labels``
(T,) already shifted INSIDE each document (the last position of every document is ``-100``: no
next-token target crosses a boundary) and a :class:`SeqInfo`. Reference:
src/kohakuwullm/data/packing.py:20-307.
"""

from __future__ import annotations

from dataclasses import dataclass, replace

import torch

from kohakuwullm_b200.models.seqinfo import SeqInfo

IGNORE = -100


@dataclass
class PackedBatch:
    tokens: torch.Tensor
    labels: torch.Tensor
    seq_info: SeqInfo
    n_trained: int | None = None   # cached count of positions with a target

    @property
    def num_tokens(self) -> int:
        return int(self.tokens.numel())

    def trained_tokens(self) -> int:
        """Count of positions with a target. Counted once (on the host when the labels are there) and
        carried along by ``to`` / ``pin_memory``, so a batch that already lives on the device costs a
        device synchronisation only the first time it is asked."""
        if self.n_trained is None:
            self.n_trained = int((self.labels != IGNORE).sum())
        return self.n_trained

    def pin_memory(self) -> "PackedBatch":
        return PackedBatch(self.tokens.pin_memory(), self.labels.pin_memory(), self.seq_info.pin_memory(),
                           self.n_trained)

    def to(self, device, non_blocking: bool = True) -> "PackedBatch":
        if self.n_trained is None and not self.labels.is_cuda:
            self.trained_tokens()
        return PackedBatch(self.tokens.to(device, non_blocking=non_blocking),
                           self.labels.to(device, non_blocking=non_blocking),
                           self.seq_info.to(device, non_blocking=non_blocking), self.n_trained)

    def nbytes(self) -> int:
        n = self.tokens.numel() * self.tokens.element_size() + self.labels.numel() * self.labels.element_size()
        n += self.seq_info.position_ids.numel() * self.seq_info.position_ids.element_size()
        if self.seq_info.cu_seqlens is not None:
            n += self.seq_info.cu_seqlens.numel() * self.seq_info.cu_seqlens.element_size()
        return n


def shift_labels(ids: torch.Tensor, mask: torch.Tensor | None = None) -> torch.Tensor:
    """Next-token targets for ONE document: ``labels[i] = ids[i+1]``, last position ignored.
    ``mask`` (same length, bool) marks positions whose TOKEN is trained on."""
    labels = torch.full_like(ids, IGNORE)
    if ids.numel() > 1:
        nxt = ids[1:].clone()
        if mask is not None:
            nxt[~mask[1:]] = IGNORE
        labels[:-1] = nxt
    return labels


def collate_packed(samples, pad_to_multiple: int | None = None, pad_id: int = 0) -> PackedBatch:
    """``samples``: iterable of ``ids`` tensors or ``(ids, train_mask)`` pairs. Documents of one token
    or fewer are dropped (they carry no target). An optional fully-masked filler document pads the
    pack to a multiple of ``pad_to_multiple``."""
    ids_list, label_list, lengths = [], [], []
    for s in samples:
        ids, mask = (s if isinstance(s, tuple) else (s, None))
        ids = torch.as_tensor(ids, dtype=torch.long)
        if ids.numel() <= 1:
            continue
        ids_list.append(ids)
        label_list.append(shift_labels(ids, None if mask is None else torch.as_tensor(mask, dtype=torch.bool)))
        lengths.append(ids.numel())
    total = sum(lengths)
    if pad_to_multiple and total % pad_to_multiple:
        fill = pad_to_multiple - total % pad_to_multiple
        ids_list.append(torch.full((fill,), pad_id, dtype=torch.long))
        label_list.append(torch.full((fill,), IGNORE, dtype=torch.long))
        lengths.append(fill)
    if not lengths:
        raise ValueError("empty batch: every sample had <= 1 token")
    return PackedBatch(torch.cat(ids_list), torch.cat(label_list), SeqInfo.from_lengths(lengths))


def slice_documents(batch: PackedBatch, doc_indices) -> PackedBatch:
    lens = batch.seq_info.lengths or tuple(batch.seq_info.seqlens.tolist())
    starts = [0]
    for n in lens:
        starts.append(starts[-1] + n)
    pieces = [(starts[i], starts[i + 1]) for i in doc_indices]
    tok = torch.cat([batch.tokens[s:e] for s, e in pieces])
    lab = torch.cat([batch.labels[s:e] for s, e in pieces])
    return PackedBatch(tok, lab, SeqInfo.from_lengths([lens[i] for i in doc_indices], device=tok.device))


def split_packed(batch: PackedBatch, parts: int) -> list[PackedBatch]:
    """Document-aligned split into ``parts`` micro-batches: longest document first onto the currently
    smallest bin. Bins that stay empty are dropped, so fewer than ``parts`` pieces may come back."""
    if parts <= 1:
        return [batch]
    lens = batch.seq_info.lengths or tuple(batch.seq_info.seqlens.tolist())
    order = sorted(range(len(lens)), key=lambda i: -lens[i])
    bins: list[list[int]] = [[] for _ in range(parts)]
    load = [0] * parts
    for i in order:
        b = min(range(parts), key=lambda j: load[j])
        bins[b].append(i)
        load[b] += lens[i]
    return [slice_documents(batch, sorted(b)) for b in bins if b]
