"""Token-budget packing loaders with exact resume.

``IterativePackLoader`` walks a record source in a deterministic (Feistel) order, renders and tokenises
records, and emits packs of at most ``k`` tokens (never fewer than ``k - m``): a document that does not
fit is carried to the next pack; documents longer than ``ctx_max`` are truncated. Every batch comes
with the POSITION needed to continue right after it: ``{shard, shards, pass, cursor, carry, emitted}``.

``MicroBatchedLoader`` is the pipeline variant: every micro-batch holds EXACTLY ``k`` tokens (the
straddling document is cut and its tail opens the next micro-batch; a fully masked filler closes a
short last one) and ``num_microbatches`` of them form one ``MicroBatchedStep``.

``ResumableLoader`` wraps either of them (optionally behind ``torch.utils.data.DataLoader`` workers),
records the position of the batch that was last CONSUMED, all-gathers every rank's positions into
``state_dict()`` and refuses to resume under a different world size / worker count / shard layout.
Reference: src/kohakuwullm/data/loader/iterative.py:24-358, microbatch.py:20-261, resume.py:20-274.
"""

from __future__ import annotations

import random
from dataclasses import dataclass, field
from typing import Callable, Iterator, Sequence

import torch
import torch.distributed as dist

from kohakuwullm_b200.data.loader.permute import ShardIndices
from kohakuwullm_b200.data.packing import IGNORE, PackedBatch, collate_packed


def tokenize_segments(segments, encode: Callable[[str], Sequence[int]], bos: int | None, eos: int | None):
    """Segments -> (ids, train_mask). BOS is never trained; EOS is trained when the last segment is."""
    ids: list[int] = []
    mask: list[bool] = []
    if bos is not None:
        ids.append(bos)
        mask.append(False)
    last_trained = False
    for text, trained in segments:
        piece = list(encode(text))
        ids.extend(piece)
        mask.extend([trained] * len(piece))
        last_trained = trained
    if eos is not None:
        ids.append(eos)
        mask.append(last_trained)
    return torch.tensor(ids, dtype=torch.long), torch.tensor(mask, dtype=torch.bool)


@dataclass
class MicroBatchedStep:
    """One optimizer step for a pipeline: ``num_microbatches`` packs of exactly ``k`` tokens."""

    micro: list[PackedBatch]

    def __iter__(self):
        return iter(self.micro)

    def __len__(self):
        return len(self.micro)

    def __getitem__(self, i):
        return self.micro[i]

    def pin_memory(self):
        return MicroBatchedStep([m.pin_memory() for m in self.micro])


@dataclass
class LoaderPosition:
    shard: int
    shards: int
    epoch: int = 0          # "pass" over the data
    cursor: int = 0         # next index inside the shard's strided order
    carry: list = field(default_factory=list)  # documents rendered but not yet emitted: (ids, mask) lists
    emitted: int = 0

    def as_dict(self) -> dict:
        return {"shard": self.shard, "shards": self.shards, "pass": self.epoch, "cursor": self.cursor,
                "carry": [(i.tolist(), m.tolist()) for i, m in self.carry], "emitted": self.emitted}

    @classmethod
    def from_dict(cls, d: dict) -> "LoaderPosition":
        carry = [(torch.tensor(i, dtype=torch.long), torch.tensor(m, dtype=torch.bool)) for i, m in d.get("carry", [])]
        return cls(d["shard"], d["shards"], d.get("pass", 0), d.get("cursor", 0), carry, d.get("emitted", 0))


class EmptyShard(LookupError):
    """This loader's shard holds no records."""


class IterativePackLoader:
    def __init__(self, records, renderer, encode, *, k: int, m: int = 0, ctx_max: int | None = None,
                 shard: int = 0, shards: int = 1, seed: int = 0, bos: int | None = None, eos: int | None = None,
                 shuffle: bool = True, exact: bool = False, pad_id: int = 0, min_tokens: int = 2,
                 doc_filter: Callable | None = None, max_retries: int = 64, max_deferred: int = 16):
        self.records, self.renderer, self.encode = records, renderer, encode
        self.k, self.m, self.ctx_max = k, m, ctx_max or k
        self.order = ShardIndices(len(records), shard, shards, seed, shuffle)
        self.seed, self.bos, self.eos, self.exact, self.pad_id = seed, bos, eos, exact, pad_id
        self.min_tokens, self.doc_filter, self.max_retries = min_tokens, doc_filter, max_retries
        self.max_deferred = max_deferred
        self.pos = LoaderPosition(shard, shards)

    # ------------------------------------------------------------------ resume
    def state_dict(self) -> dict:
        return self.pos.as_dict()

    def load_state_dict(self, state: dict) -> None:
        if state["shard"] != self.order.shard or state["shards"] != self.order.shards:
            raise ValueError(f"loader position belongs to shard {state['shard']}/{state['shards']}, this loader is "
                             f"shard {self.order.shard}/{self.order.shards}")
        self.pos = LoaderPosition.from_dict(state)

    # ------------------------------------------------------------------ documents
    def _next_document(self):
        tries = 0
        while True:
            if self.pos.cursor >= self.order.length():
                self.pos.epoch += 1
                self.pos.cursor = 0
                if self.order.length() == 0:
                    raise EmptyShard(f"shard {self.order.shard}/{self.order.shards} of {len(self.records)} records is empty")
            idx = self.order.index(self.pos.epoch, self.pos.cursor)
            self.pos.cursor += 1
            rng = random.Random((self.seed * 1000003 + idx) ^ (self.pos.epoch << 32))
            ids, mask = tokenize_segments(self.renderer(self.records[idx], rng), self.encode, self.bos, self.eos)
            if ids.numel() > self.ctx_max:
                ids, mask = ids[: self.ctx_max], mask[: self.ctx_max]
            ok = ids.numel() >= self.min_tokens and (self.doc_filter is None or self.doc_filter(ids.tolist()))
            if ok:
                return ids, mask
            tries += 1
            if tries > self.max_retries:
                raise RuntimeError(f"{self.max_retries} consecutive records were rejected; check the filter / renderer")

    def _next_pack(self) -> PackedBatch:
        docs, used, deferred = [], 0, 0
        carry, self.pos.carry = self.pos.carry, []
        queue = list(carry)
        while True:
            if queue:
                ids, mask = queue.pop(0)
            else:
                ids, mask = self._next_document()
            room = self.k - used
            if ids.numel() <= room:
                docs.append((ids, mask))
                used += ids.numel()
                if used >= self.k - self.m and not self.exact or used == self.k:
                    break
                continue
            if self.exact:
                # cut the straddling document; its tail opens the next micro-batch
                if room >= self.min_tokens:
                    docs.append((ids[:room], mask[:room]))
                    used += room
                    tail = (ids[room:], mask[room:])
                    if tail[0].numel() >= self.min_tokens:
                        self.pos.carry.append(tail)
                else:
                    self.pos.carry.append((ids, mask))
                break
            self.pos.carry.append((ids, mask))
            deferred += 1
            # a pack that no upcoming document fits into (the room is smaller than every document but larger than
            # the slack) must still close: after a few deferrals it is emitted as it is
            if used >= self.k - self.m or not docs or deferred >= self.max_deferred:
                break
        self.pos.carry = queue + self.pos.carry
        self.pos.emitted += 1
        return collate_packed(docs, pad_to_multiple=self.k if self.exact else None, pad_id=self.pad_id)

    def __iter__(self) -> Iterator[tuple[PackedBatch, dict]]:
        while True:
            try:
                batch = self._next_pack()
            except EmptyShard:
                return                 # nothing to read (a hold-out split of a tiny corpus): an empty iteration, not an error
            yield batch, self.pos.as_dict()


class MicroBatchedLoader:
    """``num_microbatches`` exact-``k`` packs per item. Built with the same arguments on every pipeline
    rank (``shard=0, shards=1``) so all ranks see identical steps."""

    def __init__(self, records, renderer, encode, *, k: int, num_microbatches: int, **kw):
        kw.setdefault("exact", True)
        self.inner = IterativePackLoader(records, renderer, encode, k=k, **kw)
        self.num_microbatches = num_microbatches

    def state_dict(self):
        return self.inner.state_dict()

    def load_state_dict(self, state):
        self.inner.load_state_dict(state)

    def __iter__(self):
        it = iter(self.inner)
        while True:
            micro, pos = [], None
            for _ in range(self.num_microbatches):
                batch, pos = next(it)
                micro.append(batch)
            yield MicroBatchedStep(micro), pos


class ResumableLoader:
    """Yields batches, remembers the position of the last batch handed out, and checkpoints all ranks'
    positions together."""

    def __init__(self, loader, group=None):
        self.loader, self.group = loader, group
        self._last: dict | None = None

    def __iter__(self):
        for batch, pos in self.loader:
            self._last = pos
            yield batch

    def _world(self):
        ok = dist.is_available() and dist.is_initialized()
        return (dist.get_world_size(self.group), dist.get_rank(self.group)) if ok else (1, 0)

    def state_dict(self) -> dict:
        world, rank = self._world()
        mine = self._last if self._last is not None else self.loader.state_dict()
        if world == 1:
            return {"world": 1, "positions": [mine]}
        parts: list = [None] * world
        dist.all_gather_object(parts, mine, group=self.group)
        return {"world": world, "positions": parts}

    def load_state_dict(self, state: dict) -> None:
        world, rank = self._world()
        if state["world"] != world:
            raise ValueError(f"loader state was saved with {state['world']} ranks and cannot resume on {world}: "
                             "per-rank shard positions do not transfer across world sizes")
        self.loader.load_state_dict(state["positions"][rank])
        self._last = state["positions"][rank]
