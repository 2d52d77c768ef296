"""Data pipeline: record sources -> renderers -> tokenisation -> packing -> (resumable) loaders."""

from __future__ import annotations

from typing import Any, Callable

from kohakuwullm_b200.data import filters  # noqa: F401
from kohakuwullm_b200.data.loader.iterative import (  # noqa: F401
    IterativePackLoader, LoaderPosition, MicroBatchedLoader, MicroBatchedStep, ResumableLoader, tokenize_segments,
)
from kohakuwullm_b200.data.loader.padded import PaddedBatch, collate_padded, split_padded  # noqa: F401
from kohakuwullm_b200.data.loader.permute import FeistelPermutation, ShardIndices, is_validation  # noqa: F401
from kohakuwullm_b200.data.packing import PackedBatch, collate_packed, split_packed  # noqa: F401
from kohakuwullm_b200.data.renderers import base as _renderers  # noqa: F401  (registrations)
from kohakuwullm_b200.data.sources import kvstore as _kvstore  # noqa: F401  (registrations)
from kohakuwullm_b200.data.sources import records as _records  # noqa: F401  (registrations)
from kohakuwullm_b200.data.synthetic import make_pack, make_packs  # noqa: F401
from kohakuwullm_b200.registry import DATASET, LOADER, RENDERER, build


class ByteTokenizer:
    """256 byte values + BOS/EOS: a dependency-free tokenizer for tests and smoke runs."""

    bos_token_id, eos_token_id, vocab_size = 256, 257, 258

    def encode(self, text: str) -> list[int]:
        return list(text.encode("utf-8"))

    def decode(self, ids) -> str:
        return bytes(i for i in ids if i < 256).decode("utf-8", errors="replace")


def build_records(spec: Any):
    return build(spec, DATASET)


def build_dataset(records_spec: Any, renderer_spec: Any = "plain"):
    return build(records_spec, DATASET), build(renderer_spec, RENDERER)


def build_loader(kind: str, records, renderer, encode: Callable, *, rank: int = 0, world: int = 1,
                 worker: int = 0, workers: int = 1, **kw):
    """``iterative`` one shard; ``ddp`` one shard per (rank, worker); ``pipeline`` identical exact-k
    micro-batched steps on every rank; ``torch`` / ``map`` map-style loaders of whole documents, ``samples_per_batch``
    per batch, ``layout="packed"`` (one row) or ``"padded"`` (one row per document)."""
    if kind == "iterative":
        return ResumableLoader(IterativePackLoader(records, renderer, encode, **kw))
    if kind == "ddp":
        shards = world * workers
        return ResumableLoader(IterativePackLoader(records, renderer, encode, shard=rank * workers + worker,
                                                   shards=shards, **kw))
    if kind == "pipeline":
        if workers > 1:
            from kohakuwullm_b200.data.loader.workers import WorkerPackLoader

            return ResumableLoader(WorkerPackLoader(records, renderer, encode, workers=workers, kind="pipeline", **kw))
        return ResumableLoader(MicroBatchedLoader(records, renderer, encode, **kw))
    if kind == "workers":
        # rendering, tokenisation and packing in ``workers`` child processes, one shard each
        from kohakuwullm_b200.data.loader.workers import WorkerPackLoader

        return ResumableLoader(WorkerPackLoader(records, renderer, encode, workers=workers, rank=rank, world=world, **kw))
    if kind in ("torch", "map"):
        import torch
        from torch.utils.data import DataLoader, Dataset

        bos, eos = kw.pop("bos", None), kw.pop("eos", None)
        samples = kw.pop("samples_per_batch", 8)
        layout, ctx_max, pad_id = kw.pop("layout", "packed"), kw.pop("ctx_max", None), kw.pop("pad_id", 0)
        if layout not in ("packed", "padded"):
            raise ValueError(f"layout must be 'packed' or 'padded', not {layout!r}")

        def collate(rows):
            if layout == "padded":
                return collate_padded(rows, pad_id=pad_id, pad_to_multiple=8, max_length=ctx_max)
            return collate_packed([(i[:ctx_max], None if m is None else m[:ctx_max]) if ctx_max else (i, m)
                                   for i, m in rows])

        class _Docs(Dataset):
            def __len__(self):
                return len(records)

            def __getitem__(self, i):
                return tokenize_segments(renderer(records[i], None), encode, bos, eos)

        return DataLoader(_Docs(), batch_size=samples, shuffle=kw.pop("shuffle", True), collate_fn=collate,
                          num_workers=kw.pop("num_workers", 0), generator=torch.Generator().manual_seed(kw.pop("seed", 0)))
    raise KeyError(f"unknown loader kind {kind!r}; choose from iterative, ddp, workers, pipeline, torch, map")


for _kind in ("iterative", "ddp", "workers", "pipeline", "torch", "map"):
    LOADER.register(_kind, (lambda k: (lambda *a, **kw: build_loader(k, *a, **kw)))(_kind))
