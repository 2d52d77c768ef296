"""Synthetic packed token streams of a named shape (benchmarks, smoke tests, autotuning).

``make_pack(tokens, len_min, len_max)`` draws document lengths from a seeded generator (uniform or
log-uniform in ``[len_min, len_max]``), truncates the document that straddles the end so the pack holds
exactly ``tokens`` tokens, and fills it with uniform random ids. Reference:
src/kohakuwullm/bench (``make_packs`` / ``make_tokens``) as used by
scripts/bench/e2e/step_throughput.py:125-130.
"""

from __future__ import annotations

import math

import torch

from kohakuwullm_b200.data.packing import IGNORE, PackedBatch
from kohakuwullm_b200.models.seqinfo import SeqInfo


def draw_lengths(total: int, len_min: int, len_max: int, gen: torch.Generator, log_uniform: bool = False) -> list[int]:
    lengths, used = [], 0
    while used < total:
        u = torch.rand((), generator=gen).item()
        if log_uniform:
            n = int(round(math.exp(math.log(len_min) + u * (math.log(len_max) - math.log(len_min)))))
        else:
            n = len_min + int(u * (len_max - len_min + 1))
        n = max(1, min(n, len_max, total - used))
        lengths.append(n)
        used += n
    # a trailing 1-token document has no target; merge it into its neighbour
    if len(lengths) > 1 and lengths[-1] == 1:
        last = lengths.pop()
        lengths[-1] += last
    return lengths


def make_pack(tokens: int, len_min: int, len_max: int, vocab_size: int, seed: int = 0,
              log_uniform: bool = False) -> PackedBatch:
    gen = torch.Generator().manual_seed(seed)
    lengths = draw_lengths(tokens, len_min, len_max, gen, log_uniform)
    ids = torch.randint(0, vocab_size, (tokens,), generator=gen, dtype=torch.long)
    labels = torch.full((tokens,), IGNORE, dtype=torch.long)
    start = 0
    for n in lengths:
        if n > 1:
            labels[start:start + n - 1] = ids[start + 1:start + n]
        start += n
    return PackedBatch(ids, labels, SeqInfo.from_lengths(lengths))


def make_packs(n_micro: int, tokens: int, len_min: int, len_max: int, vocab_size: int, seed: int = 0,
               log_uniform: bool = False) -> list[PackedBatch]:
    return [make_pack(tokens, len_min, len_max, vocab_size, seed * 1000003 + i, log_uniform) for i in range(n_micro)]
