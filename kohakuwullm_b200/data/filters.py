"""Cheap text-quality filters. ``ngram_repeat_ratio`` is the share of n-grams that repeat an earlier
one; ``passes_repeat_filter`` rejects degenerate (looping) documents.
Reference: src/kohakuwullm/data/filters.py:14-88."""

from __future__ import annotations

from typing import Sequence


def ngram_repeat_ratio(tokens: Sequence, n: int = 4) -> float:
    if len(tokens) < n + 1:
        return 0.0
    seen, repeats, total = set(), 0, 0
    for i in range(len(tokens) - n + 1):
        gram = tuple(tokens[i:i + n])
        total += 1
        if gram in seen:
            repeats += 1
        else:
            seen.add(gram)
    return repeats / total


def passes_repeat_filter(tokens: Sequence, n: int = 4, max_ratio: float = 0.3, min_length: int = 16) -> bool:
    if len(tokens) < min_length:
        return True
    return ngram_repeat_ratio(tokens, n) <= max_ratio
