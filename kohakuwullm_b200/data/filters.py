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


def text_units(text: str) -> list[str]:
    """Words, or single characters where whitespace does not segment the text (CJK, base64 or hex runs):
    a 'word' longer than 40 characters is cut into characters."""
    out: list[str] = []
    for word in text.split():
        if len(word) > 40 or any("぀" <= ch <= "ヿ" or "㐀" <= ch <= "鿿" for ch in word):
            out.extend(word)
        else:
            out.append(word)
    return out


def longest_consecutive_repeat(units: Sequence, max_n: int = 13) -> tuple[int, int]:
    """(repeats, n) of the n-gram (n <= ``max_n``) that repeats back to back most often: ``a b a b a b`` gives
    (3, 2). Loss spikes in pretraining have been traced to documents with long runs of this shape, and filtering
    them also reduces repetition in generation. O(len * max_n)."""
    best, best_n = 1, 1
    L = len(units)
    for n in range(1, max_n + 1):
        if 2 * n > L:
            break
        run = 0                      # consecutive positions i with units[i] == units[i + n]
        for i in range(L - n):
            if units[i] == units[i + n]:
                run += 1
                reps = run // n + 1
                if reps > best:
                    best, best_n = reps, n
            else:
                run = 0
    return best, best_n


def passes_consecutive_repeat_filter(text: str, max_n: int = 13, threshold: int = 32) -> bool:
    return longest_consecutive_repeat(text_units(text), max_n)[0] < threshold


def passes_consecutive_token_repeat(tokens: Sequence, max_n: int = 13, threshold: int = 32) -> bool:
    """The consecutive-repeat rule on token ids (what a loader filter sees)."""
    return longest_consecutive_repeat(tokens, max_n)[0] < threshold


DOC_FILTERS = {"ngram": passes_repeat_filter, "consecutive": passes_consecutive_token_repeat}


def build_doc_filter(spec):
    """A loader's ``doc_filter`` (token ids -> keep?) from a name, ``{"name": ..., **arguments}`` or a callable;
    ``None`` / ``""`` is no filter. The result is a ``functools.partial`` of a module-level function, so it pickles
    into loader worker processes."""
    import functools

    if not spec:
        return None
    if callable(spec):
        return spec
    cfg = {"name": spec} if isinstance(spec, str) else dict(spec)
    name = cfg.pop("name")
    if name not in DOC_FILTERS:
        raise KeyError(f"unknown document filter {name!r}; known: {', '.join(sorted(DOC_FILTERS))}")
    return functools.partial(DOC_FILTERS[name], **cfg)
