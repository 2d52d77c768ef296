"""Prompts for training-time sample previews, taken from real documents.

``prompts_from_batch`` cuts documents of the batch that was just trained on: where a document has a
masked (untrained) prefix followed by trained tokens — a chat turn — the prompt is everything up to the
start of a trained span, read from the document's own loss mask; otherwise (plain text) the prompt is a
fixed fraction of the document. ``corpus_prompts`` cuts held-out records at a token fraction. Both are
seeded, so every rank draws the same prompts without communicating.
Reference behaviour: src/kohakuwullm/data/preview.py:18-215.
"""

from __future__ import annotations

import random
from typing import Callable, Sequence

import torch

IGNORE_INDEX = -100
MIN_FILLER_TOKENS = 32


def batch_documents(batch) -> list[tuple[torch.Tensor, torch.Tensor]]:
    """``[(tokens, labels)]`` per document of a packed batch, a list of packed micro-batches, a pipeline step
    (``micro``: its packs), or an object
    with ``tokens`` / ``labels`` and ``seq_infos`` (one layout per equally sized micro-batch)."""
    if hasattr(batch, "micro"):                      # a pipeline step: its packs, in order
        batch = list(batch.micro)
    if isinstance(batch, (list, tuple)):
        out = []
        for b in batch:
            out.extend(batch_documents(b))
        return out
    tokens, labels = batch.tokens, batch.labels
    infos = getattr(batch, "seq_infos", None) or [batch.seq_info]
    width = tokens.numel() // len(infos)
    docs = []
    for m, info in enumerate(infos):
        bounds = info.cu_seqlens.tolist()
        for a, b in zip(bounds, bounds[1:]):
            if b > a:
                docs.append((tokens[m * width + a:m * width + b], labels[m * width + a:m * width + b]))
    return docs


def trained_spans(labels: torch.Tensor) -> list[tuple[int, int]]:
    """Runs of trained tokens in UNSHIFTED positions: labels are shifted inside the document, so a target
    at position i means token i + 1 is trained."""
    flags = (labels != IGNORE_INDEX).tolist()
    spans, start = [], None
    for i, on in enumerate(flags):
        if on and start is None:
            start = i
        elif not on and start is not None:
            spans.append((start + 1, i + 1))
            start = None
    if start is not None:
        spans.append((start + 1, len(flags)))
    return spans


def prompts_from_batch(batch, count: int, *, seed: int = 0, prefix_frac: float = 0.25, prefix_tokens: int = 768,
                       turns_only: bool = True) -> list[tuple[str, torch.Tensor]]:
    """Up to ``count`` ``(name, prompt_token_ids)`` pairs. A turn cut ends right before a trained span that has
    an untrained prefix; with ``turns_only=False`` documents without such a span fall back to the first
    ``prefix_frac`` of their tokens. Prompts are capped to their LAST ``prefix_tokens`` tokens."""
    rng = random.Random(seed)
    docs = batch_documents(batch)
    order = list(range(len(docs)))
    rng.shuffle(order)
    out = []
    for d in order:
        if len(out) >= count:
            break
        tokens, labels = docs[d]
        n = tokens.numel()
        cuts = [a for a, _ in trained_spans(labels) if a > 1]     # a trained span with something before it
        fully_trained = bool((labels[:-1] != IGNORE_INDEX).all()) if n > 1 else True
        if cuts and not fully_trained:
            cut = rng.choice(cuts)
            kind = "turn"
        elif not turns_only and n >= MIN_FILLER_TOKENS:
            cut = max(1, int(n * prefix_frac))
            kind = "prefix"
        else:
            continue
        prompt = tokens[max(0, cut - prefix_tokens):cut].clone()
        out.append((f"batch/{kind}/{d}", prompt))
    return out


def corpus_prompts(records: Sequence, render: Callable, encode: Callable[[str], Sequence[int]], count: int, *,
                   seed: int = 0, prefix_frac: float = 0.25, prefix_tokens: int = 768) -> list[tuple[str, torch.Tensor]]:
    """Prompts cut from held-out records: ``render(record)`` gives the text (or segments joined), the first
    ``prefix_frac`` of its tokens is the prompt."""
    rng = random.Random(seed)
    picks = rng.sample(range(len(records)), min(count, len(records)))
    out = []
    for i in picks:
        text = render(records[i])
        if not isinstance(text, str):
            text = "".join(seg[0] if isinstance(seg, (tuple, list)) else str(seg) for seg in text)
        ids = list(encode(text))
        if len(ids) < 2:
            continue
        cut = max(1, min(int(len(ids) * prefix_frac), prefix_tokens))
        out.append((f"corpus/{i}", torch.tensor(ids[:cut], dtype=torch.long)))
    return out
