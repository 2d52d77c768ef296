"""Prune a byte-level BPE tokenizer to a fixed vocabulary size.

BPE ids are assigned in merge order, so keeping the first ``n`` ids keeps the ``n`` most frequent merges
and every merge whose parts survive. The pruned vocabulary = first ``base`` ids (bytes + earliest merges)
+ named special tokens + reserved ``<|reserved_i|>`` slots up to ``target`` (65536 by default).
Works on the ``tokenizer.json`` structure (vocab + merges), no network needed.
Reference: src/kohakuwullm/tokenizer/prune.py:16-115."""

from __future__ import annotations

import json


def prune_tokenizer_json(data: dict, target: int = 65536, specials: list[str] | None = None,
                         reserved_prefix: str = "<|reserved_{}|>", base: int | None = None) -> dict:
    """``base``: how many ordinary ids to keep (default: all that fit next to the specials). With a smaller
    ``base`` the ids between the specials and ``target`` become reserved placeholders, so a control token
    added later is an id assignment, not a re-embedding."""
    specials = list(specials or [])
    model = data["model"]
    vocab = model["vocab"]
    if base is None:
        base = target - len(specials)
    if base <= 0 or base + len(specials) > target:
        raise ValueError("target vocabulary is smaller than the ordinary ids plus the special-token list")
    keep = {tok: i for tok, i in vocab.items() if i < base}
    merges = []
    for m in model.get("merges", []):
        a, b = m if isinstance(m, (list, tuple)) else m.split(" ", 1)
        if a in keep and b in keep and (a + b) in keep:
            merges.append(m)
    new_vocab = dict(keep)
    next_id = max(new_vocab.values()) + 1 if new_vocab else 0
    added = []
    for tok in specials:
        new_vocab[tok] = next_id
        added.append({"id": next_id, "content": tok, "single_word": False, "lstrip": False, "rstrip": False,
                      "normalized": False, "special": True})
        next_id += 1
    r = 0
    while next_id < target:
        tok = reserved_prefix.format(r)
        new_vocab[tok] = next_id
        added.append({"id": next_id, "content": tok, "single_word": False, "lstrip": False, "rstrip": False,
                      "normalized": False, "special": True})
        next_id += 1
        r += 1
    out = json.loads(json.dumps(data))
    out["model"]["vocab"] = new_vocab
    out["model"]["merges"] = merges
    out["added_tokens"] = added
    return out


def prune_file(src: str, dst: str, target: int = 65536, specials: list[str] | None = None,
               base: int | None = None) -> None:
    with open(src) as f:
        data = json.load(f)
    with open(dst, "w") as f:
        json.dump(prune_tokenizer_json(data, target, specials, base=base), f, ensure_ascii=False)
