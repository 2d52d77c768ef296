"""Build the training tokenizer from a byte-level BPE ``tokenizer.json`` on disk.

    python -m kohakuwullm_b200.cli.build_tokenizer --source SRC/tokenizer.json --out models/tokenizer
    python -m kohakuwullm_b200.cli.build_tokenizer --source SRC --out models/tokenizer \\
        --check-corpus data/en/web/part-0.jsonl --check-samples 2000

The result has exactly ``--target`` (65536) ids:

    [0, base)            ordinary BPE tokens in merge order (``--base``, 64000)
    [base, base + n)     named specials: BOS / EOS / PAD / UNK, the ChatML markers, the TIPO task vocabulary
    [., target)          ``<|reserved_i|>`` placeholders

A power-of-two vocabulary keeps the head GEMM's N dimension tile-aligned (65536 = 512 tiles of 128), and the
reserved block makes a later control token an id assignment instead of a re-embedding. BOS is prepended by the
post-processor. With ``--check-corpus`` a sample of real text is tokenised with the source and the pruned
tokenizer and the change in tokens per sample is reported: pruning that quietly lengthens every sequence costs
more than the embedding rows it saves, so it is measured. No network: the source tokenizer is a local file.
Reference: scripts/tokenizer/build_tokenizer.py:1-168.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

from kohakuwullm_b200.tokenizer.prune import prune_tokenizer_json

CORE_SPECIALS = ["<|bos|>", "<|eos|>", "<|pad|>", "<|unk|>"]
CHAT_SPECIALS = ["<|im_start|>", "<|im_end|>"]


def tipo_specials() -> list[str]:
    from kohakuwullm_b200.data.renderers.base import TIPORenderer

    return [f"<|{name}|>" for name in TIPORenderer.LENGTHS] + [f"<|{t}|>" for t in TIPORenderer.TASKS]


def with_bos(post_processor: dict | None, bos: str, bos_id: int) -> dict:
    """The existing post-processor followed by one that prepends BOS to single sequences and pairs."""
    template = {
        "type": "TemplateProcessing",
        "single": [{"SpecialToken": {"id": bos, "type_id": 0}}, {"Sequence": {"id": "A", "type_id": 0}}],
        "pair": [{"SpecialToken": {"id": bos, "type_id": 0}}, {"Sequence": {"id": "A", "type_id": 0}},
                 {"Sequence": {"id": "B", "type_id": 1}}],
        "special_tokens": {bos: {"id": bos, "ids": [bos_id], "tokens": [bos]}},
    }
    if not post_processor:
        return template
    return {"type": "Sequence", "processors": [post_processor, template]}


def build(source_json: dict, base: int, target: int, extra_specials: list[str] | None = None) -> dict:
    specials = CORE_SPECIALS + CHAT_SPECIALS + tipo_specials() + list(extra_specials or [])
    specials = list(dict.fromkeys(specials))
    out = prune_tokenizer_json(source_json, target=target, specials=specials, base=base)
    bos_id = out["model"]["vocab"]["<|bos|>"]
    out["post_processor"] = with_bos(source_json.get("post_processor"), "<|bos|>", bos_id)
    return out


def tokens_per_sample(tokenizer_json: dict, texts: list[str]) -> float:
    from tokenizers import Tokenizer

    tok = Tokenizer.from_str(json.dumps(tokenizer_json))
    return sum(len(tok.encode(t).ids) for t in texts) / max(len(texts), 1)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--source", required=True, help="tokenizer.json, or a directory that holds one")
    ap.add_argument("--out", required=True)
    ap.add_argument("--base", type=int, default=64000)
    ap.add_argument("--target", type=int, default=65536)
    ap.add_argument("--specials", help="JSON list of further named special tokens")
    ap.add_argument("--check-corpus", help="a .jsonl shard with a 'text' field")
    ap.add_argument("--check-samples", type=int, default=2000)
    a = ap.parse_args(argv)
    src = os.path.join(a.source, "tokenizer.json") if os.path.isdir(a.source) else a.source
    with open(src) as f:
        source = json.load(f)
    extra = json.loads(a.specials) if a.specials else None
    built = build(source, a.base, a.target, extra)
    os.makedirs(a.out, exist_ok=True)
    with open(os.path.join(a.out, "tokenizer.json"), "w") as f:
        json.dump(built, f, ensure_ascii=False)
    with open(os.path.join(a.out, "tokenizer_config.json"), "w") as f:
        json.dump({"tokenizer_class": "PreTrainedTokenizerFast", "bos_token": "<|bos|>", "eos_token": "<|eos|>",
                   "pad_token": "<|pad|>", "unk_token": "<|unk|>", "model_max_length": 1 << 30}, f, indent=1)
    with open(os.path.join(a.out, "special_tokens_map.json"), "w") as f:
        json.dump({"bos_token": "<|bos|>", "eos_token": "<|eos|>", "pad_token": "<|pad|>", "unk_token": "<|unk|>"}, f, indent=1)
    report = {"vocab": len(built["model"]["vocab"]), "merges": len(built["model"]["merges"]),
              "named_specials": sum(1 for t in built["added_tokens"] if not t["content"].startswith("<|reserved_")),
              "reserved": sum(1 for t in built["added_tokens"] if t["content"].startswith("<|reserved_"))}
    if a.check_corpus:
        texts = []
        with open(a.check_corpus) as f:
            for line in f:
                if len(texts) >= a.check_samples:
                    break
                if line.strip():
                    texts.append(str(json.loads(line).get("text", "")))
        before = tokens_per_sample(source, texts)
        # the comparison is about the BPE body: measure the pruned tokenizer without its BOS
        after = tokens_per_sample({**built, "post_processor": source.get("post_processor")}, texts)
        report.update(samples=len(texts), tokens_per_sample_source=before, tokens_per_sample_pruned=after,
                      length_ratio=after / max(before, 1e-9))
    print(json.dumps(report))
    return 0


if __name__ == "__main__":
    sys.exit(main())
