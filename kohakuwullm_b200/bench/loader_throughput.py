"""Tokens per second of the data path alone: records -> renderer -> tokenizer -> packing, in process and with worker
processes, with nothing consuming the batches but a counter.

    python -m kohakuwullm_b200.bench.loader_throughput --workers 0 2 4 8 --seconds 5
    python -m kohakuwullm_b200.bench.loader_throughput --corpus data/en/web --tokenizer models/tokenizer --workers 0 8 16

Without ``--corpus`` a synthetic jsonl corpus of English-like text is written to a temporary directory (documents of
``--doc-chars`` characters on average, log-uniform between a tenth and ten times that), so the number depends on the
tokenizer and the host CPU only. The byte tokenizer is the floor of tokenizer cost; ``bpe:<vocab>`` trains a byte-level
BPE on the corpus itself and a tokenizer directory loads a real one: the figures a real run sees. One JSON line per
worker count: tokens / s, packs / s, mean tokens per pack (the fill of the token budget). A training job needs ``tokens/s of the model x ranks`` from this path, with headroom: a loader slower
than the step shows up as idle GPUs, not as an error. Reference: docs/internals/data.md (loader throughput by worker
count), scripts/bench/data/loader.py.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import random
import sys
import tempfile
import time

WORDS = ("the of and to in a is that for it as was with be by on not he this are or his from at which but have an had "
         "they you were their one all we can her has there been if more when will would who so no out up into than them "
         "time only some could these two may then do first any my now such like our over man me even most made after also "
         "did many before must through back years where much your way well down should because each just those people how "
         "too little state good very make world still own see men work long get here between both life being under never").split()


def write_synthetic_corpus(root: str, documents: int, doc_chars: int, seed: int = 0, shards: int = 4) -> int:
    """jsonl shards of word salad with sentence punctuation; returns the number of characters written."""
    rng = random.Random(seed)
    os.makedirs(root, exist_ok=True)
    total = 0
    files = [open(os.path.join(root, f"part-{i}.jsonl"), "w") for i in range(shards)]
    try:
        for d in range(documents):
            want = int(doc_chars * 10 ** rng.uniform(-1.0, 1.0))
            parts, n = [], 0
            while n < want:
                words = [rng.choice(WORDS) for _ in range(rng.randint(4, 18))]
                sentence = " ".join(words).capitalize() + rng.choice(".....?!")
                parts.append(sentence)
                n += len(sentence) + 1
            text = " ".join(parts)
            total += len(text)
            files[d % shards].write(json.dumps({"text": text}) + "\n")
    finally:
        for f in files:
            f.close()
    return total


class _FastBPE:
    """Picklable wrapper of a ``tokenizers.Tokenizer`` (worker processes rebuild it from its JSON)."""

    bos_token_id, eos_token_id = 0, 1

    def __init__(self, spec: str):
        from tokenizers import Tokenizer

        self.spec = spec
        self.tok = Tokenizer.from_str(spec)

    def encode(self, text: str) -> list[int]:
        return self.tok.encode(text).ids

    def __getstate__(self):
        return {"spec": self.spec}

    def __setstate__(self, state):
        self.__init__(state["spec"])


def train_bpe(root: str, vocab: int, sample_documents: int = 2000) -> _FastBPE:
    """A byte-level BPE of ``vocab`` ids trained on the first documents of the corpus: what a real tokenizer costs,
    without needing tokenizer files on the machine."""
    import glob

    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers

    texts = []
    for path in sorted(glob.glob(os.path.join(root, "*.jsonl"))):
        with open(path) as fh:
            for line in fh:
                texts.append(json.loads(line).get("text", ""))
                if len(texts) >= sample_documents:
                    break
        if len(texts) >= sample_documents:
            break
    tok = Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    trainer = trainers.BpeTrainer(vocab_size=vocab, special_tokens=["<bos>", "<eos>"], show_progress=False,
                                  initial_alphabet=pre_tokenizers.ByteLevel.alphabet())
    tok.train_from_iterator(texts, trainer)
    return _FastBPE(tok.to_str())


def measure(records, renderer, encode, *, workers: int, k: int, ctx_max: int, seconds: float, warmup_packs: int = 8,
            bos=None, eos=None) -> dict:
    from kohakuwullm_b200.data import build_loader

    common = dict(k=k, m=k // 16, ctx_max=ctx_max, seed=0, bos=bos, eos=eos)
    if workers > 0:
        loader = build_loader("workers", records, renderer, encode, workers=workers, **common)
    else:
        loader = build_loader("iterative", records, renderer, encode, **common)
    it = iter(loader)
    for _ in range(warmup_packs):
        next(it)
    tokens = packs = 0
    t0 = time.perf_counter()
    while True:
        batch = next(it)
        tokens += batch.num_tokens
        packs += 1
        dt = time.perf_counter() - t0
        if dt >= seconds:
            break
    close = getattr(getattr(loader, "loader", loader), "close", None)
    if callable(close):
        close()
    return {"workers": workers, "tokens_per_s": tokens / dt, "packs_per_s": packs / dt, "tokens_per_pack": tokens / packs,
            "fill": tokens / packs / k, "seconds": dt}


def main(argv=None) -> int:
    from kohakuwullm_b200.data import ByteTokenizer, build_dataset

    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--corpus", default=None, help="a directory of jsonl / txt shards (default: a synthetic one)")
    ap.add_argument("--documents", type=int, default=20000)
    ap.add_argument("--doc-chars", type=int, default=2000)
    ap.add_argument("--tokenizer", default="byte", help="byte, bpe:<vocab> (trained on the corpus), or a tokenizer directory")
    ap.add_argument("--renderer", default="plain")
    ap.add_argument("--workers", type=int, nargs="+", default=[0, 2, 4, 8])
    ap.add_argument("--pack-tokens", type=int, default=16384)
    ap.add_argument("--ctx-max", type=int, default=4096)
    ap.add_argument("--seconds", type=float, default=5.0)
    args = ap.parse_args(argv)
    tmp = None
    root = args.corpus
    if root is None:
        tmp = tempfile.TemporaryDirectory()
        root = tmp.name
        chars = write_synthetic_corpus(root, args.documents, args.doc_chars)
        print(json.dumps({"corpus": "synthetic", "documents": args.documents, "characters": chars}))
    if args.tokenizer == "byte":
        tok = ByteTokenizer()
    elif args.tokenizer.startswith("bpe:"):
        tok = train_bpe(root, int(args.tokenizer.split(":", 1)[1]))
    else:
        from transformers import AutoTokenizer

        tok = AutoTokenizer.from_pretrained(args.tokenizer)
    records, renderer = build_dataset({"name": "corpus", "root": root}, args.renderer)
    rows = []
    for w in args.workers:
        row = measure(records, renderer, tok.encode, workers=w, k=args.pack_tokens, ctx_max=args.ctx_max,
                      seconds=args.seconds, bos=getattr(tok, "bos_token_id", None), eos=getattr(tok, "eos_token_id", None))
        row.update(tokenizer=args.tokenizer, cpus=os.cpu_count(), pack_tokens=args.pack_tokens)
        rows.append(row)
        print(json.dumps(row))
    if tmp is not None:
        tmp.cleanup()
    best = max(rows, key=lambda r: r["tokens_per_s"])
    print(json.dumps({"best_workers": best["workers"], "best_tokens_per_s": best["tokens_per_s"],
                      "speedup_over_in_process": best["tokens_per_s"] / rows[0]["tokens_per_s"]
                      if rows[0]["workers"] == 0 and math.isfinite(rows[0]["tokens_per_s"]) else None}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
