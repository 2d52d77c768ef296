"""Corpus tools: what a data mixture decision needs before a run is planned.

    python -m kohakuwullm_b200.cli.data_tools census       --root DATA --out census.json
    python -m kohakuwullm_b200.cli.data_tools profile      --root DATA --tokenizer TOK_DIR --sample 2000
    python -m kohakuwullm_b200.cli.data_tools mixture      --stats profile.json --targets targets.json --budget 105e9
    python -m kohakuwullm_b200.cli.data_tools ngram-filter --root DATA/en/source --sample 20000 --show 3
    python -m kohakuwullm_b200.cli.data_tools token-census --records '{"name":"corpus","root":"DATA/en/source"}' \\
                                                           --renderer plain --limit 20000
    python -m kohakuwullm_b200.cli.data_tools to-corpus-chat --src chat.jsonl --dst DATA/sft/chat
    python -m kohakuwullm_b200.cli.data_tools to-vault-chat  --src chat.jsonl --root VAULT --corpus sft/chat

A corpus is laid out as ``<root>/<category>/<source>/*.jsonl`` (one JSON object per line). Everything streams:
memory is the counters, the duplicate table and one tokenizer batch. ``to-corpus-chat`` writes conversation
datasets as corpus shards with their manifest (byte offsets per record), the random-access layout the loaders
read. Reference: scripts/data/{dataset_census,dataset_profile,mixture,ngram_filter,token_census,to_vault_chat}.py.
"""

from __future__ import annotations

import argparse
import hashlib
import json
import os
import random
import statistics
import sys
from collections import Counter
from typing import Iterable, Iterator


def iter_sources(root: str) -> Iterator[tuple[str, list[str]]]:
    """(``category/source``, shard paths) for every source directory under ``root``; a directory that holds
    shards itself is one source named after it."""
    def shards(d):
        return sorted(os.path.join(d, f) for f in os.listdir(d) if f.endswith(".jsonl"))

    own = shards(root)
    if own:
        yield os.path.basename(os.path.normpath(root)), own
        return
    for cat in sorted(os.listdir(root)):
        cdir = os.path.join(root, cat)
        if not os.path.isdir(cdir):
            continue
        if shards(cdir):
            yield cat, shards(cdir)
            continue
        for src in sorted(os.listdir(cdir)):
            sdir = os.path.join(cdir, src)
            if os.path.isdir(sdir) and shards(sdir):
                yield f"{cat}/{src}", shards(sdir)


def iter_rows(paths: Iterable[str]) -> Iterator[dict]:
    for path in paths:
        with open(path, "rb") as f:
            for line in f:
                if line.strip():
                    try:
                        yield json.loads(line)
                    except json.JSONDecodeError:
                        yield {"__broken__": True}


def row_text(row: dict, fields=("text", "response", "output", "content")) -> str:
    for k in fields:
        v = row.get(k)
        if isinstance(v, str):
            return v
    msgs = row.get("messages")
    if isinstance(msgs, list):
        return "\n".join(str(m.get("content", "")) for m in msgs if isinstance(m, dict))
    return ""


def census(root: str, truncation_cap: int = 4000) -> dict:
    """Rows, fields, empty / truncated / duplicated shares per source. ``dup_frac`` counts a non-empty row whose
    text was seen before ANYWHERE in the corpus (64-bit hashes); ``truncated_frac`` rows whose text has exactly
    ``truncation_cap`` characters (a cap applied upstream leaves that fingerprint)."""
    seen: set[bytes] = set()
    out = {}
    for name, paths in iter_sources(root):
        rows = empty = dup = trunc = broken = 0
        fields: Counter = Counter()
        for row in iter_rows(paths):
            rows += 1
            if row.get("__broken__"):
                broken += 1
                continue
            fields.update(row.keys())
            text = row_text(row)
            if not text.strip():
                empty += 1
                continue
            if len(text) == truncation_cap:
                trunc += 1
            h = hashlib.blake2b(text.encode("utf-8", "replace"), digest_size=8).digest()
            if h in seen:
                dup += 1
            else:
                seen.add(h)
        nonempty = max(rows - empty - broken, 1)
        out[name] = {"rows": rows, "shards": len(paths), "fields": dict(fields), "broken_rows": broken,
                     "empty_frac": empty / max(rows, 1), "dup_frac": dup / nonempty, "truncated_frac": trunc / nonempty}
    return out


def profile(root: str, encode=None, sample: int = 2000, seed: int = 0) -> dict:
    """Characters, length percentiles, content markers and a token estimate per source. A bounded random sample
    of each source is really tokenised to fix that source's own characters-per-token ratio (code and prose
    differ by almost a factor of two, so one global constant would misprice the mixture)."""
    rng = random.Random(seed)
    out = {}
    for name, paths in iter_sources(root):
        lengths, picked, seen_rows = [], [], 0
        markers: Counter = Counter()
        for row in iter_rows(paths):
            text = row_text(row)
            seen_rows += 1
            lengths.append(len(text))
            markers["code_fence"] += "```" in text
            markers["url"] += "http://" in text or "https://" in text
            markers["non_ascii"] += any(ord(c) > 127 for c in text[:2000])
            if len(picked) < sample:                       # reservoir sample
                picked.append(text)
            else:
                j = rng.randrange(seen_rows)
                if j < sample:
                    picked[j] = text
        chars = sum(lengths)
        ratio = None
        if encode is not None and picked:
            toks = sum(len(encode(t)) for t in picked)
            ratio = sum(len(t) for t in picked) / max(toks, 1)
        qs = statistics.quantiles(lengths, n=100) if len(lengths) >= 2 else [lengths[0] if lengths else 0] * 99
        out[name] = {"rows": seen_rows, "chars": chars, "chars_per_token": ratio,
                     "est_tokens": (chars / ratio) if ratio else None, "mean_chars": chars / max(seen_rows, 1),
                     "p50": qs[49], "p90": qs[89], "p99": qs[98],
                     "markers": {k: v / max(seen_rows, 1) for k, v in markers.items()}}
    return out


def mixture(stats: dict, targets: dict, budget: float | None = None, absorb: str | None = None) -> dict:
    """Per-source ``repeat`` weights for a target TOKEN mixture. ``stats``: source -> {"rows", "est_tokens"}
    (the output of ``profile``); ``targets``: source -> target tokens (scaled to ``budget`` when given). A
    source smaller than its target is repeated at most ``max_repeat`` = 4 times; the shortfall goes to
    ``absorb`` (or is spread over the sources with room, in proportion to their targets)."""
    max_repeat = 4.0
    total_target = sum(targets.values())
    scale = (budget / total_target) if budget else 1.0
    want = {k: v * scale for k, v in targets.items()}
    have = {k: float(stats[k]["est_tokens"]) for k in targets}
    repeat = {k: min(want[k] / have[k], max_repeat) for k in targets}
    short = sum(want[k] - repeat[k] * have[k] for k in targets)
    if short > 1e-9:
        takers = [absorb] if absorb else [k for k in targets if repeat[k] < max_repeat]
        room = sum(want[k] for k in takers) or 1.0
        for k in takers:
            repeat[k] = min((repeat[k] * have[k] + short * want[k] / room) / have[k], max_repeat if not absorb else 1e9)
    tokens = {k: repeat[k] * have[k] for k in targets}
    whole = sum(tokens.values())
    return {k: {"repeat": repeat[k], "tokens": tokens[k], "share": tokens[k] / whole,
                "documents": repeat[k] * stats[k]["rows"]} for k in targets}


def ngram_scan(paths, sample: int, max_n: int, threshold: int, show: int) -> dict:
    from kohakuwullm_b200.data.filters import longest_consecutive_repeat, text_units

    rejected, worst, n = 0, [], 0
    for row in iter_rows(paths):
        if sample and n >= sample:          # a prefix: shards are shuffled when they are written
            break
        n += 1
        text = row_text(row)
        reps, gram = longest_consecutive_repeat(text_units(text), max_n)
        if reps >= threshold:
            rejected += 1
        worst.append((reps, gram, text[:200]))
        worst = sorted(worst, reverse=True)[:max(show, 1)]
    return {"documents": n, "rejected": rejected, "rejected_frac": rejected / max(n, 1),
            "worst": [{"repeats": r, "n": g, "head": t} for r, g, t in worst[:show]]}


def token_census(records_spec, renderer_spec, encode, limit: int, max_length: int | None = None, seed: int = 0) -> dict:
    """Tokens per epoch, measured on a sample THROUGH the loader's own render + tokenise + collate path (a
    record's rendered length is not a function of anything cheap to look up); the record count is exact, only
    the mean length is estimated, with its standard error."""
    from kohakuwullm_b200.data import build_dataset
    from kohakuwullm_b200.data.loader.iterative import tokenize_segments
    from kohakuwullm_b200.data.packing import collate_packed

    records, renderer = build_dataset(records_spec, renderer_spec)
    rng = random.Random(seed)
    n = len(records)
    ids = range(n) if limit >= n else rng.sample(range(n), limit)
    counts, trained = [], 0
    for i in ids:
        sample = tokenize_segments(renderer(records[i], None), encode, None, None)
        batch = collate_packed([sample])
        t = int(batch.num_tokens if max_length is None else min(batch.num_tokens, max_length))
        counts.append(t)
        trained += int((batch.labels[:t] >= 0).sum())
    mean = statistics.fmean(counts) if counts else 0.0
    sem = (statistics.pstdev(counts) / max(len(counts), 1) ** 0.5) if len(counts) > 1 else 0.0
    return {"records": n, "sampled": len(counts), "mean_tokens": mean, "sem": sem, "epoch_tokens": mean * n,
            "trained_share": trained / max(sum(counts), 1)}


def to_corpus_chat(src: str, dst: str, rows_per_shard: int = 200_000) -> dict:
    """Conversation rows (``{"messages": [{"role", "content"}, ...]}`` or ``{"conversations": [...]}``) -> corpus
    shards ``dst/part-00000.jsonl`` ... plus ``manifest.json``; read them with ``{"name": "corpus", "root": dst}`` records and
    render them with ``chatml``."""
    from kohakuwullm_b200.data.sources.records import CorpusRecords

    os.makedirs(dst, exist_ok=True)
    paths = [src] if os.path.isfile(src) else sorted(os.path.join(src, f) for f in os.listdir(src) if f.endswith(".jsonl"))
    shard, rows, kept, dropped, out = 0, 0, 0, 0, None
    for row in iter_rows(paths):
        msgs = row.get("messages") or row.get("conversations")
        if not isinstance(msgs, list) or not msgs:
            dropped += 1
            continue
        clean = [{"role": str(m.get("role") or m.get("from") or "user"), "content": str(m.get("content") or m.get("value") or "")}
                 for m in msgs if isinstance(m, dict)]
        if out is None or rows >= rows_per_shard:
            if out:
                out.close()
            out = open(os.path.join(dst, f"part-{shard:05d}.jsonl"), "w")
            shard, rows = shard + 1, 0
        out.write(json.dumps({"messages": clean}, ensure_ascii=False) + "\n")
        rows += 1
        kept += 1
    if out:
        out.close()
    manifest = CorpusRecords.build_manifest(dst)
    with open(os.path.join(dst, CorpusRecords.MANIFEST), "w") as f:
        json.dump(manifest, f)
    return {"kept": kept, "dropped": dropped, "shards": shard}


def to_vault_chat(src: str, root: str, corpus: str, rows_per_shard: int = 200_000) -> dict:
    """The same conversion into key-value shards ``root/corpus/part-NNNNN.kv`` with sequential int64 keys; read them
    with ``{"name": "vault_corpus", "corpus": corpus, "root": root, "schema": "json"}``."""
    from kohakuwullm_b200.data.sources.kvstore import KVWriter

    d = os.path.join(root, corpus)
    os.makedirs(d, exist_ok=True)
    paths = [src] if os.path.isfile(src) else sorted(os.path.join(src, f) for f in os.listdir(src) if f.endswith(".jsonl"))
    shard, rows, kept, dropped, out = 0, 0, 0, 0, None
    for row in iter_rows(paths):
        msgs = row.get("messages") or row.get("conversations")
        if not isinstance(msgs, list) or not msgs:
            dropped += 1
            continue
        if out is None or rows >= rows_per_shard:
            if out:
                out.close()
            out = KVWriter(os.path.join(d, f"part-{shard:05d}.kv"))
            shard, rows = shard + 1, 0
        out.put(kept, {"messages": [{"role": str(m.get("role") or m.get("from") or "user"),
                                     "content": str(m.get("content") or m.get("value") or "")} for m in msgs if isinstance(m, dict)]})
        rows += 1
        kept += 1
    if out:
        out.close()
    return {"kept": kept, "dropped": dropped, "shards": shard}


def _encoder(path: str | None):
    if not path:
        from kohakuwullm_b200.data import ByteTokenizer

        return ByteTokenizer().encode
    from tokenizers import Tokenizer

    tok = Tokenizer.from_file(os.path.join(path, "tokenizer.json") if os.path.isdir(path) else path)
    return lambda text: tok.encode(text).ids


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("census"); p.add_argument("--root", required=True); p.add_argument("--cap", type=int, default=4000)
    p = sub.add_parser("profile"); p.add_argument("--root", required=True); p.add_argument("--tokenizer"); p.add_argument("--sample", type=int, default=2000)
    p = sub.add_parser("mixture"); p.add_argument("--stats", required=True); p.add_argument("--targets", required=True)
    p.add_argument("--budget", type=float); p.add_argument("--absorb")
    p = sub.add_parser("ngram-filter"); p.add_argument("--root", required=True); p.add_argument("--sample", type=int, default=20000)
    p.add_argument("--max-n", type=int, default=13); p.add_argument("--threshold", type=int, default=32); p.add_argument("--show", type=int, default=3)
    p = sub.add_parser("token-census"); p.add_argument("--records", required=True); p.add_argument("--renderer", default="plain")
    p.add_argument("--tokenizer"); p.add_argument("--limit", type=int, default=20000); p.add_argument("--max-length", type=int)
    p = sub.add_parser("to-corpus-chat"); p.add_argument("--src", required=True); p.add_argument("--dst", required=True)
    p.add_argument("--rows-per-shard", type=int, default=200_000)
    p = sub.add_parser("to-vault-chat"); p.add_argument("--src", required=True); p.add_argument("--root", required=True)
    p.add_argument("--corpus", required=True); p.add_argument("--rows-per-shard", type=int, default=200_000)
    for sp in sub.choices.values():
        sp.add_argument("--out", help="write the JSON result here instead of stdout")
    a = ap.parse_args(argv)
    if a.cmd == "census":
        res = census(a.root, a.cap)
    elif a.cmd == "profile":
        res = profile(a.root, _encoder(a.tokenizer), a.sample)
    elif a.cmd == "mixture":
        with open(a.stats) as f, open(a.targets) as g:
            res = mixture(json.load(f), json.load(g), a.budget, a.absorb)
    elif a.cmd == "ngram-filter":
        res = {name: ngram_scan(paths, a.sample, a.max_n, a.threshold, a.show) for name, paths in iter_sources(a.root)}
    elif a.cmd == "token-census":
        spec = json.loads(a.records) if a.records.lstrip().startswith("{") else a.records
        rend = json.loads(a.renderer) if a.renderer.lstrip().startswith("{") else a.renderer
        res = token_census(spec, rend, _encoder(a.tokenizer), a.limit, a.max_length)
    elif a.cmd == "to-vault-chat":
        res = to_vault_chat(a.src, a.root, a.corpus, a.rows_per_shard)
    else:
        res = to_corpus_chat(a.src, a.dst, a.rows_per_shard)
    text = json.dumps(res, indent=1, ensure_ascii=False)
    if a.out:
        os.makedirs(os.path.dirname(os.path.abspath(a.out)), exist_ok=True)
        with open(a.out, "w") as f:
            f.write(text)
    else:
        print(text)
    return 0


if __name__ == "__main__":
    sys.exit(main())
