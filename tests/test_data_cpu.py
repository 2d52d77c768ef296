"""Data pipeline: permutation, packing, label shifting, loaders and exact resume."""

import random

import pytest
import torch
from hypothesis import given, settings, strategies as st

from kohakuwullm_b200.data import (ByteTokenizer, FeistelPermutation, IterativePackLoader, MicroBatchedLoader,
                                   ResumableLoader, ShardIndices, collate_packed, collate_padded, is_validation,
                                   split_packed, split_padded)
from kohakuwullm_b200.data.filters import ngram_repeat_ratio, passes_repeat_filter
from kohakuwullm_b200.data.renderers.base import ChatMLRenderer, PlainRenderer, TIPORenderer
from kohakuwullm_b200.data.sources.records import CorpusRecords, ListRecords


@settings(max_examples=40, deadline=None)
@given(st.integers(1, 3000), st.integers(0, 2 ** 40))
def test_feistel_is_a_permutation(n, key):
    perm = FeistelPermutation(n, key)
    assert sorted(perm(i) for i in range(n)) == list(range(n))


def test_shards_partition_every_epoch_and_epochs_differ():
    n, shards = 103, 4
    for epoch in (0, 1):
        seen = []
        for s in range(shards):
            seen += [idx for _, idx in ShardIndices(n, s, shards, seed=5).iterate(epoch)]
        assert sorted(seen) == list(range(n))
    a = [i for _, i in ShardIndices(n, 0, 1, seed=5).iterate(0)]
    b = [i for _, i in ShardIndices(n, 0, 1, seed=5).iterate(1)]
    assert a != b


def test_validation_split_is_stable():
    flags = [is_validation(f"doc{i}", 0.1, seed=3) for i in range(2000)]
    assert 120 < sum(flags) < 280
    assert flags == [is_validation(f"doc{i}", 0.1, seed=3) for i in range(2000)]


def test_labels_are_shifted_inside_each_document():
    a, b = torch.tensor([1, 2, 3, 4]), torch.tensor([7, 8, 9])
    batch = collate_packed([a, (b, torch.tensor([False, False, True])), torch.tensor([5])])
    assert batch.tokens.tolist() == [1, 2, 3, 4, 7, 8, 9]
    assert batch.labels.tolist() == [2, 3, 4, -100, -100, 9, -100]   # no target crosses a boundary
    assert batch.seq_info.cu_seqlens.tolist() == [0, 4, 7]
    assert batch.seq_info.position_ids.tolist() == [0, 1, 2, 3, 0, 1, 2]


def test_split_packed_is_document_aligned_and_complete():
    docs = [torch.arange(n) + 10 * n for n in (9, 3, 7, 5, 2, 8)]
    whole = collate_packed(docs)
    parts = split_packed(whole, 3)
    assert sum(p.num_tokens for p in parts) == whole.num_tokens
    assert sum(p.trained_tokens() for p in parts) == whole.trained_tokens()
    sizes = sorted(p.num_tokens for p in parts)
    assert sizes[-1] - sizes[0] <= 9


def test_padded_twin():
    batch = collate_padded([torch.arange(5), torch.arange(3)], pad_id=0)
    assert batch.tokens.shape == (2, 5) and batch.labels[1].tolist() == [1, 2, -100, -100, -100]
    assert [p.tokens.shape[0] for p in split_padded(batch, 2)] == [1, 1]


def test_renderers_mark_trained_roles_only():
    chat = ChatMLRenderer()
    segs = chat({"messages": [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "yo"}]})
    assert [t for _, t in segs] == [False, False, False, True]
    assert PlainRenderer()("abc") == [("abc", True)]
    rec = {"tags": [f"t{i}" for i in range(12)], "caption": "A long caption. More.", "rating": "g"}
    prompt, completion = TIPORenderer()(rec, random.Random(1))
    assert prompt[1] is False and completion[1] is True


def _loader(records, **kw):
    tok = ByteTokenizer()
    return IterativePackLoader(records, PlainRenderer(), tok.encode, k=64, m=16, bos=tok.bos_token_id,
                               eos=tok.eos_token_id, seed=7, **kw)


def test_iterative_loader_respects_budget_and_resumes_exactly():
    records = ListRecords([{"text": "x" * n} for n in random.Random(0).choices(range(3, 50), k=200)])
    full = []
    it = iter(ResumableLoader(_loader(records)))
    for _ in range(12):
        full.append(next(it))
    assert all(48 <= b.num_tokens <= 64 for b in full[:-1])
    # stop after 5 batches, checkpoint, resume in a new loader: the stream continues identically
    first = ResumableLoader(_loader(records))
    it = iter(first)
    head = [next(it) for _ in range(5)]
    state = first.state_dict()
    second = ResumableLoader(_loader(records))
    second.load_state_dict(state)
    it2 = iter(second)
    tail = [next(it2) for _ in range(7)]
    for a, b in zip(head + tail, full):
        assert torch.equal(a.tokens, b.tokens) and torch.equal(a.labels, b.labels)
    with pytest.raises(ValueError):
        ResumableLoader(_loader(records, shard=1, shards=2)).load_state_dict(state)


def test_pipeline_loader_emits_exact_microbatches():
    tok = ByteTokenizer()
    records = ListRecords([{"text": "y" * n} for n in random.Random(1).choices(range(3, 90), k=100)])
    loader = MicroBatchedLoader(records, PlainRenderer(), tok.encode, k=64, num_microbatches=3, seed=1)
    step, _ = next(iter(loader))
    assert len(step) == 3 and all(m.num_tokens == 64 for m in step)


def test_corpus_records_and_manifest(tmp_path):
    (tmp_path / "a.jsonl").write_text('{"text": "one"}\n{"text": "two"}\n')
    (tmp_path / "b.txt").write_text("three\n\nfour\n")
    corpus = CorpusRecords(str(tmp_path))
    assert len(corpus) == 4 and [corpus[i]["text"] for i in range(4)] == ["one", "two", "three", "four"]
    assert (tmp_path / "manifest.json").exists()


def test_repeat_filter():
    assert ngram_repeat_ratio(list(range(100))) == 0.0
    assert not passes_repeat_filter([1, 2, 3, 4] * 30)


@pytest.mark.timeout(120)
def test_worker_process_loader_matches_in_process_shards_and_resumes():
    """Packs rendered in worker processes: the stream is the round-robin interleave of the per-worker shards the
    in-process loader produces, it resumes exactly (consumed position, not produced), and a state written with
    another worker count is refused."""
    from kohakuwullm_b200.data.loader.workers import WorkerPackLoader

    tok = ByteTokenizer()
    records = ListRecords([{"text": "z" * n} for n in random.Random(2).choices(range(3, 50), k=300)])
    kw = dict(k=64, m=16, seed=3, bos=tok.bos_token_id, eos=tok.eos_token_id)

    def make(workers=2):
        return ResumableLoader(WorkerPackLoader(records, PlainRenderer(), tok.encode, workers=workers, rank=1, world=2, **kw))

    full_loader = make()
    it = iter(full_loader)
    full = [next(it) for _ in range(10)]
    full_loader.loader.close()
    # the same shards, in process: worker w of rank 1 of 2 is shard 2 + w of 4
    shards = [iter(IterativePackLoader(records, PlainRenderer(), tok.encode, shard=2 + w, shards=4, **kw)) for w in range(2)]
    for i, b in enumerate(full):
        want, _ = next(shards[i % 2])
        assert torch.equal(b.tokens, want.tokens) and torch.equal(b.labels, want.labels)
    # resume after 5 consumed batches (the workers had produced more than that)
    first = make()
    it = iter(first)
    head = [next(it) for _ in range(5)]
    state = first.state_dict()
    first.loader.close()
    second = make()
    second.load_state_dict(state)
    it2 = iter(second)
    tail = [next(it2) for _ in range(5)]
    second.loader.close()
    for a, b in zip(head + tail, full):
        assert torch.equal(a.tokens, b.tokens)
    with pytest.raises(ValueError, match="worker processes"):
        make(workers=3).load_state_dict(state)
    # a failing renderer in a worker surfaces in the trainer process
    def broken(record, rng):
        raise KeyError("no such field")

    bad = WorkerPackLoader(records, broken, tok.encode, workers=1, **kw)
    with pytest.raises(RuntimeError, match="loader worker 0 failed: KeyError"):
        next(iter(bad))


def test_corpus_tools_census_profile_mixture_and_chat_conversion(tmp_path):
    import json

    from kohakuwullm_b200.cli import data_tools as dt
    from kohakuwullm_b200.data import ByteTokenizer
    from kohakuwullm_b200.data.filters import longest_consecutive_repeat, passes_consecutive_repeat_filter, text_units

    root = tmp_path / "data"
    a, b = root / "en" / "web", root / "code" / "repo"
    a.mkdir(parents=True)
    b.mkdir(parents=True)
    web = [{"text": f"document number {i} " * 5} for i in range(40)] + [{"text": "document number 3 " * 5}, {"text": " "}]
    code = [{"text": "```python\nprint(%d)\n```" % i, "lang": "py"} for i in range(10)] + [{"text": "x" * 4000}]
    (a / "part-0.jsonl").write_text("\n".join(json.dumps(r) for r in web) + "\n")
    (b / "part-0.jsonl").write_text("\n".join(json.dumps(r) for r in code) + "\nnot json\n")
    cen = dt.census(str(root))
    assert set(cen) == {"en/web", "code/repo"}
    assert cen["en/web"]["rows"] == 42 and abs(cen["en/web"]["dup_frac"] - 1 / 41) < 1e-9
    assert cen["en/web"]["empty_frac"] == 1 / 42
    assert cen["code/repo"]["broken_rows"] == 1 and cen["code/repo"]["truncated_frac"] == 1 / 11
    assert cen["code/repo"]["fields"]["lang"] == 10

    prof = dt.profile(str(root), ByteTokenizer().encode, sample=8)
    assert prof["code/repo"]["markers"]["code_fence"] == 10 / 12
    assert abs(prof["en/web"]["chars_per_token"] - 1.0) < 1e-9          # a byte tokenizer on ASCII
    assert prof["en/web"]["est_tokens"] == prof["en/web"]["chars"]

    stats = {"big": {"rows": 1000, "est_tokens": 1e6}, "small": {"rows": 10, "est_tokens": 1e4}}
    mix = dt.mixture(stats, {"big": 0.5e6, "small": 0.5e6})
    assert mix["small"]["repeat"] == 4.0                                  # capped: the rest goes to the big source
    assert abs(sum(v["tokens"] for v in mix.values()) - 1e6) < 1e-3
    assert abs(mix["big"]["tokens"] - (1e6 - 4e4)) < 1e-3

    assert longest_consecutive_repeat("a b a b a b c".split(), 5) == (3, 2)
    assert longest_consecutive_repeat(list("xyz"), 5) == (1, 1)
    assert text_units("ab " + "Q" * 50)[:2] == ["ab", "Q"] and len(text_units("ab " + "Q" * 50)) == 51
    assert not passes_consecutive_repeat_filter("spam " * 40) and passes_consecutive_repeat_filter("one two three four")
    scan = dt.ngram_scan([str(a / "part-0.jsonl")], sample=0, max_n=13, threshold=5, show=1)
    assert scan["documents"] == 42 and scan["rejected"] >= 41 and scan["worst"][0]["repeats"] >= 5

    chat = tmp_path / "chat.jsonl"
    chat.write_text("\n".join(json.dumps(r) for r in [
        {"messages": [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "hello"}]},
        {"conversations": [{"from": "human", "value": "2+2?"}, {"from": "gpt", "value": "4"}]},
        {"text": "no conversation here"}]) + "\n")
    res = dt.to_corpus_chat(str(chat), str(tmp_path / "sft"), rows_per_shard=1)
    assert res == {"kept": 2, "dropped": 1, "shards": 2}
    tc = dt.token_census({"name": "corpus", "root": str(tmp_path / "sft")}, "chatml", ByteTokenizer().encode, limit=10)
    assert tc["records"] == 2 and tc["sampled"] == 2 and tc["mean_tokens"] > 10 and 0 < tc["trained_share"] < 1
    assert dt.to_vault_chat(str(chat), str(tmp_path / "vault"), "sft/chat", rows_per_shard=1) == {"kept": 2, "dropped": 1, "shards": 2}
    tv = dt.token_census({"name": "vault_corpus", "corpus": "sft/chat", "root": str(tmp_path / "vault"), "schema": "json"},
                         "chatml", ByteTokenizer().encode, limit=10)
    assert tv["records"] == 2 and tv["mean_tokens"] == tc["mean_tokens"]      # the same rows through the other store
    assert dt.main(["census", "--root", str(root), "--out", str(tmp_path / "out" / "census.json")]) == 0
    assert json.loads((tmp_path / "out" / "census.json").read_text())["en/web"]["rows"] == 42


def test_kv_store_and_vault_style_sources(tmp_path):
    import os
    import random

    from kohakuwullm_b200.data import build_dataset
    from kohakuwullm_b200.data.sources.kvstore import KVFile, KVWriter, TagRecords, VaultCorpusRecords, quality_of

    # the store: any key order, three value kinds, last write wins, integer keys sort numerically
    path = str(tmp_path / "a.kv")
    with KVWriter(path) as w:
        for i in (5, 3, 300, 4):
            w.put(i, f"doc {i}")
        w.put("blob", b"\x00\x01")
        w.put("meta", {"n": 1})
        w.put("meta", {"n": 2})
    kv = KVFile(path)
    assert len(kv) == 6 and kv.get(300) == "doc 300" and kv.get("blob") == b"\x00\x01" and kv.get("meta") == {"n": 2}
    assert kv.get(7) is None and [k for k in kv.keys() if len(k) == 8] == sorted(k for k in kv.keys() if len(k) == 8)
    kv._pid = -1                      # what a forked loader worker sees: the mapping belongs to another process
    assert kv.get(3) == "doc 3" and kv._pid == os.getpid()
    import pickle

    assert pickle.loads(pickle.dumps(kv)).get(5) == "doc 5"          # travels to spawned workers by path
    (tmp_path / "cut.kv").write_bytes(open(path, "rb").read()[:-10])
    with pytest.raises(ValueError):
        KVFile(str(tmp_path / "cut.kv"))

    # corpus shards with sequential ids, text and conversation schemas, snapshot check
    d = tmp_path / "vault" / "en" / "web"
    d.mkdir(parents=True)
    for s in range(2):
        with KVWriter(str(d / f"part-{s}.kv")) as w:
            for i in range(3):
                w.put(s * 3 + i, f"text {s * 3 + i}")
    corpus = VaultCorpusRecords("en/web", str(tmp_path / "vault"))
    assert len(corpus) == 6 and corpus[4] == {"text": "text 4", "source": "en/web"} and corpus.snapshot() == [3, 3]
    with pytest.raises(ValueError):
        VaultCorpusRecords("en/web", str(tmp_path / "vault"), snapshot=[3, 2])
    records, renderer = build_dataset({"name": "vault_corpus", "corpus": "en/web", "root": str(tmp_path / "vault")}, "plain")
    assert len(records) == 6 and renderer(records[0], None)[0][0].startswith("text 0")

    # tag records joined with captions, rendered by the TIPO renderer
    with KVWriter(str(tmp_path / "meta.kv")) as w:
        w.put("00000012", {"id": 12, "general": ["1girl", "smile"], "artist": ["someone"], "character": ["alice"],
                           "copyright": [], "meta": ["highres"], "rating": "g", "score": 120, "width": 800, "height": 1200,
                           "year": 2021, "has_image": True})
        w.put("00000013", {"id": 13, "general": ["tree"], "score": -3})
    with KVWriter(str(tmp_path / "cap.kv")) as w:
        w.put("/img/12.webp", {"brief": "a girl", "description": "a smiling girl under a tree", "title": "t"})
    tags = TagRecords(str(tmp_path / "meta.kv"), str(tmp_path / "cap.kv"), caption_key="/img/{id}.webp")
    assert len(tags) == 2 and quality_of(120) == "best quality" and quality_of(-3) == "worst quality"
    r = tags[0]
    assert r["quality"] == "best quality" and r["long"].startswith("a smiling") and r["aspect_ratio"] == 0.67
    assert tags[1]["long"] is None and tags[1]["tags"] == ["tree"]                      # tag-only post
    assert len(TagRecords(str(tmp_path / "meta.kv"), image_only=True)) == 1
    from kohakuwullm_b200.data.renderers.base import TIPORenderer

    segs = TIPORenderer()(r, random.Random(0))
    assert len(segs) == 2 and segs[1][1] is True and "<|" in segs[0][0]


def test_mixture_and_split_records():
    from kohakuwullm_b200.data import build_dataset
    from kohakuwullm_b200.data.sources.records import ListRecords, MixtureRecords, SplitRecords

    a = ListRecords([{"text": f"a{i}"} for i in range(10)])
    b = ListRecords([{"text": f"b{i}", "source": "given"} for i in range(4)])
    mix = MixtureRecords([{"records": a, "repeat": 1.5, "source": "web"}, {"records": b, "repeat": 3}])
    assert len(mix) == 15 + 12 and mix.composition() == {"web": 15, "source1": 12}
    texts = [mix[i]["text"] for i in range(len(mix))]
    assert texts[:10] == [f"a{i}" for i in range(10)]
    tail = texts[10:15]
    assert len(set(tail)) == 5 and set(tail) <= {f"a{i}" for i in range(10)}         # half of the source, no repeats
    assert [mix[i]["text"] for i in range(10, 15)] == tail                           # and always the same half
    assert texts[15:] == [f"b{i % 4}" for i in range(12)]
    assert mix[0]["source"] == "web" and mix[20]["source"] == "given"
    train, val = SplitRecords(a, 0.3, "train", seed=1), SplitRecords(a, 0.3, "val", seed=1)
    assert len(train) + len(val) == 10 and not ({r["text"] for r in train} & {r["text"] for r in val})
    records, _ = build_dataset({"name": "mixture", "sources": [{"records": {"name": "list", "records": [{"text": "x"}]},
                                                                "repeat": 2}]}, "plain")
    assert len(records) == 2


def test_kv_store_and_mixture_properties():
    """Property tests: any set of keys / values written in any order reads back exactly; a mixture's length and
    per-source counts follow the repeat weights, and its fractional part never repeats a record."""
    import tempfile

    from hypothesis import given, settings
    from hypothesis import strategies as st

    from kohakuwullm_b200.data.sources.kvstore import KVFile, KVWriter, encode_key
    from kohakuwullm_b200.data.sources.records import ListRecords, MixtureRecords

    values = st.one_of(st.binary(max_size=40), st.text(max_size=20), st.dictionaries(st.text(max_size=5), st.integers(), max_size=3))
    keys = st.one_of(st.integers(min_value=0, max_value=2 ** 40), st.text(min_size=1, max_size=12))

    @settings(max_examples=40, deadline=None)
    @given(st.lists(st.tuples(keys, values), min_size=1, max_size=30))
    def store(pairs):
        with tempfile.TemporaryDirectory() as tmp:
            path = f"{tmp}/x.kv"
            with KVWriter(path) as w:
                for k, v in pairs:
                    w.put(k, v)
            kv = KVFile(path)
            want = {}
            for k, v in pairs:
                want[encode_key(k)] = (k, v)                       # the last write of a key wins
            assert len(kv) == len(want)
            for k, v in want.values():
                assert kv.get(k) == v
            assert kv.keys() == sorted(kv.keys())

    @settings(max_examples=40, deadline=None)
    @given(st.lists(st.tuples(st.integers(1, 30), st.floats(0.1, 3.0)), min_size=1, max_size=4), st.integers(0, 100))
    def mix(parts, seed):
        sources = [{"records": ListRecords([{"text": f"{i}:{j}"} for j in range(n)]), "repeat": r, "source": f"s{i}"}
                   for i, (n, r) in enumerate(parts)]
        m = MixtureRecords(sources, seed=seed)
        assert len(m) == sum(int(n * r + 1e-9) for n, r in parts)
        start = 0
        for i, (n, r) in enumerate(parts):
            total = int(n * r + 1e-9)
            got = [m[start + j]["text"] for j in range(total)]
            assert all(t.startswith(f"{i}:") for t in got)
            whole = (total // n) * n
            assert len(set(got[whole:])) == total - whole          # the fractional tail is a subset without repeats
            start += total

    store()
    mix()


def test_doc_filter_builder_names_arguments_and_pickling():
    import pickle

    from kohakuwullm_b200.data.filters import build_doc_filter

    assert build_doc_filter("") is None and build_doc_filter(None) is None
    looping = [1, 2, 3, 4] * 40
    varied = list(range(160))
    ngram = build_doc_filter("ngram")
    assert ngram(varied) and not ngram(looping)
    strict = build_doc_filter({"name": "consecutive", "threshold": 8})
    assert strict(varied) and not strict(looping) and build_doc_filter("consecutive")(looping[:100])   # 25 runs < 32
    again = pickle.loads(pickle.dumps(strict))                  # travels into loader worker processes
    assert not again(looping)
    keep_all = lambda ids: True                                  # noqa: E731
    assert build_doc_filter(keep_all) is keep_all
    with pytest.raises(KeyError):
        build_doc_filter("perplexity")


def test_pack_closes_when_no_document_fits_the_remaining_room():
    """Every document is 30 tokens, the budget 100 and the slack 4: after three documents the room (10) is larger
    than the slack and smaller than any document, so nothing upcoming ever fits. The pack must close anyway (the
    packer looks a bounded number of documents ahead), nothing may be lost or doubled, and the documents it looked at
    open the following packs."""
    from kohakuwullm_b200.data import build_loader
    from kohakuwullm_b200.registry import DATASET, build

    texts = [f"{i:04d}" + chr(65 + i % 26) * 24 for i in range(400)]   # 28 bytes + BOS + EOS = 30 tokens, all distinct
    records = build({"name": "list", "records": [{"text": t} for t in texts]}, DATASET)
    loader = build_loader("iterative", records, lambda r, rng=None: [(r["text"], True)], lambda s: list(s.encode()),
                          k=100, m=4, ctx_max=64, seed=3, bos=256, eos=257, shuffle=False)
    emitted = []
    it = iter(loader)
    for _ in range(40):
        batch = next(it)
        assert batch.num_tokens == 90 and batch.seq_info.num_seqs == 3
        cu = batch.seq_info.cu_seqlens.tolist()
        emitted += [bytes(t for t in batch.tokens[a:b].tolist() if t < 256).decode() for a, b in zip(cu, cu[1:])]
    state = loader.state_dict()["positions"][0]
    assert len(emitted) == len(set(emitted)) == 120
    assert len(state["carry"]) <= 16                                  # the look-ahead queue stays bounded
    # what was read is what was emitted plus what waits in the queue: nothing lost
    assert state["pass"] == 0 and state["cursor"] == 120 + len(state["carry"])
    assert set(emitted) <= set(texts[: state["cursor"]])


@pytest.mark.timeout(120)
def test_packing_properties_over_random_lengths_budgets_and_slack():
    """For arbitrary document lengths, budgets and slack, in both packing modes: the loader always yields, a pack never
    exceeds its budget, exact packs are exactly full, and over the packs of one epoch the documents come out once each
    (whole in the non-exact mode, as the concatenation of their pieces in the exact mode)."""
    from hypothesis import given, settings
    from hypothesis import strategies as st

    from kohakuwullm_b200.data import build_loader
    from kohakuwullm_b200.registry import DATASET, build

    @settings(max_examples=40, deadline=None)
    @given(lengths=st.lists(st.integers(1, 60), min_size=3, max_size=40), k=st.integers(16, 96),
           slack=st.integers(0, 15), exact=st.booleans(), seed=st.integers(0, 5))
    def check(lengths, k, slack, exact, seed):
        texts = [f"{i:03d}" + "x" * (n - 1) if n > 3 else "y" * n for i, n in enumerate(lengths)]
        records = build({"name": "list", "records": [{"text": t} for t in texts]}, DATASET)
        ctx = min(k, 48)
        loader = build_loader("iterative", records, lambda r, rng=None: [(r["text"], True)], lambda s: list(s.encode()),
                              k=k, m=min(slack, k // 2), ctx_max=ctx, seed=seed, bos=256, eos=257, exact=exact)
        total = sum(min(len(t) + 2, ctx) for t in texts)                  # tokens of one epoch after the cut to ctx
        seen_tokens, packs = 0, 0
        it = iter(loader)
        while seen_tokens < total and packs < 4 * len(texts) + 8:
            batch = next(it)
            packs += 1
            real = int((batch.tokens != 0).sum()) if exact else batch.num_tokens    # exact packs pad the very last one
            assert batch.num_tokens <= k
            if exact:
                assert batch.num_tokens == k
            seen_tokens += real
        assert seen_tokens >= total, (seen_tokens, total, packs)          # the epoch was delivered, the loader never stalled

    check()


def test_a_loader_without_records_is_an_empty_iteration():
    """A hold-out split of a tiny corpus can be empty: iterating it yields nothing (it used to escape as a
    ``StopIteration`` inside a generator, which Python turns into a RuntimeError)."""
    from kohakuwullm_b200.data import build_loader
    from kohakuwullm_b200.data.sources.records import SplitRecords
    from kohakuwullm_b200.registry import DATASET, build

    records = build({"name": "list", "records": [{"text": "abc def"} for _ in range(3)]}, DATASET)
    held_out = SplitRecords(records, 0.0001, "val", 0)
    assert len(held_out) == 0
    loader = build_loader("ddp", held_out, lambda r, rng=None: [(r["text"], True)], lambda s: list(s.encode()), k=64, m=4)
    assert list(loader) == []
    # more shards than records: the shards beyond the records are empty iterations too
    extra = build_loader("ddp", records, lambda r, rng=None: [(r["text"], True)], lambda s: list(s.encode()), k=64, m=4,
                         rank=5, world=8)
    assert list(extra) == []


def test_vault_corpus_json_schema_reads_dict_values_and_json_text(tmp_path):
    import json

    from kohakuwullm_b200.data.sources.kvstore import KVWriter, VaultCorpusRecords

    d = tmp_path / "sft" / "chat"
    d.mkdir(parents=True)
    with KVWriter(str(d / "shard-0.kv")) as w:
        w.put("00000000", {"messages": [{"role": "user", "content": "hi"}]})          # stored as JSON by the writer
        w.put("00000001", json.dumps({"messages": [{"role": "user", "content": "yo"}]}))   # JSON kept as text by another tool
    recs = VaultCorpusRecords("sft/chat", str(tmp_path), schema="json")
    assert [r["messages"][0]["content"] for r in (recs[0], recs[1])] == ["hi", "yo"]


def test_worker_loader_refuses_more_shards_than_records():
    from kohakuwullm_b200.data import build_loader
    from kohakuwullm_b200.registry import DATASET, build

    records = build({"name": "list", "records": [{"text": "abc"} for _ in range(3)]}, DATASET)
    with pytest.raises(ValueError, match="use fewer workers"):
        build_loader("workers", records, lambda r, rng=None: [(r["text"], True)], lambda s: list(s.encode()), workers=4, k=64)
