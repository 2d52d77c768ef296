"""Export: the Hugging Face model reproduces the framework's logits; tokenizer pruning; GGUF header."""

import struct

import torch

from kohakuwullm_b200.export.hf.convert import export_hf
from kohakuwullm_b200.models import LMBackbone, SeqInfo, get_preset
from kohakuwullm_b200.tokenizer.prune import prune_tokenizer_json


def _check(cfg, tmp_path):
    torch.manual_seed(0)
    model = LMBackbone(cfg).eval()
    for blk in model.blocks:
        if hasattr(blk.mlp, "router"):
            blk.mlp.router.expert_bias.normal_(0, 0.3)
    hf = export_hf(model, cfg, str(tmp_path), dtype=torch.float32).eval()
    tokens = torch.randint(0, cfg.vocab_size, (2, 12))
    with torch.no_grad():
        ours = model.head.logits(model(tokens, SeqInfo.padded(2, 12)))
        theirs = hf(tokens).logits
    torch.testing.assert_close(ours, theirs, rtol=1e-4, atol=1e-4)


def test_hf_export_dense_with_windows_sinks_yarn(tmp_path):
    _check(get_preset("B200-sliding-1B", vocab_size=101, dim=64, depth=4, heads=2, kv_heads=1, head_dim=32,
                      mlp_hidden=128, sliding_window=5, max_position=16, init_std=0.2), tmp_path)


def test_hf_export_moe(tmp_path):
    _check(get_preset("B200-moe-991M", vocab_size=101, dim=64, depth=3, heads=2, kv_heads=1, head_dim=32, mlp_hidden=128,
                      moe_num_experts=4, moe_top_k=2, moe_hidden=64, mxfp8=False, init_std=0.2), tmp_path)


def test_prune_tokenizer():
    vocab = {chr(97 + i): i for i in range(6)}
    vocab.update({"ab": 6, "cd": 7, "abcd": 8, "ef": 9})
    data = {"model": {"vocab": vocab, "merges": ["a b", "c d", "ab cd", "e f"]}, "added_tokens": []}
    out = prune_tokenizer_json(data, target=12, specials=["<|bos|>", "<|eos|>"])
    assert len(out["model"]["vocab"]) == 12
    assert out["model"]["merges"] == ["a b", "c d", "ab cd", "e f"][: len(out["model"]["merges"])]
    assert "<|reserved_0|>" not in out["model"]["vocab"] and out["model"]["vocab"]["<|eos|>"] == 11
    small = prune_tokenizer_json(data, target=10, specials=["<|bos|>"])
    assert "ef" not in small["model"]["vocab"] and "e f" not in small["model"]["merges"]


def test_gguf_writer(tmp_path):
    from kohakuwullm_b200.cli.to_gguf import GGUF_MAGIC, write_gguf

    path = str(tmp_path / "m.gguf")
    write_gguf(path, {"w": torch.ones(4, 8), "b": torch.zeros(8)}, {"general.architecture": "kohaku", "n": 3})
    raw = open(path, "rb").read()
    magic, version, n_tensors, n_kv = struct.unpack("<IIQQ", raw[:24])
    assert (magic, version, n_tensors, n_kv) == (GGUF_MAGIC, 3, 2, 2)


def test_build_tokenizer_cli(tmp_path, capsys):
    """Train a small byte-level BPE, prune it through the CLI: exact vocabulary size, named specials then reserved
    slots, BOS prepended by the post-processor, and the measured growth in tokens per sample."""
    import json

    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers

    from kohakuwullm_b200.cli import build_tokenizer as bt

    corpus = ["the quick brown fox jumps over the lazy dog %d times" % i for i in range(200)]
    tok = Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    tok.train_from_iterator(corpus, trainers.BpeTrainer(vocab_size=400, initial_alphabet=pre_tokenizers.ByteLevel.alphabet(),
                                                        show_progress=False))
    src = tmp_path / "src"
    src.mkdir()
    tok.save(str(src / "tokenizer.json"))
    shard = tmp_path / "part.jsonl"
    shard.write_text("\n".join(json.dumps({"text": t}) for t in corpus) + "\n")
    n_named = len(bt.CORE_SPECIALS + bt.CHAT_SPECIALS + bt.tipo_specials())
    target = 320 + n_named + 10
    assert bt.main(["--source", str(src), "--out", str(tmp_path / "out"), "--base", "320", "--target", str(target),
                    "--check-corpus", str(shard), "--check-samples", "50"]) == 0
    report = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert report["vocab"] == target and report["named_specials"] == n_named and report["reserved"] == 10
    assert report["length_ratio"] >= 1.0 and report["samples"] == 50
    built = Tokenizer.from_file(str(tmp_path / "out" / "tokenizer.json"))
    vocab = built.get_vocab()
    assert vocab["<|bos|>"] == 320 and vocab["<|reserved_9|>"] == target - 1
    ids = built.encode("the quick fox").ids
    assert ids[0] == vocab["<|bos|>"] and built.decode(ids[1:]) == "the quick fox"
