"""Export: the Hugging Face model reproduces the framework's logits; tokenizer pruning; GGUF header."""

import struct

import pytest

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


def test_hf_export_widths_derived_from_ratios(tmp_path):
    """No explicit hidden sizes: the dense and the expert widths come from ``ratio * dim * 2/3`` rounded up to the
    multiple, exactly as the model resolves them (an export that wrote 0 for a derived expert width failed to load)."""
    _check(get_preset("B200-smoke", vocab_size=101, dim=96, depth=3, heads=2, kv_heads=1, head_dim=32, mlp_hidden=None,
                      mlp_ratio=3.0, mlp_multiple_of=32, moe_every=1, moe_first_dense=1, moe_num_experts=4, moe_top_k=2,
                      moe_hidden=None, moe_ratio=1.5, moe_num_shared=2, mxfp8=False, init_std=0.2), tmp_path)


BASE = dict(vocab_size=101, dim=64, depth=3, heads=2, kv_heads=1, head_dim=32, mlp_hidden=128, init_std=0.2, mxfp8=False)
MOE4 = dict(moe_every=1, moe_num_experts=4, moe_top_k=2, moe_hidden=64)


@pytest.mark.parametrize("overrides", [
    dict(tie_embeddings=True, embedding_scale=True, logit_soft_cap=20.0),
    dict(rope_scaling="ntk", rope_factor=2.0, rope_partial=0.5),
    dict(rope_scaling="yarn", rope_factor=4.0, rope_partial=0.75),
    dict(rope_scaling="linear", rope_factor=4.0),
    dict(norm="gemma_rmsnorm"),
    dict(mlp="geglu"),
    dict(scale_residual_by_depth=True, qk_norm=False),
    dict(**MOE4, moe_router_kwargs={"score": "sqrtsoftplus", "norm_topk_prob": False, "routed_scaling_factor": 2.5}),
])
def test_hf_export_reproduces_every_supported_option(tmp_path, overrides):
    cfg = get_preset("B200-smoke", **{**BASE, **overrides})
    torch.manual_seed(0)
    model = LMBackbone(cfg).eval()
    with torch.no_grad():
        for n, p in model.named_parameters():
            if "norm" in n:
                p.add_(torch.randn_like(p) * 0.2)          # a gain of exactly 1 (or 0) would hide a wrong scaling rule
    hf = export_hf(model.state_dict(), cfg, str(tmp_path), dtype=torch.float32).eval()
    tokens = torch.randint(0, cfg.vocab_size, (2, 11))
    with torch.no_grad():
        ours = model.head.logits(model(tokens, SeqInfo.padded(2, 11)))
        theirs = hf(tokens).logits
    torch.testing.assert_close(ours, theirs, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("overrides,word", [
    (dict(attn_bias=True), "attn_bias"), (dict(post_norm=True), "post_norm"), (dict(qk_norm_affine=False), "qk_norm_affine"),
    (dict(norm="layernorm"), "layernorm"), (dict(mlp="gelu"), "gelu"), (dict(posenc="none"), "posenc"),
    (dict(**MOE4, moe_router="sinkhorn"), "sinkhorn"), (dict(**MOE4, moe_mlp="latent_moe"), "latent_moe"),
])
def test_exports_refuse_what_their_target_cannot_express(tmp_path, overrides, word):
    """An option that keeps every parameter name (a routing variant, a residual rule) would load into the exported
    model and silently compute something else: both exporters name the option and refuse."""
    from kohakuwullm_b200.cli.to_gguf import convert, unrepresentable

    cfg = get_preset("B200-smoke", **{**BASE, **overrides})
    state = LMBackbone(cfg).state_dict()
    with pytest.raises(ValueError, match=word):
        export_hf(state, cfg, str(tmp_path / "hf"))
    with pytest.raises(ValueError, match=word):
        convert(state, cfg, str(tmp_path / "m.gguf"))
    assert any(word in item for item in unrepresentable(cfg))


def test_gguf_refuses_windows_sinks_and_scaling_unless_told_to_write_anyway(tmp_path):
    from kohakuwullm_b200.cli.to_gguf import convert, unrepresentable

    plain = get_preset("B200-smoke", **BASE)
    assert unrepresentable(plain) == []
    fancy = get_preset("B200-smoke", **BASE, sliding_window=4, global_layer_every=2, attn_sink=True, rope_scaling="yarn",
                       rope_factor=4.0, logit_soft_cap=30.0)
    lossy = unrepresentable(fancy)
    assert {"sliding windows", "attention sinks", "logit_soft_cap"} <= set(lossy) and any("yarn" in x for x in lossy)
    state = LMBackbone(fancy).state_dict()
    with pytest.raises(ValueError, match="sliding windows"):
        convert(state, fancy, str(tmp_path / "m.gguf"))
    info = convert(state, fancy, str(tmp_path / "m.gguf"), allow_lossy=True)
    assert info["lossy"] == lossy and (tmp_path / "m.gguf").stat().st_size > 1000


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


def _read_gguf(path):
    """A minimal GGUF v3 reader: metadata (scalars, strings, arrays) and tensors as float32 arrays."""
    import numpy as np

    raw = open(path, "rb").read()
    pos = 0

    def take(fmt):
        nonlocal pos
        out = struct.unpack_from("<" + fmt, raw, pos)
        pos += struct.calcsize("<" + fmt)
        return out if len(out) > 1 else out[0]

    def string():
        nonlocal pos
        n = take("Q")
        s = raw[pos:pos + n].decode("utf-8")
        pos += n
        return s

    def value(t):
        if t == 8:
            return string()
        if t == 9:
            et, n = take("I"), take("Q")
            return [value(et) for _ in range(n)]
        return take({4: "I", 5: "i", 6: "f", 7: "B", 10: "Q"}[t])

    magic, version, n_tensors, n_kv = take("I"), take("I"), take("Q"), take("Q")
    meta = {}
    for _ in range(n_kv):
        k = string()
        meta[k] = value(take("I"))
    infos = []
    for _ in range(n_tensors):
        name = string()
        nd = take("I")
        dims = [take("Q") for _ in range(nd)]
        infos.append((name, list(reversed(dims)), take("I"), take("Q")))
    base = (pos + 31) // 32 * 32
    tensors = {}
    for name, shape, code, off in infos:
        n = int(np.prod(shape))
        if code == 0:
            arr = np.frombuffer(raw, np.float32, n, base + off)
        elif code == 1:
            arr = np.frombuffer(raw, np.float16, n, base + off).astype(np.float32)
        else:
            arr = (np.frombuffer(raw, np.uint16, n, base + off).astype(np.uint32) << 16).view(np.float32)
        tensors[name] = torch.from_numpy(arr.reshape(shape).copy())
    return (magic, version), meta, tensors


def test_gguf_export_in_llama_cpp_layouts(tmp_path):
    """dots1 for a sparse model, qwen3 for a dense one: hyper-parameters, tensor names, the q/k/v and gate/up splits,
    GQA expansion, dtype choice, and the tokenizer block."""
    import json

    from kohakuwullm_b200.cli import to_gguf

    common = dict(vocab_size=101, dim=64, depth=2, heads=4, kv_heads=2, head_dim=16, mlp_hidden=96, mxfp8=False)
    sparse = get_preset("B200-moe-991M", **common, moe_first_dense=1, moe_num_experts=4, moe_top_k=2, moe_hidden=48, moe_num_shared=1)
    torch.manual_seed(0)
    model = LMBackbone(sparse)
    state = model.state_dict()
    tokdir = tmp_path / "tok"
    tokdir.mkdir()
    vocab = {f"t{i}": i for i in range(99)}
    (tokdir / "tokenizer.json").write_text(json.dumps({
        "model": {"vocab": vocab, "merges": [["t0", "t1"], "t2 t3"]},
        "added_tokens": [{"id": 99, "content": "<|bos|>", "special": True}, {"id": 100, "content": "<|im_end|>", "special": True}]}))
    (tokdir / "tokenizer_config.json").write_text(json.dumps({"bos_token": "<|bos|>", "eos_token": {"content": "<|im_end|>"},
                                                              "chat_template": "{{ messages }}"}))
    out = str(tmp_path / "moe.gguf")
    info = to_gguf.convert(state, sparse, out, name="tiny-moe", out_dtype="bf16", tokenizer=str(tokdir))
    assert info["arch"] == "dots1"
    (magic, version), meta, tensors = _read_gguf(out)
    assert (magic, version) == (to_gguf.GGUF_MAGIC, 3)
    assert meta["general.architecture"] == "dots1" and meta["general.file_type"] == 32
    assert meta["dots1.block_count"] == 2 and meta["dots1.attention.head_count_kv"] == 4        # expanded to one per query head
    assert meta["dots1.expert_count"] == 4 and meta["dots1.expert_used_count"] == 2 and meta["dots1.leading_dense_block_count"] == 1
    assert meta["dots1.feed_forward_length"] == 96 and meta["dots1.expert_feed_forward_length"] == 48
    assert meta["tokenizer.ggml.model"] == "gpt2" and len(meta["tokenizer.ggml.tokens"]) == 101
    assert meta["tokenizer.ggml.merges"] == ["t0 t1", "t2 t3"] and meta["tokenizer.ggml.token_type"][99] == 3
    assert meta["tokenizer.ggml.bos_token_id"] == 99 and meta["tokenizer.ggml.eos_token_id"] == 100
    assert meta["tokenizer.ggml.eot_token_id"] == 100 and meta["tokenizer.chat_template"] == "{{ messages }}"
    qkv = state["blocks.0.attn.qkv_proj.weight"].float()
    bf = lambda t: t.to(torch.bfloat16).float()  # noqa: E731
    assert torch.equal(tensors["blk.0.attn_q.weight"], bf(qkv[:64]))
    k = qkv[64:96].reshape(2, 16, 64).repeat_interleave(2, 0).reshape(64, 64)
    assert torch.equal(tensors["blk.0.attn_k.weight"], bf(k)) and tensors["blk.0.attn_v.weight"].shape == (64, 64)
    gate, up = state["blocks.0.mlp.w_in.weight"].float().chunk(2, 0)
    assert torch.equal(tensors["blk.0.ffn_gate.weight"], bf(gate)) and torch.equal(tensors["blk.0.ffn_up.weight"], bf(up))
    assert tensors["blk.1.ffn_gate_exps.weight"].shape == (4, 48, 64) and tensors["blk.1.ffn_down_exps.weight"].shape == (4, 64, 48)
    assert tensors["blk.1.ffn_gate_shexp.weight"].shape[1] == 64 and "blk.1.exp_probs_b.bias" in tensors
    assert torch.equal(tensors["blk.0.attn_q_norm.weight"], state["blocks.0.attn.q_norm"].float())   # vectors stay fp32
    assert not any("load_accum" in n for n in tensors)

    dense = get_preset("B200-smoke", **common)
    dmodel = LMBackbone(dense)
    ckpt_path = str(tmp_path / "d.ckpt")
    torch.save({"state_dict": dmodel.state_dict()}, ckpt_path)
    sets = [x for k, v in common.items() for x in ("--set", f"{k}={v}")]
    assert to_gguf.main(["--ckpt", ckpt_path, "--preset", "B200-smoke", *sets, "--out", str(tmp_path / "d.gguf"),
                         "--no-expand-kv", "--out-dtype", "f32"]) == 0
    _, dmeta, dtensors = _read_gguf(str(tmp_path / "d.gguf"))
    assert dmeta["general.architecture"] == "qwen3" and dmeta["qwen3.attention.head_count_kv"] == 2 and "qwen3.expert_count" not in dmeta
    assert dtensors["blk.1.attn_k.weight"].shape == (32, 64)
    assert torch.equal(dtensors["output.weight"], dmodel.state_dict()["head.proj.weight"].float())


def test_to_hf_cli_copies_the_tokenizer_and_checks_logits(tmp_path, capsys):
    import json
    import os

    from kohakuwullm_b200.cli import to_hf

    common = dict(vocab_size=101, dim=64, depth=2, heads=2, kv_heads=1, head_dim=32, mlp_hidden=128, init_std=0.2, mxfp8=False)
    torch.manual_seed(1)
    model = LMBackbone(get_preset("B200-smoke", **common))
    ckpt_path = str(tmp_path / "m.ckpt")
    torch.save({"state_dict": model.state_dict()}, ckpt_path)
    tokdir = tmp_path / "tok"
    tokdir.mkdir()
    (tokdir / "tokenizer.json").write_text(json.dumps({"model": {"vocab": {}, "merges": []}}))
    (tokdir / "tokenizer_config.json").write_text("{}")
    sets = [x for k, v in common.items() for x in ("--set", f"{k}={v}")]
    out = tmp_path / "hf"
    assert to_hf.main(["--ckpt", ckpt_path, "--preset", "B200-smoke", *sets, "--out", str(out), "--out-dtype", "fp32",
                       "--tokenizer", str(tokdir), "--check"]) == 0
    text = capsys.readouterr().out
    assert "check: largest relative logit difference" in text and "tokenizer.json" in text
    for name in ("config.json", "modeling_kohaku.py", "configuration_kohaku.py", "tokenizer.json", "tokenizer_config.json"):
        assert os.path.exists(out / name), name
