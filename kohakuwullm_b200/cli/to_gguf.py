"""Checkpoint -> GGUF v3 for llama.cpp, written with a small self-contained writer (no ``gguf`` package needed).

    python -m kohakuwullm_b200.cli.to_gguf --ckpt run/last.ckpt --preset Kohaku-MoE-1B --out model.gguf \\
        --tokenizer models/tokenizer --out-dtype f16

The model is emitted under an architecture llama.cpp already knows, so the file loads without a custom build:
``dots1`` for the sparse models (RMSNorm, per-head Q/K norm, GQA + NeoX-style RoPE, SwiGLU, leading dense blocks,
routed experts with shared experts, router bias for aux-loss-free balancing, sigmoid / softmax gating) and ``qwen3``
for the dense ones (the same block without experts). What the conversion does:

* the fused ``qkv_proj`` is cut into ``attn_q / attn_k / attn_v``; with ``--expand-kv`` (default) the K and V projections are
  repeated to one head per query head (query head h reads KV head h // group, so this reproduces GQA exactly and
  sidesteps back-ends without grouped KV for this architecture);
* the fused ``w_in`` is split gate-first (the model computes ``silu(h[:half]) * h[half:]``); stacked expert tensors
  already have GGUF's (expert, out, in) order;
* with ``--tokenizer`` the byte-level BPE vocabulary, merges, special-token ids, ``add_bos_token`` (every training
  document starts with BOS), the chat template and the end-of-turn token are written too.
Reference: scripts/tools/to_gguf.py.
"""

from __future__ import annotations

import argparse
import json
import os
import struct
import sys

import numpy as np
import torch

GGUF_MAGIC, GGUF_VERSION, ALIGN = 0x46554747, 3, 32
T_U32, T_I32, T_F32, T_BOOL, T_STR, T_ARR, T_U64 = 4, 5, 6, 7, 8, 9, 10
GGML_F32, GGML_F16, GGML_BF16 = 0, 1, 30
FILE_TYPE = {"f32": 0, "f16": 1, "bf16": 32}
TOKEN_NORMAL, TOKEN_CONTROL, TOKEN_USER, TOKEN_UNUSED = 1, 3, 4, 5
GATING = {"softmax": 1, "sigmoid": 2}


def _s(x: str) -> bytes:
    b = x.encode("utf-8")
    return struct.pack("<Q", len(b)) + b


def _kv(key: str, value) -> bytes:
    out = _s(key)
    if isinstance(value, bool):
        return out + struct.pack("<IB", T_BOOL, int(value))
    if isinstance(value, U32):
        return out + struct.pack("<II", T_U32, int(value))
    if isinstance(value, int):
        return out + struct.pack("<IQ", T_U64, value)
    if isinstance(value, float):
        return out + struct.pack("<If", T_F32, value)
    if isinstance(value, (list, tuple)):
        if value and isinstance(value[0], str):
            return out + struct.pack("<IIQ", T_ARR, T_STR, len(value)) + b"".join(_s(v) for v in value)
        return out + struct.pack("<IIQ", T_ARR, T_I32, len(value)) + struct.pack(f"<{len(value)}i", *value)
    return out + struct.pack("<I", T_STR) + _s(str(value))


class U32(int):
    """Marks an integer that llama.cpp reads as uint32 (most hyper-parameters)."""


def write_gguf(path: str, tensors: dict[str, torch.Tensor], meta: dict, f16: bool = True, out_dtype: str | None = None) -> None:
    """Tensors of two or more dimensions are stored in ``out_dtype`` (``f16`` when ``f16`` is true and no dtype is
    given), vectors always in f32."""
    out_dtype = out_dtype or ("f16" if f16 else "f32")
    infos, blobs, offset = b"", [], 0
    for name, t in tensors.items():
        wide = t.dim() >= 2 and out_dtype != "f32"
        if wide and out_dtype == "bf16":
            raw, code = t.detach().to(torch.bfloat16).contiguous().view(torch.int16).cpu().numpy().tobytes(), GGML_BF16
        else:
            arr = t.detach().float().cpu().numpy().astype(np.float16 if wide else np.float32)
            raw, code = arr.tobytes(), (GGML_F16 if wide else GGML_F32)
        dims = list(reversed(t.shape))
        infos += _s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        infos += struct.pack("<IQ", code, offset)
        pad = (-len(raw)) % ALIGN
        blobs.append(raw + b"\0" * pad)
        offset += len(raw) + pad
    kvs = b"".join(_kv(k, v) for k, v in meta.items())
    header = struct.pack("<IIQQ", GGUF_MAGIC, GGUF_VERSION, len(tensors), len(meta)) + kvs + infos
    with open(path, "wb") as f:
        f.write(header)
        f.write(b"\0" * ((-len(header)) % ALIGN))
        for b in blobs:
            f.write(b)


def hparams(cfg, arch: str, name: str, out_dtype: str, expand_kv: bool, dense_ff: int, expert_ff: int | None) -> dict:
    a = arch
    meta = {"general.architecture": a, "general.name": name, "general.alignment": U32(ALIGN),
            "general.file_type": U32(FILE_TYPE[out_dtype]),
            f"{a}.context_length": U32(cfg.max_position), f"{a}.embedding_length": U32(cfg.dim),
            f"{a}.block_count": U32(cfg.depth), f"{a}.feed_forward_length": U32(dense_ff),
            f"{a}.attention.head_count": U32(cfg.heads),
            f"{a}.attention.head_count_kv": U32(cfg.heads if expand_kv else cfg.kv_heads),
            f"{a}.attention.key_length": U32(cfg.head_dim), f"{a}.attention.value_length": U32(cfg.head_dim),
            f"{a}.rope.freq_base": float(cfg.rope_theta), f"{a}.rope.dimension_count": U32(int(cfg.head_dim * cfg.rope_partial)),
            f"{a}.attention.layer_norm_rms_epsilon": float(cfg.norm_eps), f"{a}.vocab_size": U32(cfg.vocab_size)}
    if expert_ff is not None:
        kw = cfg.moe_router_kwargs or {}
        meta.update({f"{a}.expert_count": U32(cfg.moe_num_experts), f"{a}.expert_used_count": U32(cfg.moe_top_k),
                     f"{a}.expert_shared_count": U32(cfg.moe_num_shared),
                     f"{a}.leading_dense_block_count": U32(cfg.moe_first_dense),
                     f"{a}.expert_feed_forward_length": U32(expert_ff),
                     f"{a}.expert_weights_norm": bool(kw.get("norm_topk_prob", True)),
                     f"{a}.expert_weights_scale": float(kw.get("routed_scaling_factor", 1.0)),
                     f"{a}.expert_gating_func": U32(GATING.get(kw.get("score", kw.get("score_func", "sigmoid")), 2))})
    return meta


def tokenizer_meta(path: str, turn_end: str = "<|im_end|>", chat_template: bool = True) -> dict:
    """Vocabulary, merges and special ids in the layout llama.cpp's ``gpt2`` (byte-level BPE) tokenizer reads."""
    with open(os.path.join(path, "tokenizer.json"), encoding="utf-8") as f:
        spec = json.load(f)
    conf = {}
    if os.path.exists(os.path.join(path, "tokenizer_config.json")):
        with open(os.path.join(path, "tokenizer_config.json"), encoding="utf-8") as f:
            conf = json.load(f)
    vocab = spec["model"]["vocab"]
    added = {a["id"]: a for a in spec.get("added_tokens", [])}
    size = max(max(vocab.values()), max(added, default=0)) + 1
    tokens, types = [f"[UNUSED{i}]" for i in range(size)], [TOKEN_UNUSED] * size
    for text, i in vocab.items():
        tokens[i], types[i] = text, TOKEN_NORMAL
    for i, entry in added.items():
        tokens[i], types[i] = entry["content"], (TOKEN_CONTROL if entry.get("special") else TOKEN_USER)
    merges = [" ".join(m) if isinstance(m, list) else m for m in spec["model"].get("merges", [])]
    meta = {"tokenizer.ggml.model": "gpt2", "tokenizer.ggml.pre": "default", "tokenizer.ggml.tokens": tokens,
            "tokenizer.ggml.token_type": types, "tokenizer.ggml.merges": merges,
            "tokenizer.ggml.add_bos_token": True, "tokenizer.ggml.add_eos_token": False}
    ids = {t["content"]: i for i, t in added.items()}
    for key, field in (("bos_token", "bos_token_id"), ("eos_token", "eos_token_id"), ("pad_token", "padding_token_id"),
                       ("unk_token", "unknown_token_id")):
        text = conf.get(key)
        text = text.get("content") if isinstance(text, dict) else text
        if text in ids:
            meta[f"tokenizer.ggml.{field}"] = U32(ids[text])
    if chat_template:
        if conf.get("chat_template"):
            meta["tokenizer.chat_template"] = conf["chat_template"]
        if turn_end in ids:
            meta["tokenizer.ggml.eot_token_id"] = U32(ids[turn_end])     # end of turn ends generation like EOS
    return meta


def tensor_map(state: dict, cfg, expand_kv: bool) -> dict[str, torch.Tensor]:
    Hq, Hkv, D = cfg.heads, cfg.kv_heads, cfg.head_dim

    def kv(w: torch.Tensor) -> torch.Tensor:
        if not expand_kv or Hkv == Hq:
            return w
        return w.reshape(Hkv, D, w.shape[-1]).repeat_interleave(Hq // Hkv, dim=0).reshape(-1, w.shape[-1])

    out = {"token_embd.weight": state["embed.weight"], "output_norm.weight": state["final_norm.weight"],
           "output.weight": state.get("head.proj.weight", state["embed.weight"])}
    for i in range(cfg.depth):
        p, b = f"blocks.{i}.", f"blk.{i}."
        qkv = state[p + "attn.qkv_proj.weight"]
        q, k, v = qkv[:Hq * D], qkv[Hq * D:(Hq + Hkv) * D], qkv[(Hq + Hkv) * D:]
        out.update({b + "attn_norm.weight": state[p + "norm_attn.weight"], b + "attn_q.weight": q, b + "attn_k.weight": kv(k),
                    b + "attn_v.weight": kv(v), b + "attn_output.weight": state[p + "attn.o_proj.weight"],
                    b + "ffn_norm.weight": state[p + "norm_mlp.weight"]})
        if p + "attn.q_norm" in state:
            out[b + "attn_q_norm.weight"], out[b + "attn_k_norm.weight"] = state[p + "attn.q_norm"], state[p + "attn.k_norm"]
        if p + "mlp.w_in.weight" in state:
            gate, up = state[p + "mlp.w_in.weight"].chunk(2, dim=0)
            out.update({b + "ffn_gate.weight": gate, b + "ffn_up.weight": up, b + "ffn_down.weight": state[p + "mlp.w_out.weight"]})
            continue
        gate, up = state[p + "mlp.w_in"].chunk(2, dim=1)
        out.update({b + "ffn_gate_exps.weight": gate, b + "ffn_up_exps.weight": up, b + "ffn_down_exps.weight": state[p + "mlp.w_out"],
                    b + "ffn_gate_inp.weight": state[p + "mlp.router.weight"]})
        if p + "mlp.shared.w_in.weight" in state:
            sg, su = state[p + "mlp.shared.w_in.weight"].chunk(2, dim=0)
            out.update({b + "ffn_gate_shexp.weight": sg, b + "ffn_up_shexp.weight": su,
                        b + "ffn_down_shexp.weight": state[p + "mlp.shared.w_out.weight"]})
        if p + "mlp.router.expert_bias" in state:
            out[b + "exp_probs_b.bias"] = state[p + "mlp.router.expert_bias"]
    return out


def unrepresentable(cfg) -> list[str]:
    """Options of the model that the ``qwen3`` / ``dots1`` graphs of llama.cpp have no place for. A file written
    anyway loads and runs, and computes a different function."""
    def name(spec):
        return spec if isinstance(spec, str) else (spec.get("name") if isinstance(spec, dict) else str(spec))

    bad = []
    if name(cfg.norm) not in ("rmsnorm", "rmsnorm_native", "rmsnorm_triton"):
        bad.append(f"norm={name(cfg.norm)!r}")
    if name(cfg.mlp) not in ("swiglu", "swiglu_native", "swiglu_triton"):
        bad.append(f"mlp={name(cfg.mlp)!r}")
    if name(cfg.posenc) != "rope":
        bad.append(f"posenc={name(cfg.posenc)!r}")
    if any(w is not None for w in cfg.windows):
        bad.append("sliding windows")
    if cfg.attn_sink:
        bad.append("attention sinks")
    if cfg.rope_scaling not in (None, "none"):
        bad.append(f"rope_scaling={cfg.rope_scaling!r}")
    if not cfg.qk_norm:
        bad.append("qk_norm=False (the graphs expect per-head q/k norm weights)")
    elif not cfg.qk_norm_affine:
        bad.append("qk_norm_affine=False (the graphs expect per-head q/k norm weights)")
    for flag in ("attn_bias", "post_norm", "scale_residual_by_depth", "embedding_scale"):
        if getattr(cfg, flag):
            bad.append(flag)
    if cfg.logit_soft_cap:
        bad.append("logit_soft_cap")
    if any(cfg.moe_layers):
        kw = cfg.moe_router_kwargs or {}
        if name(cfg.moe_router) != "topk":
            bad.append(f"moe_router={name(cfg.moe_router)!r}")
        if kw.get("score", kw.get("score_func", "sigmoid")) not in GATING:
            bad.append(f"router score {kw.get('score')!r}")
        if cfg.moe_mlp not in (None, "moe"):
            bad.append(f"moe_mlp={cfg.moe_mlp!r}")
    return bad


def convert(state: dict, cfg, out: str, *, name: str = "kohaku", arch: str = "auto", out_dtype: str = "f16", expand_kv: bool = True,
            tokenizer: str | None = None, turn_end: str = "<|im_end|>", chat_template: bool = True,
            allow_lossy: bool = False) -> dict:
    lossy = unrepresentable(cfg)
    if lossy and not allow_lossy:
        raise ValueError("llama.cpp's " + ("dots1" if any(cfg.moe_layers) else "qwen3") + " graph cannot express: "
                         + ", ".join(lossy) + " (pass allow_lossy / --allow-lossy to write the file anyway)")
    state = {k.removeprefix("module."): v for k, v in state.items()}
    sparse = any(k.endswith("mlp.router.weight") for k in state)
    if arch == "auto":
        arch = "dots1" if sparse else "qwen3"
    dense_ff = next((v.shape[0] // 2 for k, v in state.items() if k.endswith("mlp.w_in.weight") and ".shared." not in k), 0)
    expert_ff = next((v.shape[1] // 2 for k, v in state.items() if k.endswith("mlp.w_in") and v.dim() == 3), None)
    meta = hparams(cfg, arch, name, out_dtype, expand_kv, dense_ff or (expert_ff or 0), expert_ff if sparse else None)
    if tokenizer:
        meta.update(tokenizer_meta(tokenizer, turn_end, chat_template))
    tensors = tensor_map(state, cfg, expand_kv)
    write_gguf(out, tensors, meta, out_dtype=out_dtype)
    return {"arch": arch, "tensors": len(tensors), "dtype": out_dtype, "metadata_keys": len(meta), "lossy": lossy}


def main(argv=None) -> int:
    from kohakuwullm_b200.models import get_preset
    from kohakuwullm_b200.utils.config import parse_value

    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--ckpt", required=True)
    ap.add_argument("--preset", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--set", action="append", default=[], help="architecture override KEY=VALUE")
    ap.add_argument("--arch", default="auto", choices=["auto", "dots1", "qwen3"])
    ap.add_argument("--out-dtype", default="f16", choices=sorted(FILE_TYPE))
    ap.add_argument("--no-expand-kv", action="store_true")
    ap.add_argument("--tokenizer", default=None, help="directory with tokenizer.json (+ tokenizer_config.json)")
    ap.add_argument("--turn-end-token", default="<|im_end|>")
    ap.add_argument("--no-chat-template", action="store_true")
    ap.add_argument("--allow-lossy", action="store_true", help="write the file although the target graph lacks some of the model's options")
    a = ap.parse_args(argv)
    cfg = get_preset(a.preset, **{k: parse_value(v) for k, v in (kv.split("=", 1) for kv in a.set)})
    state = torch.load(a.ckpt, map_location="cpu", weights_only=False)
    state = state.get("state_dict", state)
    info = convert(state, cfg, a.out, name=a.preset, arch=a.arch, out_dtype=a.out_dtype, expand_kv=not a.no_expand_kv,
                   tokenizer=a.tokenizer, turn_end=a.turn_end_token, chat_template=not a.no_chat_template,
                   allow_lossy=a.allow_lossy)
    print(f"wrote {a.out}: {info['tensors']} tensors, arch={info['arch']}, {info['dtype']}"
          + (f" (NOT expressed in the file: {', '.join(info['lossy'])})" if info["lossy"] else ""))
    return 0


if __name__ == "__main__":
    sys.exit(main())
