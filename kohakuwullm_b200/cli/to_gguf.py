"""Checkpoint -> GGUF v3 file (tensors in f16/f32 plus architecture metadata), written with a small
self-contained writer (the ``gguf`` package is optional and absent here).
``python -m kohakuwullm_b200.cli.to_gguf --ckpt x.ckpt --preset P --out model.gguf``. Reference: scripts/tools/to_gguf.py."""

from __future__ import annotations

import argparse
import struct

import numpy as np
import torch

GGUF_MAGIC, GGUF_VERSION, ALIGN = 0x46554747, 3, 32
T_U32, T_F32, T_BOOL, T_STR, T_U64 = 4, 6, 7, 8, 10
GGML_F32, GGML_F16 = 0, 1


def _s(x: str) -> bytes:
    b = x.encode()
    return struct.pack("<Q", len(b)) + b


def _kv(key: str, value) -> bytes:
    out = _s(key)
    if isinstance(value, bool):
        return out + struct.pack("<IB", T_BOOL, int(value))
    if isinstance(value, int):
        return out + struct.pack("<IQ", T_U64, value)
    if isinstance(value, float):
        return out + struct.pack("<If", T_F32, value)
    return out + struct.pack("<I", T_STR) + _s(str(value))


def write_gguf(path: str, tensors: dict[str, torch.Tensor], meta: dict, f16: bool = True) -> None:
    infos, blobs, offset = b"", [], 0
    for name, t in tensors.items():
        arr = t.detach().float().cpu().numpy()
        use16 = f16 and arr.ndim >= 2
        arr = arr.astype(np.float16 if use16 else np.float32)
        dims = list(reversed(arr.shape))
        infos += _s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        infos += struct.pack("<IQ", GGML_F16 if use16 else GGML_F32, offset)
        raw = arr.tobytes()
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


def main(argv=None):
    from kohakuwullm_b200.models import get_preset

    ap = argparse.ArgumentParser()
    ap.add_argument("--ckpt", required=True)
    ap.add_argument("--preset", required=True)
    ap.add_argument("--out", required=True)
    args = ap.parse_args(argv)
    cfg = get_preset(args.preset)
    state = torch.load(args.ckpt, map_location="cpu", weights_only=False)["state_dict"]
    meta = {"general.architecture": "kohaku", "general.name": args.preset, "kohaku.block_count": cfg.depth,
            "kohaku.embedding_length": cfg.dim, "kohaku.attention.head_count": cfg.heads,
            "kohaku.attention.head_count_kv": cfg.kv_heads, "kohaku.attention.key_length": cfg.head_dim,
            "kohaku.rope.freq_base": float(cfg.rope_theta), "kohaku.context_length": cfg.max_position,
            "kohaku.vocab_size": cfg.vocab_size, "general.alignment": ALIGN}
    write_gguf(args.out, {k: v for k, v in state.items() if not k.endswith("load_accum")}, meta)
    print(f"wrote {args.out}")


if __name__ == "__main__":
    main()
