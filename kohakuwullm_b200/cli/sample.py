"""Generate text from a checkpoint: ``python -m kohakuwullm_b200.cli.sample --ckpt run/last.ckpt --preset ... --prompt "..."``.
Reference: scripts/tools/sample.py."""

from __future__ import annotations

import argparse

import torch


def main(argv=None):
    from kohakuwullm_b200.data import ByteTokenizer
    from kohakuwullm_b200.generation.engine import LocalGenerator
    from kohakuwullm_b200.models import LMBackbone, get_preset
    from kohakuwullm_b200.pipe import checkpoint as ckpt
    from kohakuwullm_b200.utils.config import parse_value

    ap = argparse.ArgumentParser()
    ap.add_argument("--ckpt", required=True)
    ap.add_argument("--preset", required=True)
    ap.add_argument("--set", action="append", default=[])
    ap.add_argument("--prompt", default="")
    ap.add_argument("--tokenizer", default="byte")
    ap.add_argument("--max-new-tokens", type=int, default=128)
    ap.add_argument("--temperature", type=float, default=0.8)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=0.95)
    ap.add_argument("--min-p", type=float, default=0.0)
    args = ap.parse_args(argv)
    overrides = dict(kv.split("=", 1) for kv in args.set)
    cfg = get_preset(args.preset, **{k: parse_value(v) for k, v in overrides.items()}, mxfp8=False)
    model = LMBackbone(cfg, init=False)
    ckpt.load(args.ckpt, model)
    device = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    model.to(device).eval()
    if args.tokenizer == "byte":
        tok = ByteTokenizer()
    else:
        from transformers import AutoTokenizer

        tok = AutoTokenizer.from_pretrained(args.tokenizer)
    ids = torch.tensor([[getattr(tok, "bos_token_id", 0) or 0] + list(tok.encode(args.prompt))], device=device)
    out = LocalGenerator(model, eos_id=getattr(tok, "eos_token_id", 0) or 0).generate(
        ids, args.max_new_tokens, temperature=args.temperature, top_k=args.top_k, top_p=args.top_p, min_p=args.min_p)
    print(tok.decode(out[0].tolist()))


if __name__ == "__main__":
    main()
