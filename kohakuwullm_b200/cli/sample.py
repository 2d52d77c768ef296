"""Generate text from a checkpoint.

    python -m kohakuwullm_b200.cli.sample --ckpt run/last.ckpt --preset Kohaku-500M --prompt "Once upon" --count 4
    python -m kohakuwullm_b200.cli.sample --ckpt run/last.ckpt --preset Kohaku-500M --prompts-file prompts.txt \
        --max-new-tokens 0 --min-p 0.1 --bench-steps 3

``--prompt`` may be given several times; ``--prompts-file`` holds one prompt per line. Every prompt is decoded
``--count`` times in one batch (rows of equal length decode together). ``--max-new-tokens 0`` decodes until every row
has emitted EOS or the model's context is full. ``--bench-steps N`` repeats the decode N times and prints milliseconds
per generated token. The checkpoint is a whole-model-named one (any pipeline split, DDP or single process wrote it).
Reference: scripts/tools/sample.py.
"""

from __future__ import annotations

import argparse
import sys
import time

import torch


def load_model(ckpt_path: str, preset: str, overrides: dict, device: torch.device, dtype: str, attention: str | None):
    from kohakuwullm_b200.models import LMBackbone, get_preset
    from kohakuwullm_b200.pipe import checkpoint as ckpt

    extra = dict(overrides, mxfp8=False)
    if attention:
        extra["attn"] = attention
    cfg = get_preset(preset, **extra)
    model = LMBackbone(cfg, init=False)
    ckpt.load(ckpt_path, model)
    model.to(device).eval()
    if dtype == "bf16" and device.type == "cuda":
        from kohakuwullm_b200.training.optim.lowbit import cast_parameters_

        cast_parameters_(model, torch.bfloat16)
    return model


def main(argv=None) -> int:
    from kohakuwullm_b200.data import ByteTokenizer
    from kohakuwullm_b200.generation.engine import SAMPLE_SEED, LocalGenerator
    from kohakuwullm_b200.utils.config import parse_value

    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--ckpt", required=True)
    ap.add_argument("--preset", required=True)
    ap.add_argument("--set", action="append", default=[], help="architecture override KEY=VALUE")
    ap.add_argument("--prompt", action="append", default=[])
    ap.add_argument("--prompts-file")
    ap.add_argument("--count", type=int, default=1, help="samples per prompt")
    ap.add_argument("--tokenizer", default="byte")
    ap.add_argument("--max-new-tokens", type=int, default=128, help="0: until EOS or the context is full")
    ap.add_argument("--temperature", type=float, default=0.8)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=0.95)
    ap.add_argument("--min-p", type=float, default=0.0)
    ap.add_argument("--seed", type=int, default=SAMPLE_SEED)
    ap.add_argument("--device", default="auto")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp32"])
    ap.add_argument("--attention", default=None, help="attention backend override (e.g. sdpa)")
    ap.add_argument("--no-cache", action="store_true", help="recompute the whole prefix every step (reference path)")
    ap.add_argument("--bench-steps", type=int, default=0)
    args = ap.parse_args(argv)
    overrides = {k: parse_value(v) for k, v in (kv.split("=", 1) for kv in args.set)}
    device = torch.device(("cuda" if torch.cuda.is_available() else "cpu") if args.device == "auto" else args.device)
    model = load_model(args.ckpt, args.preset, overrides, device, args.dtype, args.attention)
    if args.tokenizer == "byte":
        tok = ByteTokenizer()
    else:
        from transformers import AutoTokenizer

        tok = AutoTokenizer.from_pretrained(args.tokenizer)
    prompts = list(args.prompt)
    if args.prompts_file:
        with open(args.prompts_file) as f:
            prompts += [line.rstrip("\n") for line in f if line.strip()]
    if not prompts:
        prompts = [""]
    bos = getattr(tok, "bos_token_id", None)
    eos = getattr(tok, "eos_token_id", 0) or 0
    gen = LocalGenerator(model, eos_id=eos, use_cache=not args.no_cache)
    gen.rng(device).manual_seed(args.seed)
    budget = args.max_new_tokens if args.max_new_tokens > 0 else None
    sampling = dict(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p, min_p=args.min_p)
    for prompt in prompts:
        ids = ([bos] if bos is not None else []) + list(tok.encode(prompt))
        batch = torch.tensor([ids or [eos]] * args.count, device=device)
        out = gen.generate(batch, budget, **sampling)
        for i, row in enumerate(out.tolist()):
            text = tok.decode(row[len(ids):])
            print(f"--- prompt {prompt[:40]!r} sample {i}\n{prompt}{text}")
        if args.bench_steps > 0:
            if device.type == "cuda":
                torch.cuda.synchronize()
            t0 = time.perf_counter()
            new = 0
            for _ in range(args.bench_steps):
                o = gen.generate(batch, budget, **sampling)
                new += (o.shape[1] - batch.shape[1]) * o.shape[0]
            if device.type == "cuda":
                torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            print(f"--- decode: {1e3 * dt / max(new // max(args.count, 1), 1):.2f} ms per step, {new / dt:.1f} tokens/s "
                  f"({args.count} rows)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
