"""Checkpoint -> Hugging Face repository with stand-alone modelling code.

    python -m kohakuwullm_b200.cli.to_hf --ckpt run/last.ckpt --preset Kohaku-MoE-1B --out hf/kohaku-moe-1b \
        --tokenizer models/tokenizer --out-dtype bf16

The output directory holds ``config.json``, safetensors weights, ``configuration_kohaku.py`` / ``modeling_kohaku.py``
(loadable with ``trust_remote_code=True`` without this framework installed) and, with ``--tokenizer``, the tokenizer
files. ``--check`` reloads the export and compares its logits with the source model on a few tokens.
Reference: scripts/tools/to_hf.py.
"""

from __future__ import annotations

import argparse
import os
import shutil
import sys

import torch

DTYPES = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}
TOKENIZER_FILES = ("tokenizer.json", "tokenizer_config.json", "special_tokens_map.json", "chat_template.jinja")


def main(argv=None) -> int:
    from kohakuwullm_b200.export.hf.convert import export_hf
    from kohakuwullm_b200.models import get_preset
    from kohakuwullm_b200.utils.config import parse_value

    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--ckpt", required=True)
    ap.add_argument("--preset", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--set", action="append", default=[], help="architecture override KEY=VALUE")
    ap.add_argument("--out-dtype", default="bf16", choices=sorted(DTYPES))
    ap.add_argument("--tokenizer", default=None, help="directory whose tokenizer files are copied into the export")
    ap.add_argument("--check", action="store_true", help="reload the export and compare logits with the source weights")
    args = ap.parse_args(argv)
    cfg = get_preset(args.preset, **{k: parse_value(v) for k, v in (kv.split("=", 1) for kv in args.set)})
    payload = torch.load(args.ckpt, map_location="cpu", weights_only=False)
    state = {k.removeprefix("module."): v for k, v in payload.get("state_dict", payload).items()}
    exported = export_hf(state, cfg, args.out, dtype=DTYPES[args.out_dtype])
    copied = []
    if args.tokenizer:
        for name in TOKENIZER_FILES:
            src = os.path.join(args.tokenizer, name)
            if os.path.exists(src):
                shutil.copy(src, os.path.join(args.out, name))
                copied.append(name)
    if args.check:
        from kohakuwullm_b200.models import LMBackbone
        from kohakuwullm_b200.models.seqinfo import SeqInfo

        model = LMBackbone(cfg.replace(mxfp8=False), init=False)
        model.load_state_dict(state, strict=False)
        model.eval()
        ids = torch.randint(0, cfg.vocab_size, (1, 12), generator=torch.Generator().manual_seed(0))
        with torch.no_grad():
            want = model.head.logits(model(ids, SeqInfo.padded(1, 12)))[0].float()
            got = exported.float()(ids).logits[0].float()
        err = float((got - want).abs().max() / want.abs().max().clamp(min=1e-6))
        print(f"check: largest relative logit difference {err:.2e}")
        if err > 5e-2:
            raise SystemExit("the exported model does not reproduce the source logits")
    print(f"wrote {args.out}" + (f" (+ {', '.join(copied)})" if copied else ""))
    return 0


if __name__ == "__main__":
    sys.exit(main())
