"""Checkpoint -> Hugging Face repository: ``python -m kohakuwullm_b200.cli.to_hf --ckpt x.ckpt --preset P --out dir``.
Reference: scripts/tools/to_hf.py."""

from __future__ import annotations

import argparse

import torch


def main(argv=None):
    from kohakuwullm_b200.export.hf.convert import export_hf
    from kohakuwullm_b200.models import get_preset
    from kohakuwullm_b200.utils.config import parse_value

    ap = argparse.ArgumentParser()
    ap.add_argument("--ckpt", required=True)
    ap.add_argument("--preset", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--set", action="append", default=[])
    args = ap.parse_args(argv)
    cfg = get_preset(args.preset, **{k: parse_value(v) for k, v in (kv.split("=", 1) for kv in args.set)})
    state = torch.load(args.ckpt, map_location="cpu", weights_only=False)["state_dict"]
    export_hf(state, cfg, args.out)
    print(f"wrote {args.out}")


if __name__ == "__main__":
    main()
