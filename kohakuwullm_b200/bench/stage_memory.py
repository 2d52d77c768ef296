"""Does a preset fit on the card, stage by stage, before anything is allocated?

The model is built on the ``meta`` device (no memory, seconds even for tens of billions of parameters), split by the
pipeline planner, cast by the same rule training uses (norms, routers, sinks and biases stay fp32), and the bytes that
live for the whole run are added up per stage:

=====================  ==========================================================================================
weights                parameters in their training dtype
gradients              one fp32 ``main_grad`` element per parameter (gradients accumulate in fp32 flat buffers)
optimizer state        by optimizer: flat fused AdamW keeps fp32 master + two fp32 moments (12 B per parameter; under
                       data parallelism with the fused reduce-scatter step the three are sharded over the ranks);
                       ``adamw`` two moments in the parameter dtype; ``adamw16`` two 16-bit moments; ``adamw8bit`` /
                       ``adamw4bit`` / ``adamwfp8`` block-quantised moments with one fp32 scale per block; ``muon`` one
                       momentum for the hidden matrices and AdamW moments for the rest; ``sgd`` nothing
MXFP8 copies           with ``--mxfp8``: two e4m3 copies (along K and along N) of every converted weight, plus one
                       scale byte per 32 elements
=====================  ==========================================================================================

What is left of the card's memory after these is what activations, the attention workspaces and the allocator's
slack can use; ``bench.step_throughput`` reports the measured peak of a real step (``peak_mem_gib``) to set beside it.

    python -m kohakuwullm_b200.bench.stage_memory --preset MoE-8B-A1B --stages 4 --optimizer muon --param-dtype bf16

Reference: scripts/bench/e2e/stage_memory.py (it builds each stage on the GPU and takes a real step; this estimator
needs no GPU and is exact for the persistent bytes, which is the part that decides whether a stage fits at all).
"""

from __future__ import annotations

import argparse
import json
import sys

import torch

DTYPES = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}
CARD_GIB = 180.0
QUANT_BLOCK = {"adamw8bit": 256, "adamwfp8": 256, "adamw4bit": 128}     # elements per fp32 scale


def _bytes_of(params) -> int:
    return sum(p.numel() * p.element_size() for p in params)


def optimizer_state_bytes(named_params: list[tuple[str, torch.Tensor]], optimizer: str, shard: int = 1) -> int:
    """Bytes of optimizer state for these parameters. ``shard`` divides the state of the flat fused AdamW (the fused
    data-parallel step keeps one 1/N slice of master and moments per rank)."""
    n = sum(p.numel() for _, p in named_params)
    if optimizer in ("fused_adamw", "flat_adamw"):
        return 12 * n // max(shard, 1)
    if optimizer == "adamw":
        return 2 * _bytes_of(p for _, p in named_params)
    if optimizer == "adamw16":
        return 4 * n
    if optimizer in ("adamw8bit", "adamwfp8"):
        return 2 * (n + 4 * -(-n // QUANT_BLOCK[optimizer]))
    if optimizer == "adamw4bit":
        return 2 * (-(-n // 2) + 4 * -(-n // QUANT_BLOCK[optimizer]))
    if optimizer == "stochastic_adamw":
        return 8 * n
    if optimizer == "muon":
        hidden = sum(p.numel() * p.element_size() for name, p in named_params
                     if p.dim() >= 2 and "embed" not in name and "head" not in name)
        rest = _bytes_of(p for _, p in named_params) - hidden
        return hidden + 2 * rest
    if optimizer == "sgd":
        return 0
    raise ValueError(f"no state model for optimizer {optimizer!r}")


def mxfp8_copy_bytes(stage) -> int:
    """Two fp8 copies with their scales for every linear the MXFP8 swap would convert (bias-free, both feature sizes
    multiples of 128) and for the stacked expert weights."""
    from kohakuwullm_b200.models.components.mlp import Linear

    total = 0
    for mod in stage.modules():
        if isinstance(mod, Linear) and mod.bias is None and mod.in_features % 128 == 0 and mod.out_features % 128 == 0:
            total += 2 * (mod.weight.numel() + mod.weight.numel() // 32)
    for name, p in stage.named_parameters():
        if p.dim() == 3 and ("w_in" in name or "w_out" in name):        # stacked experts (E, out, in)
            total += 2 * (p.numel() + p.numel() // 32)
    return total


def stage_rows(preset: str, stages: int = 1, *, overrides: dict | None = None, param_dtype: str = "bf16",
               optimizer: str = "fused_adamw", mxfp8: bool = False, seq_len: int = 4096, dp: int = 1,
               card_gib: float = CARD_GIB) -> list[dict]:
    from kohakuwullm_b200.models import LMBackbone, get_preset
    from kohakuwullm_b200.training.optim.lowbit import cast_parameters_
    from kohakuwullm_b200.training.parallel.pipeline import LMStage, plan_for

    cfg = get_preset(preset, **dict(overrides or {}, mxfp8=False))
    with torch.device("meta"):
        backbone = LMBackbone(cfg, init=False)
    rows = []
    for plan in plan_for(cfg, stages, seq_len):
        stage = LMStage(backbone, plan)
        if param_dtype != "fp32":
            cast_parameters_(stage, DTYPES[param_dtype])
        named = list(stage.named_parameters())
        n = sum(p.numel() for _, p in named)
        weights = _bytes_of(p for _, p in named)
        state = optimizer_state_bytes(named, optimizer, shard=dp)
        copies = mxfp8_copy_bytes(stage) if mxfp8 else 0
        persistent = weights + 4 * n + state + copies
        rows.append({"stage": plan.index, "layers": f"{plan.start_layer}..{plan.end_layer}", "params_m": n / 1e6,
                     "kept_fp32_m": sum(p.numel() for _, p in named if p.dtype == torch.float32
                                        and param_dtype != "fp32") / 1e6,
                     "weights_gib": weights / 2 ** 30, "grads_gib": 4 * n / 2 ** 30,
                     "optimizer_gib": state / 2 ** 30, "mxfp8_gib": copies / 2 ** 30,
                     "persistent_gib": persistent / 2 ** 30, "left_gib": card_gib - persistent / 2 ** 30,
                     "fits": persistent / 2 ** 30 < card_gib})
    return rows


def table(rows: list[dict]) -> str:
    head = "| stage | layers | params (M) | weights | grads | optimizer | MXFP8 | persistent | left | fits |"
    lines = [head, "|" + "---|" * 10]
    for r in rows:
        lines.append(f"| {r['stage']} | {r['layers']} | {r['params_m']:.1f} | {r['weights_gib']:.2f} | "
                     f"{r['grads_gib']:.2f} | {r['optimizer_gib']:.2f} | {r['mxfp8_gib']:.2f} | "
                     f"{r['persistent_gib']:.2f} | {r['left_gib']:.1f} | {'yes' if r['fits'] else 'NO'} |")
    return "\n".join(lines)


def main(argv=None) -> int:
    from kohakuwullm_b200.utils.config import parse_value

    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--preset", default="MoE-8B-A1B")
    ap.add_argument("--set", action="append", default=[], help="architecture override KEY=VALUE")
    ap.add_argument("--stages", type=int, default=1)
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--param-dtype", default="bf16", choices=sorted(DTYPES))
    ap.add_argument("--optimizer", default="fused_adamw")
    ap.add_argument("--mxfp8", action="store_true")
    ap.add_argument("--dp", type=int, default=1, help="data-parallel ranks sharing the flat optimizer state")
    ap.add_argument("--card-gib", type=float, default=CARD_GIB)
    ap.add_argument("--json", action="store_true")
    args = ap.parse_args(argv)
    overrides = {k: parse_value(v) for k, v in (kv.split("=", 1) for kv in args.set)}
    rows = stage_rows(args.preset, args.stages, overrides=overrides, param_dtype=args.param_dtype,
                      optimizer=args.optimizer, mxfp8=args.mxfp8, seq_len=args.seq_len, dp=args.dp,
                      card_gib=args.card_gib)
    print(json.dumps(rows) if args.json else table(rows))
    return 0 if all(r["fits"] for r in rows) else 1


if __name__ == "__main__":
    sys.exit(main())
