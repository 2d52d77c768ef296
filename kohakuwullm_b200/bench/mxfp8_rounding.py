"""A/B of the two exponent conventions of MXFP8 block scales: round UP (the kernels' rule, nothing saturates) against
round to NEAREST (half of the blocks get a binade of extra resolution, their largest elements clip at 448).

Both arms run through the same quantise-dequantise emulation of the MXFP8 linear in plain PyTorch, so the only
difference between them is the rule: FPROP multiplies ``x`` and ``W`` quantised along K, DGRAD multiplies ``dy`` and
``W^T`` quantised along N, WGRAD stays a bf16-input product, exactly the recipe of ``ops/mxfp8``. With the round-up
rule the emulated forward equals ``mxfp8_linear_reference`` (and so the tcgen05 kernel) bit for bit.

    python -m kohakuwullm_b200.bench.mxfp8_rounding --steps 300 --replicates 2

trains a small model on the structured chain data of ``bench.loss_gap`` under both rules and prints one JSON line:
final-window loss of every run, the gap between the arm means and the floor (largest gap between two runs of one
arm). Runs on CPU or GPU. Reference: src/kohakuwullm/bench/vendor/mxfp8_rounding.py:1-82 (it rewrites its Triton
quantiser's source for the second arm; here the rule is an argument of the reference quantiser).
"""

from __future__ import annotations

import argparse
import json
import sys
import types

import torch

from kohakuwullm_b200.ops import mxfp8 as mx

RULES = ("ceil", "nearest")


def fake_quantize(t: torch.Tensor, rule: str) -> torch.Tensor:
    """Quantise (rows, K) along K and dequantise again, fp32 out."""
    q, e = mx.quantize_reference(t, rule)
    return mx.dequantize(q, e)


class _EmulatedMXFP8Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, rule: str):
        ctx.save_for_backward(x, w)
        ctx.rule = rule
        return (fake_quantize(x, rule) @ fake_quantize(w, rule).t()).to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dx = dw = None
        if ctx.needs_input_grad[0]:
            # both operands quantised along the contraction, which for DGRAD is the OUTPUT feature axis
            dx = (fake_quantize(dy.contiguous(), ctx.rule) @ fake_quantize(w.t().contiguous(), ctx.rule).t()).to(x.dtype)
        if ctx.needs_input_grad[1]:
            dw = (dy.to(torch.bfloat16).float().t() @ x.to(torch.bfloat16).float()).to(w.dtype)
        return dx, dw, None


def emulated_mxfp8_linear(x: torch.Tensor, w: torch.Tensor, rule: str = "ceil") -> torch.Tensor:
    lead = x.shape[:-1]
    return _EmulatedMXFP8Linear.apply(x.reshape(-1, x.shape[-1]), w, rule).reshape(*lead, w.shape[0])


def emulate_mxfp8_(model: torch.nn.Module, rule: str = "ceil", scope: tuple[str, ...] | None = None) -> int:
    """Route every bias-free ``Linear`` whose feature sizes are multiples of 32 (and whose qualified name contains
    one of ``scope``, if given) through the emulation, in place. Returns how many layers were rerouted. The model
    keeps its parameters; ``restore_(model)`` undoes it."""
    from kohakuwullm_b200.models.components.mlp import Linear

    if rule not in RULES:
        raise ValueError(f"unknown exponent rule {rule!r}")
    count = 0
    for name, mod in model.named_modules():
        if not isinstance(mod, Linear) or mod.bias is not None:
            continue
        if mod.in_features % 32 or mod.out_features % 32 or (scope and not any(s in name for s in scope)):
            continue

        def forward(self, x, _rule=rule):
            return emulated_mxfp8_linear(x, self.weight, _rule)

        mod.forward = types.MethodType(forward, mod)
        count += 1
    return count


def restore_(model: torch.nn.Module) -> None:
    for mod in model.modules():
        mod.__dict__.pop("forward", None)


def block_statistics(x: torch.Tensor) -> dict:
    """What the two rules do to one tensor: share of blocks whose scale differs, share of elements that saturate
    under round-to-nearest, and the relative RMS error of both."""
    x2 = x.reshape(-1, x.shape[-1]).float()
    out = {}
    qs = {}
    for rule in RULES:
        q, e = mx.quantize_reference(x2, rule)
        qs[rule] = (q, e)
        out[f"rel_rms_{rule}"] = float((mx.dequantize(q, e) - x2).pow(2).mean().sqrt() / x2.pow(2).mean().sqrt())
    out["blocks_with_smaller_scale"] = float((qs["nearest"][1] < qs["ceil"][1]).float().mean())
    out["saturated_share_nearest"] = float((qs["nearest"][0].float().abs() >= mx.E4M3_MAX).float().mean())
    out["saturated_share_ceil"] = float(((qs["ceil"][0].float().abs() >= mx.E4M3_MAX)
                                         & (x2.abs() > 0)).float().mean())
    return out


def train_arm(rule: str | None, seed: int, args, data) -> float:
    """Final-window mean loss of one run; ``rule=None`` is the unquantised arm."""
    from kohakuwullm_b200.models import LMBackbone, get_preset
    from kohakuwullm_b200.models.seqinfo import SeqInfo

    torch.manual_seed(seed)
    cfg = get_preset("B200-smoke", vocab_size=args.vocab, dim=args.dim, depth=args.depth, heads=args.dim // 32,
                     kv_heads=args.dim // 32, head_dim=32, mlp_hidden=2 * args.dim, mxfp8=False)
    model = LMBackbone(cfg).to(args.device)
    if rule is not None:
        emulate_mxfp8_(model, rule)
    opt = torch.optim.AdamW(model.parameters(), lr=args.lr, betas=(0.9, 0.95), weight_decay=0.0)
    losses = []
    for step in range(args.steps):
        ids = data[step % len(data)].to(args.device)
        hidden = model(ids[:, :-1], SeqInfo.padded(ids.shape[0], ids.shape[1] - 1, device=ids.device))
        logits = model.head.logits(hidden).float()
        loss = torch.nn.functional.cross_entropy(logits.reshape(-1, logits.shape[-1]), ids[:, 1:].reshape(-1))
        opt.zero_grad(set_to_none=True)
        loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        losses.append(float(loss.detach()))
    window = losses[-args.window:]
    return sum(window) / len(window)


def chain_data(batches: int, rows: int, length: int, vocab: int, seed: int) -> list[torch.Tensor]:
    """Order-1 Markov chains with four successors per token (best reachable loss ln 4): structured enough that the
    arms separate if the arithmetic differs."""
    g = torch.Generator().manual_seed(seed)
    succ = torch.randint(0, vocab, (vocab, 4), generator=g)
    out = []
    for _ in range(batches):
        ids = torch.empty(rows, length, dtype=torch.long)
        ids[:, 0] = torch.randint(0, vocab, (rows,), generator=g)
        pick = torch.randint(0, 4, (rows, length), generator=g)
        for t in range(1, length):
            ids[:, t] = succ[ids[:, t - 1], pick[:, t]]
        out.append(ids)
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--window", type=int, default=50)
    ap.add_argument("--replicates", type=int, default=2)
    ap.add_argument("--dim", type=int, default=128)
    ap.add_argument("--depth", type=int, default=2)
    ap.add_argument("--vocab", type=int, default=512)
    ap.add_argument("--rows", type=int, default=16)
    ap.add_argument("--length", type=int, default=65)
    ap.add_argument("--batches", type=int, default=64)
    ap.add_argument("--lr", type=float, default=2e-3)
    ap.add_argument("--seed", type=int, default=5)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    args = ap.parse_args(argv)
    data = chain_data(args.batches, args.rows, args.length, args.vocab, args.seed)
    reps = max(args.replicates, 2)            # two at least, or there is no floor to compare the gap with
    runs = {str(rule): [train_arm(rule, args.seed + r, args, data) for r in range(reps)] for rule in (None,) + RULES}
    mean = {k: sum(v) / len(v) for k, v in runs.items()}
    floor = max(max(v) - min(v) for v in runs.values())
    print(json.dumps({"bench": "mxfp8_rounding", "steps": args.steps, "window": args.window, "runs": runs,
                      "gap_ceil_vs_unquantised": mean["ceil"] - mean["None"],
                      "gap_nearest_vs_unquantised": mean["nearest"] - mean["None"],
                      "gap_nearest_vs_ceil": mean["nearest"] - mean["ceil"], "floor": floor,
                      "device": str(args.device)}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
