"""Do 16-bit weights stop moving under round-to-nearest write-back, and at which learning rate?

Round-to-nearest discards an update smaller than half a unit in the last place of the weight it lands on, so the
coordinate keeps its bits while its gradient is still non-zero. This script measures that directly as the
NEVER-MOVED share: weight elements still bit-identical to their initial value after N optimizer steps. The learning
rate is the instrument: sweeping it walks the update across the half-ulp threshold in minutes, which is what the
tail of a decaying schedule does over a whole run.

Arms differ only in the write-back rule of ``StochasticAdamW`` (fp32 moments and update arithmetic, data and seed
are shared): ``nearest``, ``stochastic``, ``kahan``. Reported per arm and learning rate: the never-moved share over
the matrices of the blocks (token-indexed tables are left out: a row whose token never occurs gets no gradient under
any rule), the share of per-step updates above half an ulp at the last step (the tail, not the median, decides
whether an element ever moves: one surviving step out of N is enough), and whether decoupled weight decay survives
(``lr * wd`` against ``2^-(m+1)``, m = 7 mantissa bits for bf16, 10 for fp16).

    python -m kohakuwullm_b200.bench.lost_update --steps 100 --out out/lost_update

Runs on CPU or GPU; ``--out`` also writes an SVG. Reference: scripts/bench/kernel/lost_update.py.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch

DTYPES = {"bf16": torch.bfloat16, "fp16": torch.float16}
MANTISSA = {torch.bfloat16: 7, torch.float16: 10}
LR_GRID = (3e-4, 3e-5, 3e-6, 3e-7)      # peak, a 0.1x cosine floor, and two decades below
ARMS = ("nearest", "stochastic", "kahan")
WEIGHT_DECAY = 0.1


def half_ulp(param: torch.Tensor) -> torch.Tensor:
    """Half of the distance to the next representable value of the parameter's own dtype, as fp32."""
    away = torch.nextafter(param, torch.full_like(param, float("inf")))
    return 0.5 * (away.float() - param.float()).abs()


def measured_parameters(model) -> dict[str, torch.Tensor]:
    """The matrices of the blocks: every element receives gradient at every step."""
    return {n: p for n, p in model.named_parameters() if p.dim() == 2 and "embed" not in n and "head" not in n
            and p.dtype in MANTISSA}


def decay_survives(lr: float, wd: float, dtype: torch.dtype) -> bool:
    """Decoupled decay shrinks a weight by the relative amount ``lr * wd``; round-to-nearest keeps it only above
    half an ulp, which relative to the weight is at least ``2^-(m+2)`` and at most ``2^-(m+1)``."""
    return lr * wd > 2.0 ** -(MANTISSA[dtype] + 1)


def run_arm(arm: str, lr: float, dtype: torch.dtype, args, data) -> dict:
    from kohakuwullm_b200.models import LMBackbone, get_preset
    from kohakuwullm_b200.models.seqinfo import SeqInfo
    from kohakuwullm_b200.training.optim.lowbit import cast_parameters_
    from kohakuwullm_b200.training.optim.lowbit_optim import StochasticAdamW

    torch.manual_seed(args.seed)
    cfg = get_preset("B200-smoke", vocab_size=args.vocab, dim=args.dim, depth=args.depth, heads=args.dim // 32,
                     kv_heads=args.dim // 32, head_dim=32, mlp_hidden=2 * args.dim, mxfp8=False)
    model = LMBackbone(cfg).to(args.device)
    cast_parameters_(model, dtype)
    watched = measured_parameters(model)
    initial = {n: p.detach().clone() for n, p in watched.items()}
    opt = StochasticAdamW(model.parameters(), lr=lr, weight_decay=WEIGHT_DECAY,
                          rounding=arm if dtype == torch.bfloat16 or arm != "stochastic" else "nearest", seed=args.seed)
    above = 0.0
    for step in range(args.steps):
        ids = data[step % len(data)].to(args.device)
        with torch.autocast(args.device.split(":")[0], dtype=dtype, enabled=args.device != "cpu" or dtype == torch.bfloat16):
            hidden = model(ids[:, :-1], SeqInfo.padded(ids.shape[0], ids.shape[1] - 1, device=ids.device))
            logits = model.head.logits(hidden).float()
        loss = torch.nn.functional.cross_entropy(logits.reshape(-1, logits.shape[-1]), ids[:, 1:].reshape(-1))
        opt.zero_grad(set_to_none=True)
        loss.backward()
        if step == args.steps - 1:
            # the update each watched element is about to receive, against half an ulp of where it stands
            n_el = n_above = 0
            for n, p in watched.items():
                st = opt.state[p]
                if not st:
                    continue
                b1, b2 = opt.param_groups[0]["betas"]
                g = p.grad.float()
                m = st["exp_avg"].float() * b1 + (1 - b1) * g
                v = st["exp_avg_sq"].float() * b2 + (1 - b2) * g * g
                t = st["step"] + 1
                upd = lr * (m / (1 - b1 ** t)) / ((v / (1 - b2 ** t)).sqrt() + 1e-8)
                n_above += int((upd.abs() > half_ulp(p.detach())).sum())
                n_el += p.numel()
            above = n_above / max(n_el, 1)
        opt.step()
    same = sum(int((p.detach() == initial[n]).sum()) for n, p in watched.items())
    total = sum(p.numel() for p in watched.values())
    return {"arm": arm, "lr": lr, "dtype": str(dtype).split(".")[-1], "never_moved": same / total,
            "updates_above_half_ulp": above, "decay_survives_nearest": decay_survives(lr, WEIGHT_DECAY, dtype),
            "final_loss": float(loss.detach())}


def main(argv=None) -> int:
    from kohakuwullm_b200.bench.mxfp8_rounding import chain_data

    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--dtype", default="bf16", choices=sorted(DTYPES))
    ap.add_argument("--lrs", type=float, nargs="+", default=list(LR_GRID))
    ap.add_argument("--arms", nargs="+", default=list(ARMS), choices=ARMS)
    ap.add_argument("--dim", type=int, default=128)
    ap.add_argument("--depth", type=int, default=2)
    ap.add_argument("--vocab", type=int, default=512)
    ap.add_argument("--rows", type=int, default=8)
    ap.add_argument("--length", type=int, default=65)
    ap.add_argument("--batches", type=int, default=32, help="distinct batches, cycled: the gradient keeps its noise")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--out", default=None, help="directory for lost_update.json and lost_update.svg")
    args = ap.parse_args(argv)
    dtype = DTYPES[args.dtype]
    data = chain_data(args.batches, args.rows, args.length, args.vocab, args.seed)
    rows = [run_arm(arm, lr, dtype, args, data) for arm in args.arms for lr in args.lrs]
    for r in rows:
        print(json.dumps(r))
    if args.out:
        from kohakuwullm_b200.bench import plotting as pl

        os.makedirs(args.out, exist_ok=True)
        with open(os.path.join(args.out, "lost_update.json"), "w") as fh:
            json.dump(rows, fh, indent=1)
        fig, pal = pl.Figure(1, 2), pl.Palette()
        left, right = fig.panels
        left.title, left.xlabel, left.ylabel, left.logx = f"never-moved share ({args.dtype}, {args.steps} steps)", "learning rate", "share", True
        right.title, right.xlabel, right.ylabel, right.logx = "updates above half an ulp", "learning rate", "share", True
        for arm in args.arms:
            mine = sorted((r for r in rows if r["arm"] == arm), key=lambda r: r["lr"])
            left.line(arm, [r["lr"] for r in mine], [r["never_moved"] for r in mine], pal.color(arm))
            right.line(arm, [r["lr"] for r in mine], [r["updates_above_half_ulp"] for r in mine], pal.color(arm))
        pl.save_figure(fig, os.path.join(args.out, "lost_update.svg"))
    return 0


if __name__ == "__main__":
    sys.exit(main())
