"""Loss-gap A/B run: train the same model with bf16 linears and with MXFP8 linears on a learnable synthetic
stream and compare the final-window loss against a replicate noise floor.

    python -m kohakuwullm_b200.bench.loss_gap --preset B200-dense-546M --depth 8 --steps 200

Data: a noisy affine token chain ``x[t+1] = (31 x[t] + 7 + e) mod V`` with ``e`` uniform in {0,1,2,3}, so the
best reachable loss is ln 4 and the curve is informative (uniform random tokens would pin every arm to ln V).
Arms: ``bf16`` (seed s), ``bf16_rep`` (same data, init seed s + 1: the run-to-run floor), ``mxfp8`` (seed s).
Prints one JSON line with the final-window means, the gap, the floor and the verdict of
``abtest.admissible``. Reference method: docs/performance/ab-testing.md of the reference
(src/kohakuwullm/bench/analysis/abtest.py).
"""

from __future__ import annotations

import argparse
import json

import torch

from kohakuwullm_b200.bench import abtest


def chain_packs(n_micro, tokens, len_min, len_max, vocab, seed):
    from kohakuwullm_b200.data.packing import collate_packed
    from kohakuwullm_b200.data.synthetic import draw_lengths

    g = torch.Generator().manual_seed(seed)
    packs = []
    for m in range(n_micro):
        docs = []
        for n in draw_lengths(tokens, len_min, len_max, g):
            x = torch.empty(n, dtype=torch.long)
            x[0] = int(torch.randint(0, vocab, (1,), generator=g))
            noise = torch.randint(0, 4, (n,), generator=g)
            for t in range(1, n):
                x[t] = (31 * int(x[t - 1]) + 7 + int(noise[t])) % vocab
            docs.append(x)
        packs.append(collate_packed(docs))
    return packs


def run_arm(args, mxfp8: bool, init_seed: int, data):
    from kohakuwullm_b200.models import LMBackbone, get_preset
    from kohakuwullm_b200.training.engine import TrainEngine

    cfg = get_preset(args.preset, depth=args.depth, vocab_size=args.vocab, mxfp8=mxfp8)
    torch.manual_seed(init_seed)
    with torch.device("cuda"):
        model = LMBackbone(cfg)
    eng = TrainEngine(model, lr=args.lr, param_dtype=torch.bfloat16)
    losses = []
    for step in range(args.steps):
        out = eng.step(data[step % len(data)])
        losses.append(out["ce"])
    return [float(x) for x in torch.stack(losses).cpu()]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", default="B200-dense-546M")
    ap.add_argument("--depth", type=int, default=8)
    ap.add_argument("--vocab", type=int, default=8192)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--window", type=int, default=40)
    ap.add_argument("--micro-tokens", type=int, default=4096)
    ap.add_argument("--accum", type=int, default=2)
    ap.add_argument("--lr", type=float, default=6e-4)
    ap.add_argument("--seed", type=int, default=5)
    ap.add_argument("--batches", type=int, default=50, help="distinct step batches (cycled)")
    args = ap.parse_args()
    data = [[p.to("cuda") for p in chain_packs(args.accum, args.micro_tokens, 64, 1024, args.vocab, args.seed * 1000 + i)]
            for i in range(args.batches)]
    a = run_arm(args, False, args.seed, data)
    rep = run_arm(args, False, args.seed + 1, data)
    b = run_arm(args, True, args.seed, data)
    gap = abtest.loss_gap(a, b, args.window)
    floor = abtest.noise_floor([a, rep], args.window)
    print(json.dumps({"preset": args.preset, "depth": args.depth, "steps": args.steps, "window": args.window,
                      "bf16_final": abtest.final_window_mean(a, args.window),
                      "bf16_replicate_final": abtest.final_window_mean(rep, args.window),
                      "mxfp8_final": abtest.final_window_mean(b, args.window), "first_loss": a[0],
                      "gap_mxfp8_minus_bf16": gap, "replicate_floor": floor,
                      "within_noise": abtest.admissible(gap, floor), "best_reachable": 1.3862943611}))


if __name__ == "__main__":
    main()
