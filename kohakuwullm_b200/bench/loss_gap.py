"""Loss-gap A/B run: train the same model with bf16 linears and with MXFP8 linears on a learnable synthetic
stream and compare the final-window loss against a replicate noise floor.

    python -m kohakuwullm_b200.bench.loss_gap --preset B200-dense-546M --depth 8 --steps 200

Data: a noisy affine token chain ``x[t+1] = (31 x[t] + 7 + e) mod V`` with ``e`` uniform in {0,1,2,3}, so the
best reachable loss is ln 4 and the curve is informative (uniform random tokens would pin every arm to ln V).
Arms: ``bf16`` with init seeds s .. s + R - 1 (R = ``--replicates``; with R = 1 one extra bf16 run with seed
s + 1 gives the run-to-run floor) and ``mxfp8`` with the same seeds, all on the same data. Prints one JSON
line with the final-window means of every run, the gap between the arm means, the floor (largest gap between
two bf16 replicates) and the verdict of ``abtest.admissible``. Reference method: docs/performance/ab-testing.md of the reference
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
            cur = int(torch.randint(0, vocab, (1,), generator=g))
            noise = torch.randint(0, 4, (n,), generator=g).tolist()
            x = [cur] * n
            for t in range(1, n):           # plain ints: a tensor element access per token is 50x slower
                cur = (31 * cur + 7 + noise[t]) % vocab
                x[t] = cur
            docs.append(torch.tensor(x, dtype=torch.long))
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
    ap.add_argument("--replicates", type=int, default=1, help="runs per arm (different init seeds)")
    args = ap.parse_args()
    data = [[p.to("cuda") for p in chain_packs(args.accum, args.micro_tokens, 64, 1024, args.vocab, args.seed * 1000 + i)]
            for i in range(args.batches)]
    import statistics

    reps = max(args.replicates, 1)
    bf16 = [run_arm(args, False, args.seed + r, data) for r in range(max(reps, 2))]   # two at least: the floor
    mx = [run_arm(args, True, args.seed + r, data) for r in range(reps)]
    w = args.window
    bf16_finals = [abtest.final_window_mean(r, w) for r in bf16]
    mx_finals = [abtest.final_window_mean(r, w) for r in mx]
    gap = statistics.fmean(mx_finals) - statistics.fmean(bf16_finals[:reps])
    floor = abtest.noise_floor(bf16, w)
    print(json.dumps({"preset": args.preset, "depth": args.depth, "steps": args.steps, "window": w,
                      "replicates": reps, "bf16_finals": bf16_finals, "mxfp8_finals": mx_finals,
                      "mxfp8_floor": abtest.noise_floor(mx, w), "first_loss": bf16[0][0],
                      "gap_mxfp8_minus_bf16": gap, "replicate_floor": floor,
                      "windowed_gaps": abtest.windowed_gaps(bf16[0], mx[0], w)[-5:],
                      "within_noise": abtest.admissible(gap, floor), "best_reachable": 1.3862943611}))

if __name__ == "__main__":
    main()
