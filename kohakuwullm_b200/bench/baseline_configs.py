"""The benchmark configurations this framework is measured on, as one command each.

    python -m kohakuwullm_b200.bench.baseline_configs --config 3                       # 1 GPU
    torchrun --nproc-per-node 8 -m kohakuwullm_b200.bench.baseline_configs --config 4  # 8 GPUs

Every configuration runs ``kohakuwullm_b200.bench.step_throughput`` (synthetic packed batches, random
initialisation, device-timed, max over ranks, one JSON line from rank 0) with the arguments below:

  2  dense 546M, MXFP8 linears, data parallel, 4096-token packs x 4 accumulation (what ``bench.py`` measures too)
  3  MoE 991M under pipeline parallelism: measured stage split, 1F1B, 16 micro-batches of 4096 tokens
  4  MoE 991M, expert parallel + data parallel, 8192-token packs, routers skewed by a seeded N(0, 0.5) bias
     (receive capacity 5x the mean: with 8 ranks the busiest rank of a layer gets up to ~4x the mean under this skew)
  5  sliding-window 1.1B (window 1024 on 3 of 4 layers, 4 sinks, YaRN x4), 16384-token packs with log-uniform
     documents, MXFP8 attention operands, data parallel
"""

from __future__ import annotations

import argparse
import sys

CONFIGS = {
    2: ["--preset", "B200-dense-546M", "--micro-tokens", "4096", "--accum", "4", "--len-min", "64", "--len-max", "4096"],
    3: ["--preset", "B200-moe-991M", "--micro-tokens", "4096", "--accum", "16", "--len-min", "64", "--len-max", "4096",
        "--pipeline", "--schedule", "1f1b"],
    4: ["--preset", "B200-moe-991M", "--micro-tokens", "8192", "--accum", "4", "--len-min", "64", "--len-max", "4096",
        "--expert-parallel", "--router-bias-std", "0.5", "--ep-capacity", "5.0"],
    5: ["--preset", "B200-sliding-1B", "--micro-tokens", "16384", "--accum", "1", "--len-min", "128", "--len-max", "16384",
        "--log-uniform", "--set", "attn='mxfp8'"],
}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", type=int, required=True, choices=sorted(CONFIGS))
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    args, extra = ap.parse_known_args(argv)
    from kohakuwullm_b200.bench import step_throughput

    step_throughput.main([*CONFIGS[args.config], "--steps", str(args.steps), "--warmup", str(args.warmup), *extra])
    return 0


if __name__ == "__main__":
    sys.exit(main())
