"""Multi-process checks of the pipeline engine, each ending in a PASS / FAIL line (exit code 0 / 1). Run under
``torch.distributed.run`` on GPUs (NCCL) or CPUs (``--backend gloo``):

    torchrun --nproc-per-node 2 -m kohakuwullm_b200.cli.dist_checks checkpoint
    torchrun --nproc-per-node 2 -m kohakuwullm_b200.cli.dist_checks generate
    torchrun --nproc-per-node 2 -m kohakuwullm_b200.cli.dist_checks gen-resume
    torchrun --nproc-per-node 4 -m kohakuwullm_b200.cli.dist_checks link-bench
    torchrun --nproc-per-node 2 -m kohakuwullm_b200.cli.dist_checks trainer-smoke
    torchrun --nproc-per-node 2 -m kohakuwullm_b200.cli.dist_checks generate-bench --rows 8 --microbatches 4

checkpoint   train under one stage split, save, load under ANOTHER split in a new trainer and compare the next
             step's loss with the uninterrupted run (weights and optimizer state are keyed by whole-model name).
generate     pipelined greedy decode equals the single-process decode of the same weights token for token
             (wide initialisation, so that the comparison can fail).
gen-resume   a few training steps, decode, checkpoint, reload into a fresh trainer, decode again: same tokens.
link-bench   cost of one hop between neighbouring ranks for boundary sizes from 4 KB to 128 MB.
trainer-smoke  the schedules named in ``--schedules`` (default: GPipe, 1F1B and, through the torch-pipelining
             adapter, interleaved 1F1B and looped BFS) build, take three steps on one batch and give finite losses
             that fall; all of them must give the SAME losses.
generate-bench  milliseconds per decoded token of the pipelined decode, with and without micro-batches
             (the tokens must be the same either way).
Reference: scripts/dist/{pp_checkpoint_smoke,pp_generate_equivalence,uwupipe_gen_resume,pp_link_bench,pp_trainer_smoke,
pp_torch_smoke,pp_generate_smoke,pp_generate_bench}.py.
"""

from __future__ import annotations

import argparse
import faulthandler
import json
import os
import sys
import tempfile

import torch
import torch.distributed as dist

CFG = dict(vocab_size=512, dim=128, depth=4, heads=2, kv_heads=1, head_dim=64, mlp_hidden=256)


def _setup(backend: str | None):
    from kohakuwullm_b200.pipe import init_pipeline

    faulthandler.dump_traceback_later(600, exit=True)   # a check that hangs ends with every thread's stack
    return init_pipeline(backend)


def _trainer(cfg, ranks, layers, lr=1e-2, micro_tokens=64, n_micro=4, dtype=None):
    from kohakuwullm_b200.pipe.trainer import PipelineTrainer
    from kohakuwullm_b200.training.parallel.pipeline import plan_for
    from kohakuwullm_b200.training.parallel.uwupipe import LMPipelineModule

    if dtype is None and ranks.device.type == "cuda":
        dtype = torch.bfloat16          # the native kernels (and the captured stages) run on 16-bit parameters
    module = LMPipelineModule(cfg, micro_tokens=micro_tokens, lr=lr, param_dtype=dtype)
    plans = plan_for(cfg, ranks.world_size, layers=layers)
    return PipelineTrainer(module, plans, rank=ranks.rank, world=ranks.world_size, device=ranks.device,
                           n_micro=n_micro, schedule="1f1b")


def _batch(cfg, step, micro_tokens=64, n_micro=4):
    from kohakuwullm_b200.data.synthetic import make_packs

    return make_packs(n_micro, micro_tokens, 8, 32, cfg.vocab_size, seed=100 + step)


def _splits(depth: int, world: int):
    """Two different contiguous splits of ``depth`` layers over ``world`` stages."""
    base = [depth // world] * world
    base[0] += depth - sum(base)
    other = list(reversed(base))
    if other == base:
        if world > 1 and base[0] > 1:
            other = base.copy()
            other[0] -= 1
            other[-1] += 1
    return base, other


def _finish(ok: bool, detail: dict, ranks) -> int:
    flag = torch.tensor([int(ok)], device=ranks.device)
    if ranks.world_size > 1:
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    ok = bool(flag.item())
    if ranks.rank == 0:
        print(json.dumps(detail))
        print("PASS" if ok else "FAIL")
    from kohakuwullm_b200.pipe import shutdown

    shutdown()
    return 0 if ok else 1


def check_checkpoint(args) -> int:
    from kohakuwullm_b200.models import get_preset

    ranks = _setup(args.backend)
    cfg = get_preset("B200-smoke", **CFG, mxfp8=False)
    first, second = _splits(cfg.depth, ranks.world_size)
    tmp = [tempfile.mkdtemp(prefix="kwu_ckpt_") if ranks.rank == 0 else None]
    if ranks.world_size > 1:
        dist.broadcast_object_list(tmp, src=0)
    path = os.path.join(tmp[0], "a.ckpt")
    a = _trainer(cfg, ranks, first)
    for s in range(2):
        a.loop.step(_batch(cfg, s))
    a.save_checkpoint(path)
    want = float(a.loop.step(_batch(cfg, 2)).loss)
    b = _trainer(cfg, ranks, second)
    b.load_checkpoint(path)
    got = float(b.loop.step(_batch(cfg, 2)).loss)
    tol = args.tol if ranks.device.type == "cpu" else max(args.tol, 2e-2)   # bf16 weights, fp32 atomics in the gradients
    return _finish(abs(got - want) < tol, {"check": "checkpoint", "splits": [first, second], "uninterrupted": want,
                                                "resumed_under_other_split": got}, ranks)


def _decode(trainer, ranks, prompt, n):
    from kohakuwullm_b200.generation.engine import PipelineGenerator

    stage = trainer.module.stages[0]
    return PipelineGenerator(stage, ranks.rank, ranks.world_size, eos_id=-1).generate(prompt.to(ranks.device), n, temperature=0.0)


def check_generate(args) -> int:
    from kohakuwullm_b200.generation.engine import LocalGenerator
    from kohakuwullm_b200.models import LMBackbone, get_preset

    ranks = _setup(args.backend)
    cfg = get_preset("B200-smoke", **CFG, mxfp8=False, init_std=0.3)   # wide init: greedy decoding is not degenerate
    first, _ = _splits(cfg.depth, ranks.world_size)
    tr = _trainer(cfg, ranks, first)
    prompt = torch.tensor([[5, 17, 33, 2, 90, 41], [7, 7, 150, 12, 3, 64]])
    got = _decode(tr, ranks, prompt, 16).cpu()
    torch.manual_seed(1234)                                           # the module's seed: the same whole model
    model = LMBackbone(cfg).to(ranks.device)
    if ranks.device.type == "cuda":
        from kohakuwullm_b200.training.optim.lowbit import cast_parameters_

        cast_parameters_(model, torch.bfloat16)
    want = LocalGenerator(model, eos_id=-1).generate(prompt.to(ranks.device), 16, temperature=0.0).cpu()
    new = want[:, prompt.shape[1]:]
    can_fail = (not torch.equal(new[0], new[1])) and new[0].unique().numel() > 2
    return _finish(bool(torch.equal(got, want)) and can_fail,
                   {"check": "generate", "equal": bool(torch.equal(got, want)), "comparison_can_fail": bool(can_fail),
                    "tokens": got[0].tolist()}, ranks)


def check_gen_resume(args) -> int:
    from kohakuwullm_b200.models import get_preset

    ranks = _setup(args.backend)
    cfg = get_preset("B200-smoke", **CFG, mxfp8=False, init_std=0.3)
    first, second = _splits(cfg.depth, ranks.world_size)
    tmp = [tempfile.mkdtemp(prefix="kwu_gen_") if ranks.rank == 0 else None]
    if ranks.world_size > 1:
        dist.broadcast_object_list(tmp, src=0)
    path = os.path.join(tmp[0], "g.ckpt")
    a = _trainer(cfg, ranks, first, lr=1e-3)
    for s in range(3):
        a.loop.step(_batch(cfg, s))
    prompt = torch.tensor([[5, 17, 33, 2, 90, 41]])
    before = _decode(a, ranks, prompt, 12).cpu()
    a.save_checkpoint(path)
    b = _trainer(cfg, ranks, second, lr=1e-3)
    b.load_checkpoint(path)
    after = _decode(b, ranks, prompt, 12).cpu()
    return _finish(bool(torch.equal(before, after)), {"check": "gen-resume", "before": before[0].tolist(),
                                                      "after": after[0].tolist()}, ranks)


def check_link_bench(args) -> int:
    from kohakuwullm_b200.pipe.latency import hop_cost, roofline

    ranks = _setup(args.backend)
    rows = []
    size = 4096
    while size <= args.max_bytes:
        r = hop_cost(size, ranks.device, repeats=args.repeats)
        r["roofline_s"] = roofline(size)
        rows.append(r)
        size *= 8
    return _finish(all(r["seconds"] > 0 for r in rows), {"check": "link-bench", "world": ranks.world_size, "hops": rows}, ranks)


def check_trainer_smoke(args) -> int:
    import math

    from kohakuwullm_b200.models import get_preset
    from kohakuwullm_b200.pipe.trainer import PipelineTrainer
    from kohakuwullm_b200.training.parallel.pipeline import plan_for
    from kohakuwullm_b200.training.parallel.uwupipe import LMPipelineModule

    ranks = _setup(args.backend)
    cfg = get_preset("B200-smoke", **{**CFG, "depth": 2 * max(ranks.world_size, 2)}, mxfp8=False)
    dtype = torch.bfloat16 if ranks.device.type == "cuda" else None
    report, ok = {}, True
    for schedule in args.schedules.split(","):
        chunks = 1 if schedule in ("gpipe", "1f1b") else 2
        try:
            module = LMPipelineModule(cfg, micro_tokens=64, lr=3e-3, param_dtype=dtype)
            plans = plan_for(cfg, ranks.world_size * chunks, style="v" if schedule in ("zbv", "dualpipe-v") else "loop")
            tr = PipelineTrainer(module, plans, rank=ranks.rank, world=ranks.world_size, device=ranks.device,
                                 n_micro=4, schedule=schedule)
            losses = [float(tr.loop.step(_batch(cfg, 0)).loss) for _ in range(3)]   # the same batch: it must fall
            fine = all(math.isfinite(x) for x in losses) and min(losses[1:]) < losses[0]
            report[schedule] = {"losses": losses, "ok": fine}
            ok = ok and fine
        except (RuntimeError, NotImplementedError, ValueError, AttributeError) as e:   # what torch's runtime refuses
            if schedule in ("gpipe", "1f1b", "interleaved-1f1b", "looped-bfs"):
                report[schedule] = {"ok": False, "error": f"{type(e).__name__}: {e}"[:300]}
                ok = False
            else:
                report[schedule] = {"skipped": f"{type(e).__name__}: {e}"[:300]}
    firsts = [r["losses"] for r in report.values() if "losses" in r]
    same = all(max(abs(a - b) for a, b in zip(x, firsts[0])) < 1e-3 for x in firsts) if firsts else False
    return _finish(ok and same, {"check": "trainer-smoke", "same_losses_across_schedules": same, "schedules": report}, ranks)


def check_generate_bench(args) -> int:
    import time

    from kohakuwullm_b200.generation.engine import PipelineGenerator
    from kohakuwullm_b200.models import get_preset

    ranks = _setup(args.backend)
    cfg = get_preset("B200-smoke", **CFG, mxfp8=False, init_std=0.3)
    first, _ = _splits(cfg.depth, ranks.world_size)
    tr = _trainer(cfg, ranks, first)
    stage = tr.module.stages[0]
    g = torch.Generator().manual_seed(3)
    prompt = torch.randint(1, cfg.vocab_size, (args.rows, 16), generator=g).to(ranks.device)
    rows = {}
    tokens = {}
    for m in sorted({1, args.microbatches}):
        gen = PipelineGenerator(stage, ranks.rank, ranks.world_size, eos_id=-1, microbatches=m)
        gen.generate(prompt, 4, temperature=0.0)                          # warm-up
        if ranks.device.type == "cuda":
            torch.cuda.synchronize()
        if ranks.world_size > 1:
            dist.barrier()
        t0 = time.perf_counter()
        tokens[m] = gen.generate(prompt, args.new_tokens, temperature=0.0).cpu()
        if ranks.device.type == "cuda":
            torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        rows[m] = {"ms_per_token": 1e3 * dt / args.new_tokens, "tokens_per_s": args.rows * args.new_tokens / dt}
    same = all(torch.equal(tokens[m], tokens[1]) for m in tokens)
    return _finish(same, {"check": "generate-bench", "rows": args.rows, "new_tokens": args.new_tokens,
                          "by_microbatches": rows, "same_tokens": same}, ranks)


CHECKS = {"trainer-smoke": check_trainer_smoke, "generate-bench": check_generate_bench, "checkpoint": check_checkpoint, "generate": check_generate, "gen-resume": check_gen_resume,
          "link-bench": check_link_bench}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("check", choices=sorted(CHECKS))
    ap.add_argument("--backend", default=None, help="gloo runs the check on CPUs")
    ap.add_argument("--tol", type=float, default=2e-3)
    ap.add_argument("--max-bytes", type=int, default=128 << 20)
    ap.add_argument("--repeats", type=int, default=10)
    ap.add_argument("--schedules", default="gpipe,1f1b,interleaved-1f1b,looped-bfs",
                    help="comma list; interleaved-zb / zbv / dualpipe-v can be named, but torch 2.11's runtime fails on them "
                         "with custom autograd functions (and on gloo a V placement sends to itself): a rank that raises "
                         "while its neighbour waits ends the check through the watchdog, not with a report")
    ap.add_argument("--rows", type=int, default=8)
    ap.add_argument("--microbatches", type=int, default=4)
    ap.add_argument("--new-tokens", type=int, default=32)
    args = ap.parse_args(argv)
    return CHECKS[args.check](args)


if __name__ == "__main__":
    sys.exit(main())
