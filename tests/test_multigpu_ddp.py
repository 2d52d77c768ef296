"""Fused reduce-scatter + AdamW + all-gather kernels (NVLink peer memory) against the NCCL all-reduce +
unsharded AdamW path, on 2 or more GPUs. Also the bounded-wait path on one GPU: a flag that nothing
sets makes the kernel give up and report a time-out instead of hanging."""

import ctypes
import os
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests.helpers import free_port


def _worker(rank, world, port, mode, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from kohakuwullm_b200.data.synthetic import make_packs
    from kohakuwullm_b200.models import LMBackbone, get_preset
    from kohakuwullm_b200.ops import native
    from kohakuwullm_b200.training.engine import TrainEngine

    torch.manual_seed(7)
    cfg = get_preset("B200-dense-546M", depth=2, vocab_size=4096, mxfp8=False)
    with torch.device("cuda", rank):
        model = LMBackbone(cfg)
    eng = TrainEngine(model, lr=1e-3, param_dtype=torch.bfloat16, grad_sync=mode, cuda_graphs=False)
    packs = make_packs(2, 1024, 64, 512, cfg.vocab_size, seed=100 + rank)
    outs = [eng.step(packs) for _ in range(3)]
    torch.cuda.synchronize()
    native.check_status()
    flat = torch.cat([g.data.float().reshape(-1) for g in eng.flat.groups.values()]).cpu()
    torch.save({"loss": [float(o["loss"]) for o in outs], "norm": [float(o["grad_norm"]) for o in outs],
                "flat": flat}, os.path.join(out_dir, f"{mode}_{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.multigpu
@pytest.mark.timeout(600)
def test_fused_ddp_matches_nccl_path():
    world = min(torch.cuda.device_count(), 4)
    with tempfile.TemporaryDirectory() as tmp:
        for mode in ("nccl", "fused"):
            mp.spawn(_worker, args=(world, free_port(), mode, tmp), nprocs=world, join=True)
        ref = torch.load(os.path.join(tmp, "nccl_0.pt"))
        for r in range(world):
            got = torch.load(os.path.join(tmp, f"fused_{r}.pt"))
            for a, b in zip(got["loss"], ref["loss"]):
                assert abs(a - b) < 2e-3, (got["loss"], ref["loss"])
            for a, b in zip(got["norm"], ref["norm"]):
                assert abs(a - b) < 1e-2 * max(b, 1e-6), (got["norm"], ref["norm"])
            # every rank holds the same parameters, equal to the NCCL path up to bf16 rounding of one step
            diff = (got["flat"] - ref["flat"]).abs().max().item()
            assert diff < 2e-2, f"rank {r}: parameters differ by {diff}"
            same = torch.load(os.path.join(tmp, "fused_0.pt"))["flat"]
            assert torch.equal(got["flat"], same), f"rank {r} diverged from rank 0"


@pytest.mark.gpu
def test_flag_wait_times_out_and_reports():
    """A peer that never arrives: the wait gives up after its limit and sets the status word."""
    from kohakuwullm_b200.ops import native

    L = native.require()
    flags = torch.zeros(24, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    result = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    rc = L.kwu_ddp_wait_probe(ctypes.c_void_p(flags.data_ptr()), ctypes.c_int(2), ctypes.c_int(1),
                              ctypes.c_void_p(status.data_ptr()), ctypes.c_longlong(2_000_000),
                              ctypes.c_void_p(result.data_ptr()), native.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    assert int(result.item()) == 0
    assert int(status.item()) == 5  # KWU_ERR_TIMEOUT_FLAG
    # and the context is still usable
    assert float(torch.ones(4, device="cuda").sum()) == 4.0
