"""Process-group set-up for pipeline runs.

``init_pipeline`` reads ``RANK`` / ``WORLD_SIZE`` / ``LOCAL_RANK`` (torchrun conventions), selects the
CUDA device and initialises the default group LAZILY (no ``device_id``), so NCCL builds a 2-rank
communicator per send/recv pair instead of one eager world communicator. ``backend="gloo"`` runs the same
code on CPU. Reference: src/kohakuwupipe/parallel/distributed.py:17-83.
"""

from __future__ import annotations

import datetime
import os
import warnings
from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class PipelineRanks:
    rank: int
    world_size: int
    local_rank: int
    device: torch.device

    @property
    def is_first(self) -> bool:
        return self.rank == 0

    @property
    def is_last(self) -> bool:
        return self.rank == self.world_size - 1


def eager_init_in_use() -> bool:
    """True when the default group was created with a bound device (eager NCCL initialisation)."""
    if not dist.is_initialized():
        return False
    pg = dist.distributed_c10d._get_default_group()
    return getattr(pg, "bound_device_id", None) is not None


def warn_on_eager_init() -> None:
    if eager_init_in_use():
        warnings.warn("the default process group was initialised eagerly (device_id given): P2P-only "
                      "pipelines then pay for a world communicator they never use", stacklevel=2)


def init_pipeline(backend: str | None = None, timeout: float = 1800.0) -> PipelineRanks:
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    use_cuda = torch.cuda.is_available() and backend != "gloo"
    if use_cuda:
        torch.cuda.set_device(local)
        device = torch.device("cuda", local)
    else:
        device = torch.device("cpu")
    if not dist.is_initialized() and world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        dist.init_process_group(backend or ("nccl" if use_cuda else "gloo"), rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout))
    warn_on_eager_init()
    return PipelineRanks(rank, world, local, device)


def shutdown() -> None:
    if dist.is_initialized():
        try:
            dist.barrier()
        finally:
            dist.destroy_process_group()
