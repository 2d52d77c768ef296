"""Data-parallel gradient synchronisation over flat fp32 gradient buffers.

``GradSync`` is the NCCL (or gloo, on CPU) baseline: the flat ``main_grad`` buffers are summed across
the data-parallel group in large contiguous buckets on a side stream. Gradients are SUMS of per-token
losses; the division by the global trained-token count happens inside the optimizer kernel through a
device scalar, which is what makes accumulation token-exact across micro-batches and ranks without a
host round trip. The fused reduce-scatter + AdamW + all-gather kernel over NVLink peer memory
(``kohakuwullm_b200.parallel.fused_ddp``) plugs into the same interface.
Reference behaviour: torch DDP bucketed all-reduce configured at scripts/train/lm.py:383-398, with
``no_sync`` on all but the last micro-batch (scripts/bench/e2e/step_throughput.py:137-159).
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from kohakuwullm_b200.parallel.flat import FlatParameters


class GradSync:
    def __init__(self, flat: FlatParameters, group=None, bucket_elems: int = 64 * 1024 * 1024):
        self.flat, self.group = flat, group
        self.bucket_elems = bucket_elems
        self.world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1

    def reduce(self) -> None:
        """Sum every gradient buffer over the group (in place)."""
        if self.world <= 1:
            return
        for key in self.flat.replicated_keys():
            buf = self.flat.groups[key].main_grad
            n = buf.numel()
            for s in range(0, n, self.bucket_elems):
                dist.all_reduce(buf[s:min(n, s + self.bucket_elems)], group=self.group)

    def all_reduce_scalar(self, t: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            dist.all_reduce(t, group=self.group)
        return t
