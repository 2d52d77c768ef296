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


COMPRESS = {None: None, "": None, "none": None, "bf16": torch.bfloat16, "fp16": torch.float16}


class GradSync:
    """``compress="bf16" | "fp16"``: the buckets cross the wire in that dtype (half the bytes; the role of torch DDP's
    ``bf16_compress_hook`` / ``fp16_compress_hook`` in the reference). The local fp32 sums are rounded once before
    the reduction, the reduction itself adds in the wire dtype, and the result is widened back into the fp32 buffer;
    fp16 buckets are divided by the group size before the cast and multiplied back after it, so that the sum of
    ``world`` near-maximal gradients cannot overflow the format."""

    def __init__(self, flat: FlatParameters, group=None, bucket_elems: int = 64 * 1024 * 1024,
                 compress: str | None = None):
        if compress not in COMPRESS:
            raise ValueError(f"unknown gradient compression {compress!r}; known: bf16, fp16, none")
        self.flat, self.group = flat, group
        self.bucket_elems = bucket_elems
        self.wire_dtype = COMPRESS[compress]
        self.world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
        self._wire: torch.Tensor | None = None      # one reusable bucket in the wire dtype

    def _wire_bucket(self, like: torch.Tensor, n: int) -> torch.Tensor:
        if self._wire is None or self._wire.numel() < n or self._wire.device != like.device:
            self._wire = torch.empty(n, dtype=self.wire_dtype, device=like.device)   # a part never exceeds a bucket
        return self._wire[:n]

    def reduce(self) -> None:
        """Sum every gradient buffer over the group (in place)."""
        if self.world <= 1:
            return
        for key in self.flat.replicated_keys():
            buf = self.flat.groups[key].main_grad
            n = buf.numel()
            for s in range(0, n, self.bucket_elems):
                part = buf[s:min(n, s + self.bucket_elems)]
                if self.wire_dtype is None:
                    dist.all_reduce(part, group=self.group)
                    continue
                wire = self._wire_bucket(part, part.numel())
                if self.wire_dtype == torch.float16:
                    torch.mul(part, 1.0 / self.world, out=part)
                wire.copy_(part)
                dist.all_reduce(wire, group=self.group)
                part.copy_(wire)
                if self.wire_dtype == torch.float16:
                    part.mul_(float(self.world))

    def all_reduce_scalar(self, t: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            dist.all_reduce(t, group=self.group)
        return t
