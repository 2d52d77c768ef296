"""Dynamic loss scaling shared by all pipeline stages (fp16 runs).

The scale is a plain Python number, identical on every rank. Each stage checks its own gradients for
inf/nan on the device; ``agree`` takes the MAX of the flags over the group (one tiny all-reduce and the
step's only host read), so either every stage steps or none does. Growth x2 after 2000 clean steps,
back-off x0.5 on overflow, never below 1. Reference: src/kohakuwupipe/training/scaler.py:13-98.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


class PipelineGradScaler:
    def __init__(self, init_scale: float = 2.0 ** 16, growth_factor: float = 2.0, backoff_factor: float = 0.5,
                 growth_interval: int = 2000, min_scale: float = 1.0, enabled: bool = True):
        self.scale = float(init_scale)
        self.growth_factor, self.backoff_factor = growth_factor, backoff_factor
        self.growth_interval, self.min_scale = growth_interval, min_scale
        self.enabled = enabled
        self._clean_steps = 0
        self._found_inf: torch.Tensor | None = None

    def scale_loss(self, loss: torch.Tensor) -> torch.Tensor:
        return loss * self.scale if self.enabled else loss

    @torch.no_grad()
    def unscale_(self, grads) -> None:
        """Divide gradients by the scale and record (on the device) whether any is non-finite."""
        grads = [g for g in grads if g is not None]
        if not self.enabled or not grads:
            self._found_inf = None
            return
        inv = 1.0 / self.scale
        flag = torch.zeros(1, dtype=torch.float32, device=grads[0].device)
        for g in grads:
            g.mul_(inv)
            flag += (~torch.isfinite(g)).any().float()
        self._found_inf = flag.clamp_(max=1.0)

    def agree(self, group=None) -> bool:
        """True when some stage overflowed (collective: every rank must call it)."""
        if not self.enabled:
            return False
        flag = self._found_inf if self._found_inf is not None else torch.zeros(1)
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
            if dist.get_backend(group) == "nccl" and not flag.is_cuda:
                flag = flag.cuda()
            dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=group)
        return bool(flag.item() > 0)

    def update(self, overflow: bool) -> None:
        if not self.enabled:
            return
        if overflow:
            self.scale = max(self.scale * self.backoff_factor, self.min_scale)
            self._clean_steps = 0
        else:
            self._clean_steps += 1
            if self._clean_steps >= self.growth_interval:
                self.scale *= self.growth_factor
                self._clean_steps = 0

    def state_dict(self) -> dict:
        return {"scale": self.scale, "clean_steps": self._clean_steps}

    def load_state_dict(self, sd: dict) -> None:
        self.scale = float(sd["scale"])
        self._clean_steps = int(sd.get("clean_steps", 0))
