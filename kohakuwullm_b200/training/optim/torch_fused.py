"""``FusedAdamW`` with the ``torch.optim`` interface (parameter groups, ``step()``, ``state_dict()``).

Parameters must be fp32 (bf16-mixed training: autocast compute over fp32 parameters); state can be kept
in bf16 (``state_dtype``). All tensors of a step share one global-norm clip: the squared norms are summed
on the device (optionally all-reduced for sharded models) and enter the update as a device scalar, so
clipping costs no host synchronisation. The flat-buffer whole-model variant used by ``TrainEngine`` is
``FlatAdamW``. Reference: src/kohakuwullm/training/optim/fused_adamw.py:7-172.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


class FusedAdamW(torch.optim.Optimizer):
    def __init__(self, params, lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, max_grad_norm: float | None = None,
                 reduce_norm_group=None, state_dtype: torch.dtype = torch.float32):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self.max_grad_norm, self.reduce_norm_group, self.state_dtype = max_grad_norm, reduce_norm_group, state_dtype

    def _clip_scale(self, grads) -> torch.Tensor | None:
        if not self.max_grad_norm or not grads:
            return None
        sq = torch.stack([g.float().pow(2).sum() for g in grads]).sum()
        if self.reduce_norm_group is not None and dist.is_initialized():
            dist.all_reduce(sq, group=self.reduce_norm_group)
        return torch.clamp(self.max_grad_norm / (sq.sqrt() + 1e-6), max=1.0)

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        all_grads = [p.grad for g in self.param_groups for p in g["params"] if p.grad is not None]
        scale = self._clip_scale(all_grads)
        for group in self.param_groups:
            b1, b2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                if p.dtype != torch.float32:
                    raise ValueError(f"FusedAdamW needs float32 parameters, got {p.dtype}; use adamw16 or "
                                     "stochastic_adamw for 16-bit parameters")
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p, dtype=self.state_dtype)
                    st["exp_avg_sq"] = torch.zeros_like(p, dtype=self.state_dtype)
                st["step"] += 1
                g = p.grad.float()
                if scale is not None:
                    g = g * scale
                m = st["exp_avg"].float().mul_(b1).add_(g, alpha=1 - b1)
                v = st["exp_avg_sq"].float().mul_(b2).addcmul_(g, g, value=1 - b2)
                bc1, bc2 = 1 - b1 ** st["step"], 1 - b2 ** st["step"]
                p.mul_(1 - group["lr"] * group["weight_decay"])
                p.addcdiv_(m, (v / bc2).sqrt_().add_(group["eps"]), value=-group["lr"] / bc1)
                st["exp_avg"].copy_(m)
                st["exp_avg_sq"].copy_(v)
        return loss
