"""``StochasticAdamW``: AdamW for 16-bit parameters with fp32 (or bf16) state and a choice of write-back:
``stochastic`` rounding (unbiased), ``kahan`` (a bf16 compensation buffer carries the rounding error) or
``nearest``. Has its own global-norm clip. Reference: src/kohakuwullm/training/optim/lowbit.py:62-218."""

from __future__ import annotations

import torch

from kohakuwullm_b200.ops.optim import sr_update_


class StochasticAdamW(torch.optim.Optimizer):
    def __init__(self, params, lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, rounding: str = "stochastic",
                 state_dtype: torch.dtype = torch.float32, max_grad_norm: float | None = None, seed: int = 0):
        if rounding not in ("stochastic", "kahan", "nearest"):
            raise ValueError(f"unknown rounding {rounding!r}")
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self.rounding, self.state_dtype, self.max_grad_norm, self.seed, self._step = rounding, state_dtype, max_grad_norm, seed, 0

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        self._step += 1
        grads = [p.grad for g in self.param_groups for p in g["params"] if p.grad is not None]
        scale = None
        if self.max_grad_norm and grads:
            norm = torch.stack([g.float().pow(2).sum() for g in grads]).sum().sqrt()
            scale = torch.clamp(self.max_grad_norm / (norm + 1e-6), max=1.0)
        offset = 0
        for group in self.param_groups:
            b1, b2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p, dtype=self.state_dtype)
                    st["exp_avg_sq"] = torch.zeros_like(p, dtype=self.state_dtype)
                    if self.rounding == "kahan":
                        st["comp"] = torch.zeros_like(p)
                st["step"] += 1
                g = p.grad.float() if scale is None else p.grad.float() * scale
                m = st["exp_avg"].float().mul_(b1).add_(g, alpha=1 - b1)
                v = st["exp_avg_sq"].float().mul_(b2).addcmul_(g, g, value=1 - b2)
                st["exp_avg"].copy_(m)
                st["exp_avg_sq"].copy_(v)
                bc1, bc2 = 1 - b1 ** st["step"], 1 - b2 ** st["step"]
                update = (m / bc1) / ((v / bc2).sqrt() + group["eps"])
                decay = group["lr"] * group["weight_decay"]
                if self.rounding == "stochastic" and p.dtype == torch.bfloat16:
                    sr_update_(p, update.contiguous(), decay, -group["lr"], seed=self.seed + self._step, offset=offset)
                elif self.rounding == "kahan" and p.dtype != torch.float32:
                    target = p.float() * (1 - decay) - group["lr"] * update + st["comp"].float()
                    new = target.to(p.dtype)
                    st["comp"].copy_((target - new.float()).to(p.dtype))
                    p.copy_(new)
                else:
                    p.copy_((p.float() * (1 - decay) - group["lr"] * update).to(p.dtype))
                offset += p.numel()
        return loss
