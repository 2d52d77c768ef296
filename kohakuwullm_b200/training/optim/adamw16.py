"""``AdamW16``: AdamW whose state lives in the parameter dtype (bf16): first moment and the SQUARE ROOT of
the second moment (which keeps its dynamic range inside bf16), fp32 math in registers, optional stochastic
rounding of the written-back parameter and momentum. One kernel per tensor (``csrc/optim16.cu``).
Reference: src/kohakuwullm/training/optim/adamw16.py:14-95."""

from __future__ import annotations

import torch

from kohakuwullm_b200.ops.optim import adamw16_step_


class AdamW16(torch.optim.Optimizer):
    def __init__(self, params, lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, rounding: str = "nearest",
                 seed: int = 0):
        if rounding not in ("nearest", "stochastic"):
            raise ValueError(f"rounding must be 'nearest' or 'stochastic', got {rounding!r}")
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self.rounding, self.seed, self._step = rounding, seed, 0

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        self._step += 1
        offset = 0
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p)
                    st["exp_avg_sqrt"] = torch.zeros_like(p)
                st["step"] += 1
                # the seed advances with the step and is the same on every data-parallel replica
                adamw16_step_(p, st["exp_avg"], st["exp_avg_sqrt"], p.grad, lr=group["lr"], betas=group["betas"],
                              eps=group["eps"], wd=group["weight_decay"], step=st["step"],
                              stochastic=self.rounding == "stochastic", seed=self.seed + self._step, offset=offset)
                offset += 2 * p.numel()
        return loss
