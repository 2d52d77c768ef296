"""``MuonW``: Muon (momentum + Newton-Schulz orthogonalisation) for hidden matrices, AdamW for the rest.

The orthogonalisation runs in bf16 on the tcgen05 GEMM without any transposes: with ``X`` (n, m), n <= m,
``A = X X^T`` is ``matmul(X, X)`` (both operands K-major), ``A A`` is ``matmul(A, A)`` (A is symmetric) and
``B X`` is ``matmul(B, X, b_mn=True)``. Five quintic iterations ``X <- a X + (b A + c A A) X`` with the
coefficients (3.4445, -4.7750, 2.0315); matrices of equal shape are processed as one stacked batch.
Update scale ``spectral``: ``sqrt(max(1, rows/cols))``; ``rms``: ``0.2 * sqrt(max(rows, cols))``.
Reference: src/kohakuwullm/training/optim/muon.py:20-442.
"""

from __future__ import annotations

import torch

from kohakuwullm_b200.ops.gemm import matmul

NS_COEFFS = (3.4445, -4.7750, 2.0315)


def newton_schulz(G: torch.Tensor, steps: int = 5, eps: float = 1e-7) -> torch.Tensor:
    """Approximate orthogonalisation of a 2-D matrix (returns the dtype of the input)."""
    a, b, c = NS_COEFFS
    X = G.to(torch.bfloat16) if G.is_cuda else G.float()
    transposed = X.shape[0] > X.shape[1]
    if transposed:
        X = X.t().contiguous()
    X = X / (X.float().norm() + eps).to(X.dtype)
    for _ in range(steps):
        A = matmul(X, X)                       # X X^T
        B = matmul(A, A)                       # A A (A symmetric)
        B = (b * A.float() + c * B.float()).to(X.dtype)
        X = (a * X.float() + matmul(B, X, b_mn=True).float()).to(X.dtype)
    if transposed:
        X = X.t().contiguous()
    return X.to(G.dtype)


class MuonW(torch.optim.Optimizer):
    def __init__(self, hidden_params, adam_groups, lr=3e-4, muon_lr=0.02, weight_decay=0.1, betas=(0.9, 0.95),
                 momentum: float = 0.95, nesterov: bool = True, ns_steps: int = 5, scale: str = "spectral",
                 eps: float = 1e-8):
        groups = [{"params": list(hidden_params), "muon": True, "lr": muon_lr, "weight_decay": weight_decay * lr / muon_lr}]
        for g in adam_groups:
            if g["params"]:
                groups.append({"params": g["params"], "muon": False, "lr": lr, "weight_decay": g.get("weight_decay", 0.0)})
        super().__init__(groups, dict(betas=betas, eps=eps))
        self.momentum, self.nesterov, self.ns_steps, self.scale_mode = momentum, nesterov, ns_steps, scale

    def _scale(self, shape) -> float:
        rows, cols = shape[-2], shape[-1]
        if self.scale_mode == "rms":
            return 0.2 * max(rows, cols) ** 0.5
        return max(1.0, rows / cols) ** 0.5

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            if group["muon"]:
                for p in group["params"]:
                    if p.grad is None:
                        continue
                    st = self.state[p]
                    if not st:
                        st["momentum"] = torch.zeros_like(p, dtype=torch.float32)
                    buf = st["momentum"].mul_(self.momentum).add_(p.grad.float())
                    g = p.grad.float().add(buf, alpha=self.momentum) if self.nesterov else buf
                    mats = g.reshape(-1, g.shape[-2], g.shape[-1])      # stacked experts: one matrix each
                    upd = torch.stack([newton_schulz(m, self.ns_steps) for m in mats]).reshape(g.shape)
                    p.mul_(1 - group["lr"] * group["weight_decay"])
                    p.add_(upd.to(p.dtype), alpha=-group["lr"] * self._scale(g.shape))
            else:
                b1, b2 = group["betas"]
                for p in group["params"]:
                    if p.grad is None:
                        continue
                    st = self.state[p]
                    if not st:
                        st["step"] = 0
                        st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                        st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
                    st["step"] += 1
                    g = p.grad.float()
                    st["exp_avg"].mul_(b1).add_(g, alpha=1 - b1)
                    st["exp_avg_sq"].mul_(b2).addcmul_(g, g, value=1 - b2)
                    bc1, bc2 = 1 - b1 ** st["step"], 1 - b2 ** st["step"]
                    upd = (st["exp_avg"] / bc1) / ((st["exp_avg_sq"] / bc2).sqrt() + group["eps"])
                    p.copy_((p.float() * (1 - group["lr"] * group["weight_decay"]) - group["lr"] * upd).to(p.dtype))
        return loss
