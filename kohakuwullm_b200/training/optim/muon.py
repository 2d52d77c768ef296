"""``MuonW``: Muon (momentum + Newton-Schulz orthogonalisation) for hidden matrices, 16-bit-state AdamW for
everything else.

Orthogonalisation. For a matrix ``X`` (n, m), n <= m (taller matrices are handled through their transpose),
scaled into the iteration's convergence radius, two iterations are offered:

* ``quintic``  ``X <- a X + (b G + c G G) X`` with ``G = X X^T`` and the fixed coefficients
  (3.4445, -4.7750, 2.0315): three products per step.
* ``cubic5``   five steps ``X <- (a_k I + b_k G) X`` with a per-step schedule: two products per step. Steps can
  be chained in GRAM SPACE: with ``S = a I + b G`` the next Gram matrix is ``S G S`` (n x n products only), so a
  phase of L steps needs one Gram product, 2 (L - 1) small products and ONE n x m product. Shapes whose aspect
  ratio m / n is at least ``gram_aspect`` use the phases (2, 3); squarer ones run the five steps directly.

Batching. All matrices of one shape (the q/k/v/o, MLP and stacked expert weights of every layer) are stacked
and orthogonalised as ONE batch per product, up to ``ns_batch_elems`` elements at a time. On a B200 the batched
products run on the tcgen05 grouped GEMM (every matrix of the batch is one "expert" of a grouped product: one
launch per product for the whole batch, no transposes: ``X X^T`` and ``G G`` take both operands K-major, ``P X``
takes X MN-major); elsewhere ``torch.bmm``.

Write-back: ``p <- p (1 - lr wd) - lr scale U`` with ``scale`` = ``sqrt(max(1, rows / cols))`` (``spectral``) or
``rms_target sqrt(max(rows, cols))`` (``rms``); ``rounding="stochastic"`` rounds the bf16 result stochastically
(Philox stream, offset advancing by each parameter's element count so the stream does not depend on batching).
Reference: src/kohakuwullm/training/optim/muon.py:20-107 (iterations), :178-442 (optimizer).
"""

from __future__ import annotations

import math

import torch

from kohakuwullm_b200.ops import native
from kohakuwullm_b200.ops.optim import adamw16_step_, sr_update_

NS_QUINTIC = (3.4445, -4.7750, 2.0315)
NS_CUBIC5 = ((3.3656576, -3.3420992), (2.5744352, -1.4957376), (2.5368962, -1.4312570),
             (2.4418906, -1.2764040), (2.2230472, -0.9630650))
PHASES_GRAM = (2, 3)
PHASES_DIRECT = (1, 1, 1, 1, 1)


# ------------------------------------------------------------------------------------ batched products
def _native_batched(a: torch.Tensor, b: torch.Tensor) -> bool:
    return (a.is_cuda and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and native.available()
            and a.shape[1] % 128 == 0 and a.shape[2] % 8 == 0 and b.shape[2] % 8 == 0)


_tile_tables: dict[tuple, torch.Tensor] = {}


def _tiles(batch: int, rows: int, device) -> torch.Tensor:
    """Row-tile table of the grouped GEMM for ``batch`` matrices of ``rows`` rows: (first row, matrix, valid, 0)."""
    key = (batch, rows, str(device))
    t = _tile_tables.get(key)
    if t is None:
        per = rows // 128
        m0 = torch.arange(batch * per, dtype=torch.int32) * 128
        t = torch.stack([m0, m0 // rows, torch.ones_like(m0), torch.zeros_like(m0)], dim=1).contiguous().to(device)
        _tile_tables[key] = t
    return t


def bmm_nt(a: torch.Tensor, b: torch.Tensor, b_mn: bool = False) -> torch.Tensor:
    """Batched ``a[i] @ op(b[i])``: a (B, M, K); b (B, N, K) with ``b_mn`` false (product with b^T), or b (B, K, N)
    with ``b_mn`` true (plain product). One grouped tcgen05 launch on a B200, ``torch.bmm`` elsewhere."""
    B, M, K = a.shape
    N = b.shape[2] if b_mn else b.shape[1]
    if not (_native_batched(a, b) and a.is_contiguous() and b.is_contiguous()):
        return torch.bmm(a, b if b_mn else b.transpose(1, 2))
    import ctypes

    L = native.require()
    out = torch.empty(B, M, N, dtype=a.dtype, device=a.device)
    tiles = _tiles(B, M, a.device)
    ci = ctypes.c_int
    rc = L.kwu_gemm_bf16_grouped_rows(native.ptr(a), native.ptr(b), native.ptr(out), ci(B * M), ci(N), ci(K), ci(K),
                                      ci(b.shape[2]), ci(N), ci(int(b_mn)), ci(B), native.ptr(tiles),
                                      ci(tiles.shape[0]), ci(0), native.ptr(None), native.stream_ptr(),
                                      native.ptr(native.status_word()))
    native.check(rc, "muon batched gemm")
    return out


# ------------------------------------------------------------------------------------ Newton-Schulz
def _prepare(grad: torch.Tensor, dtype: torch.dtype):
    """(B, n, m) in ``dtype`` with n <= m and every matrix scaled to Frobenius norm 1 / 1.01; plus the flag that
    says the result must be transposed back."""
    x = grad.reshape(-1, grad.shape[-2], grad.shape[-1])
    norm = torch.linalg.vector_norm(x, dim=(-2, -1), keepdim=True, dtype=torch.float32).clamp_min(1e-7) * 1.01
    x = (x.float() / norm).to(dtype)
    transposed = x.shape[-2] > x.shape[-1]
    if transposed:
        x = x.transpose(1, 2).contiguous()
    return x, transposed


def _finish(x: torch.Tensor, transposed: bool, shape) -> torch.Tensor:
    if transposed:
        x = x.transpose(1, 2)
    return x.reshape(shape)


def newton_schulz(grad: torch.Tensor, steps: int = 5, dtype: torch.dtype = torch.bfloat16,
                  coeffs=NS_QUINTIC) -> torch.Tensor:
    """Quintic iteration, batched over every leading dimension. Returns ``dtype``."""
    a, b, c = coeffs
    x, transposed = _prepare(grad, dtype)
    for _ in range(steps):
        gram = bmm_nt(x, x)                                   # X X^T
        poly = torch.add(gram * b, bmm_nt(gram, gram), alpha=c)   # b G + c G G (G is symmetric: G G^T = G G)
        x = torch.add(bmm_nt(poly, x, b_mn=True), x, alpha=a)
    return _finish(x, transposed, grad.shape)


def newton_schulz_cubic(grad: torch.Tensor, dtype: torch.dtype = torch.bfloat16, schedule=NS_CUBIC5,
                        phases=PHASES_DIRECT) -> torch.Tensor:
    """Cubic schedule with gram-space phases (see the module docstring). ``phases`` must sum to the number of
    steps of the schedule."""
    if sum(phases) != len(schedule):
        raise ValueError(f"phases {phases} sum to {sum(phases)}, the schedule has {len(schedule)} steps")
    x, transposed = _prepare(grad, dtype)
    n = x.shape[1]
    eye = torch.eye(n, dtype=dtype, device=x.device)
    k = 0
    for length in phases:
        gram = bmm_nt(x, x)
        product = None
        for j in range(length):
            a, b = schedule[k + j]
            step = torch.add(eye * a, gram, alpha=b)          # S = a I + b G (symmetric)
            product = step if product is None else bmm_nt(step, product, b_mn=True)
            if j + 1 < length:
                gram = bmm_nt(bmm_nt(step, gram, b_mn=True), step, b_mn=True)   # S G S
        x = bmm_nt(product, x, b_mn=True)
        k += length
    return _finish(x, transposed, grad.shape)


def orthogonal_update_scale(shape, mode: str, rms_target: float = 0.2) -> float:
    rows, cols = shape[-2], shape[-1]
    if mode == "spectral":
        return max(1.0, rows / cols) ** 0.5
    if mode == "rms":
        return rms_target * max(rows, cols) ** 0.5
    raise ValueError(f"unknown update_scale {mode!r}; use 'spectral' or 'rms'")


# ------------------------------------------------------------------------------------ optimizer
class MuonW(torch.optim.Optimizer):
    """``hidden_params``: the matrices that take the orthogonalised step (>= 2-D; a stacked (E, out, in) expert
    weight is E matrices). ``adam_groups``: parameter groups for the internal AdamW (state in the parameter's
    dtype with the second moment stored as its square root, fp32 arithmetic)."""

    def __init__(self, hidden_params, adam_groups, lr: float = 3e-4, muon_lr: float = 0.02, weight_decay: float = 0.1,
                 betas=(0.9, 0.95), momentum: float = 0.95, nesterov: bool = True, ns_steps: int = 5,
                 ns_variant: str = "cubic5", ns_dtype: torch.dtype = torch.bfloat16, ns_batch_elems: int = 64 << 20,
                 gram_aspect: float = 1.5, update_scale: str = "spectral", rms_target: float = 0.2,
                 rounding: str = "nearest", seed: int = 0, eps: float = 1e-8, scale: str | None = None):
        if ns_variant not in ("cubic5", "quintic"):
            raise ValueError(f"unknown ns_variant {ns_variant!r}")
        if rounding not in ("nearest", "stochastic"):
            raise ValueError(f"unknown rounding rule {rounding!r}")
        update_scale = scale or update_scale
        hidden = list(hidden_params)
        for p in hidden:
            if p.dim() < 2:
                raise ValueError(f"a {p.dim()}-D parameter reached the Muon group: it has no singular values to equalise")
        # decay is decoupled and expressed per unit of the AdamW learning rate, so that both kinds of group
        # shrink at the same rate: wd_muon * muon_lr == weight_decay * lr
        groups = [{"params": hidden, "use_muon": True, "lr": muon_lr,
                   "weight_decay": weight_decay * lr / muon_lr if muon_lr else 0.0}]
        for g in adam_groups:
            if g["params"]:
                groups.append({"params": list(g["params"]), "use_muon": False, "lr": g.get("lr", lr),
                               "weight_decay": g.get("weight_decay", 0.0)})
        super().__init__(groups, dict(betas=betas, eps=eps))
        self.momentum, self.nesterov, self.ns_steps = momentum, nesterov, ns_steps
        self.ns_variant, self.ns_dtype, self.ns_batch_elems = ns_variant, ns_dtype, ns_batch_elems
        self.gram_aspect, self.update_scale, self.rms_target = gram_aspect, update_scale, rms_target
        self.stochastic, self.seed, self._sr_offset = rounding == "stochastic", seed, 0
        self._phases: dict[tuple, tuple] = {}

    # ------------------------------------------------------------------ helpers
    def phases_for(self, shape) -> tuple:
        """Gram-space grouping for wide shapes, direct steps for squarish ones (decided once per shape)."""
        key = tuple(shape[-2:])
        if key not in self._phases:
            short, long = sorted(key)
            self._phases[key] = PHASES_GRAM if long >= self.gram_aspect * short else PHASES_DIRECT
        return self._phases[key]

    def orthogonalize(self, batch: torch.Tensor) -> torch.Tensor:
        dtype = self.ns_dtype if batch.is_cuda else torch.float32
        if self.ns_variant == "cubic5":
            return newton_schulz_cubic(batch, dtype, phases=self.phases_for(batch.shape))
        return newton_schulz(batch, self.ns_steps, dtype)

    def _batch_size(self, shape) -> int:
        return max(1, self.ns_batch_elems // max(math.prod(shape), 1))

    # ------------------------------------------------------------------ step
    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            if group["use_muon"]:
                self._muon_group(group)
            else:
                self._adam_group(group)
        return loss

    def _muon_group(self, group) -> None:
        by_shape: dict[tuple, list] = {}
        for p in group["params"]:
            if p.grad is None:
                continue
            st = self.state[p]
            if "momentum_buffer" not in st:
                st["momentum_buffer"] = torch.zeros_like(p)
            by_shape.setdefault(tuple(p.shape), []).append(p)
        lr, wd, beta = group["lr"], group["weight_decay"], self.momentum
        for shape, params in by_shape.items():
            per = self._batch_size(shape)
            scale = orthogonal_update_scale(shape, self.update_scale, self.rms_target)
            for s in range(0, len(params), per):
                chunk = params[s:s + per]
                bufs = [self.state[p]["momentum_buffer"] for p in chunk]
                grads = [p.grad.to(b.dtype) for p, b in zip(chunk, bufs)]
                torch._foreach_lerp_(bufs, grads, 1 - beta)              # momentum EMA, one fused pass
                if self.nesterov:
                    direction = torch._foreach_lerp(grads, bufs, beta)   # look-ahead; .grad is left untouched
                else:
                    direction = bufs
                updates = self.orthogonalize(torch.stack(direction))    # (chunk, *shape)
                if self.stochastic and chunk[0].dtype == torch.bfloat16:
                    for p, u in zip(chunk, updates):
                        sr_update_(p, u.float().contiguous(), lr * wd, -lr * scale, seed=self.seed, offset=self._sr_offset)
                        self._sr_offset += p.numel()
                else:
                    torch._foreach_mul_(chunk, 1 - lr * wd)
                    torch._foreach_add_(chunk, [u.to(p.dtype) for p, u in zip(chunk, updates)], alpha=-lr * scale)

    def _adam_group(self, group) -> None:
        b1, b2 = group["betas"]
        for p in group["params"]:
            if p.grad is None:
                continue
            st = self.state[p]
            if "exp_avg" not in st:
                st["exp_avg"] = torch.zeros_like(p)
                st["exp_avg_rms"] = torch.zeros_like(p)
                st["step"] = 0
            st["step"] += 1
            adamw16_step_(p, st["exp_avg"], st["exp_avg_rms"], p.grad.to(p.dtype), lr=group["lr"], betas=(b1, b2),
                          eps=group["eps"], wd=group["weight_decay"], step=st["step"],
                          stochastic=self.stochastic and p.dtype == torch.bfloat16, seed=self.seed)
