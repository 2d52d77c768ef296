"""AdamW over flat buffers: one kernel launch updates the whole model.

State per dtype group: fp32 ``exp_avg`` / ``exp_avg_sq`` and, for the 16-bit group, an fp32 master copy
(the fp32 group is its own master). The gradient is ``main_grad * grad_scale`` where ``grad_scale`` is
a DEVICE scalar (1 / global trained tokens, times the clipping coefficient), so neither token-exact
normalisation nor clipping needs a host round trip. The kernel also zeroes ``main_grad``.

With ``shard=(rank, world)`` only the rank's contiguous 1/world slice of every group is updated and
holds state (ZeRO-1 style); the caller all-gathers the updated parameters. ``state_dict`` always
returns whole-model, per-parameter-name tensors, whatever the sharding.
Reference: src/kohakuwullm/training/optim/fused_adamw.py:7-172.
"""

from __future__ import annotations

import ctypes

import torch

from kohakuwullm_b200.ops import native
from kohakuwullm_b200.parallel.flat import FlatGroup, FlatParameters


def default_decay_rule(name: str, p: torch.Tensor, decay_embeddings: bool = False) -> bool:
    """Decay only matrices; never the selection bias; the input embedding only on request."""
    if p.dim() < 2 or "expert_bias" in name or name.endswith("sink"):
        return False
    if not decay_embeddings and "embed" in name.split("."):
        return False
    return True


class FlatAdamW:
    def __init__(self, flat: FlatParameters, lr: float = 3e-4, betas=(0.9, 0.95), eps: float = 1e-8,
                 weight_decay: float = 0.1, decay_rule=default_decay_rule, lr_mult_rule=None,
                 shard: tuple[int, int] | None = None):
        self.flat = flat
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.step_count = 0
        self.shard = shard
        self.state: dict[str, dict[str, torch.Tensor]] = {}
        self.param_groups = [{"lr": lr}]  # for schedulers that set group["lr"]
        for key, g in flat.groups.items():
            lo, hi = self._range(g)
            n = hi - lo
            dev = g.data.device
            seg_start, seg_wd, seg_lr = [], [], []
            for i, (name, p) in enumerate(zip(g.names, g.params)):
                seg_start.append(g.offsets[i])
                seg_wd.append(weight_decay if decay_rule(name, p) else 0.0)
                seg_lr.append(lr_mult_rule(name, p) if lr_mult_rule else 1.0)
            st = {
                "exp_avg": torch.zeros(n, dtype=torch.float32, device=dev),
                "exp_avg_sq": torch.zeros(n, dtype=torch.float32, device=dev),
                "seg_start": torch.tensor(seg_start, dtype=torch.int64, device=dev),
                "seg_wd": torch.tensor(seg_wd, dtype=torch.float32, device=dev),
                "seg_lr": torch.tensor(seg_lr, dtype=torch.float32, device=dev),
            }
            if g.dtype != torch.float32:
                st["master"] = g.data[lo:hi].float()
            self.state[key] = st

    def _range(self, g: FlatGroup) -> tuple[int, int]:
        if self.shard is None or g.key.endswith("_ep"):  # expert-parallel shards are already rank-local
            return 0, g.total
        # equal shards rounded UP to 8 elements (the fused kernels move 8 at a time), the last one clipped:
        # every element has exactly one owner for any world size (total is a multiple of 1024, not of 8 * world)
        rank, world = self.shard
        per = -(-g.total // world)
        per = -(-per // 8) * 8
        return min(rank * per, g.total), min((rank + 1) * per, g.total)

    # ------------------------------------------------------------------
    @torch.no_grad()
    def step(self, grad_scale: torch.Tensor | None = None, zero_grad: bool = True, only=None,
             advance: bool = True) -> None:
        """``only``: restrict the update to these group keys; ``advance=False`` keeps the step counter
        (used when another kernel already updated the remaining groups of the same step)."""
        if advance:
            self.step_count += 1
        lr = self.param_groups[0]["lr"]
        for key, g in self.flat.groups.items():
            if only is not None and key not in only:
                continue
            st = self.state[key]
            lo, hi = self._range(g)
            master = st.get("master")
            grad = g.main_grad[lo:hi]
            if g.data.is_cuda and native.available():
                L = native.require()
                lp = g.data[lo:hi] if master is not None else None
                mst = master if master is not None else g.data[lo:hi]
                # the segment table is in whole-buffer coordinates; shift by the shard start
                seg_start = st["seg_start"] if lo == 0 else (st["seg_start"] - lo).clamp(min=0)
                rc = L.kwu_adamw_flat(
                    native.ptr(mst), native.ptr(st["exp_avg"]), native.ptr(st["exp_avg_sq"]),
                    native.ptr(grad), native.ptr(lp), native.ptr(seg_start), native.ptr(st["seg_wd"]),
                    native.ptr(st["seg_lr"]), ctypes.c_int(len(g.names)), ctypes.c_longlong(hi - lo),
                    native.ptr(grad_scale), ctypes.c_float(lr), ctypes.c_float(self.betas[0]),
                    ctypes.c_float(self.betas[1]), ctypes.c_float(self.eps), ctypes.c_int(self.step_count),
                    ctypes.c_int(int(zero_grad)), native.stream_ptr())
                native.check(rc, "adamw_flat")
            else:
                self._step_torch(g, st, lo, hi, grad, grad_scale, lr, zero_grad)

    def _step_torch(self, g, st, lo, hi, grad, grad_scale, lr, zero_grad):
        b1, b2 = self.betas
        gs = grad if grad_scale is None else grad * grad_scale.to(grad.dtype)
        m, v = st["exp_avg"], st["exp_avg_sq"]
        m.mul_(b1).add_(gs, alpha=1 - b1)
        v.mul_(b2).addcmul_(gs, gs, value=1 - b2)
        bc1 = 1 - b1 ** self.step_count
        bc2 = 1 - b2 ** self.step_count
        update = (m / bc1) / ((v / bc2).sqrt() + self.eps)
        master = st.get("master")
        target = master if master is not None else g.data[lo:hi]
        # expand the segment table into per-element decay / lr multipliers
        starts = st["seg_start"].tolist() + [g.total]
        wd = torch.zeros(hi - lo, dtype=torch.float32, device=grad.device)
        lrm = torch.ones(hi - lo, dtype=torch.float32, device=grad.device)
        for i in range(len(g.names)):
            s, e = max(starts[i], lo) - lo, min(starts[i + 1], hi) - lo
            if e > s:
                wd[s:e] = st["seg_wd"][i]
                lrm[s:e] = st["seg_lr"][i]
        target.mul_(1 - lr * lrm * wd).sub_(lr * lrm * update)
        if master is not None:
            g.data[lo:hi].copy_(master)
        if zero_grad:
            grad.zero_()

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.flat.zero_grad()

    # ------------------------------------------------------------------ checkpointing
    def state_dict(self) -> dict:
        """Per-parameter-name state of the locally held range (whole model when unsharded)."""
        named: dict[str, dict[str, torch.Tensor]] = {}
        for key, g in self.flat.groups.items():
            st = self.state[key]
            lo, hi = self._range(g)
            for i, name in enumerate(g.names):
                s, e = g.span(i)
                a, b = max(s, lo), min(e, hi)
                if b <= a:
                    continue
                entry = {"exp_avg": st["exp_avg"][a - lo:b - lo].clone(),
                         "exp_avg_sq": st["exp_avg_sq"][a - lo:b - lo].clone(),
                         "range": (a - s, b - s)}
                if "master" in st:
                    entry["master"] = st["master"][a - lo:b - lo].clone()
                named[name] = entry
        return {"step": self.step_count, "named_optimizer_state": named,
                "hyper": {"lr": self.param_groups[0]["lr"], "betas": self.betas, "eps": self.eps,
                          "weight_decay": self.weight_decay}}

    def load_state_dict(self, sd: dict) -> None:
        self.step_count = int(sd.get("step", 0))
        named = sd["named_optimizer_state"]
        for key, g in self.flat.groups.items():
            st = self.state[key]
            lo, hi = self._range(g)
            for i, name in enumerate(g.names):
                if name not in named:
                    continue
                entry = named[name]
                s, e = g.span(i)
                src_lo, src_hi = entry.get("range", (0, e - s))
                a, b = max(s + src_lo, lo), min(s + src_hi, hi)
                if b <= a:
                    continue
                sl = slice(a - s - src_lo, b - s - src_lo)
                st["exp_avg"][a - lo:b - lo].copy_(entry["exp_avg"].reshape(-1)[sl])
                st["exp_avg_sq"][a - lo:b - lo].copy_(entry["exp_avg_sq"].reshape(-1)[sl])
                if "master" in st:
                    if "master" in entry:
                        st["master"][a - lo:b - lo].copy_(entry["master"].reshape(-1)[sl])
                    else:
                        st["master"][a - lo:b - lo].copy_(g.data[a:b].float())
