"""Fused data-parallel step: gradient reduce-scatter + token-count scaling + global-norm clipping +
partitioned AdamW + parameter all-gather, in two kernels over NVLink peer memory
(``csrc/fused_ddp.cu``). Optimizer state (fp32 master, exp_avg, exp_avg_sq) is held only for the
rank's 1/W shard; checkpoints still carry whole-model-named state (``FlatAdamW.state_dict`` + the
gather in ``pipe/checkpoint.py``).

Usage::

    pool = SymmetricPool(group)
    flat = FlatParameters(model, allocator=pool.empty)     # params and grads in symmetric memory
    sync = FusedGradSync(flat, pool, group)
    opt  = FlatAdamW(flat, ..., shard=(rank, world))
    ...backward of all micro-batches...
    sync.step(opt, inv_tokens, max_grad_norm)              # replaces all-reduce + clip + optimizer.step
"""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from kohakuwullm_b200.ops import native
from kohakuwullm_b200.parallel.flat import FlatParameters
from kohakuwullm_b200.parallel.symm import SymmetricPool

c_int, c_ll, c_float = ctypes.c_int, ctypes.c_longlong, ctypes.c_float


class FusedGradSync:
    def __init__(self, flat: FlatParameters, pool: SymmetricPool, group=None, wait_limit_cycles: int = 0):
        self.flat, self.pool, self.group = flat, pool, group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > 8:
            raise ValueError("the fused data-parallel kernels support up to 8 ranks (one NVSwitch domain)")
        dev = next(iter(flat.groups.values())).data.device
        self.device = dev
        # flag block: [ready W][sq W][done W] int32, and W float slots for the shard norms
        self.flags = pool.empty(3 * 8, torch.int32, dev)
        self.slots = pool.empty(8, torch.float32, dev)
        self.flags.zero_()
        self.slots.zero_()
        pool.rendezvous_all()
        torch.cuda.synchronize(dev)
        dist.barrier(group=group)
        self._flag_tab = pool.find(self.flags).ptr_table()
        self._slot_tab = pool.find(self.slots).ptr_table()
        self._tabs = {key: (pool.find(g.main_grad).ptr_table(), pool.find(g.data).ptr_table())
                      for key, g in flat.groups.items()}
        L = native.require()
        self._partial = torch.zeros(L.kwu_ddp_blocks(), dtype=torch.float32, device=dev)
        self._counter = torch.zeros(1, dtype=torch.int32, device=dev)
        self._sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        self.norm = torch.zeros(1, dtype=torch.float32, device=dev)
        self.epoch = 0
        self.limit = wait_limit_cycles
        self._sq_partial = None

    # plain collectives used around the fused step (token counts, logged scalars)
    def all_reduce_scalar(self, t: torch.Tensor) -> torch.Tensor:
        dist.all_reduce(t, group=self.group)
        return t

    def reduce(self) -> None:  # the reduction is part of step()
        pass

    @torch.no_grad()
    def step(self, optimizer, inv_tokens: torch.Tensor, max_grad_norm: float) -> None:
        L = native.require()
        self.epoch += 1
        optimizer.step_count += 1
        lr = optimizer.param_groups[0]["lr"]
        keys = self.flat.replicated_keys()
        local_keys = self.flat.local_keys()
        status = native.ptr(native.status_word())
        stream = native.stream_ptr()
        # expert-parallel shards are not reduced, but their squared norm belongs to the global norm: seed
        # this rank's partial sum with it before the reduced shards are added
        for j, key in enumerate(local_keys):
            buf = self.flat.groups[key].main_grad
            if self._sq_partial is None:
                self._sq_partial = torch.empty(L.kwu_sumsq_blocks(), dtype=torch.float32, device=self.device)
            rc = L.kwu_sumsq_flat(native.ptr(buf), c_ll(buf.numel()), native.ptr(self._sq_partial),
                                  native.ptr(self._sumsq), c_int(int(j > 0)), stream)
            native.check(rc, "sumsq_flat")
        seeded = bool(local_keys)
        for i, key in enumerate(keys):
            g = self.flat.groups[key]
            lo, hi = optimizer._range(g)
            grad_tab, param_tab = self._tabs[key]
            rc = L.kwu_ddp_reduce_shard(grad_tab, param_tab, self._flag_tab, self._slot_tab, c_int(self.rank),
                                        c_int(self.world), c_int(self.epoch), c_ll(lo), c_ll(hi - lo),
                                        native.ptr(self._partial), native.ptr(self._counter),
                                        native.ptr(self._sumsq), c_int(int(i == 0 and not seeded)),
                                        c_int(int(i == len(keys) - 1)), c_int(int(i == 0)), c_ll(self.limit),
                                        stream, status)
            native.check(rc, "ddp_reduce_shard")
        for i, key in enumerate(keys):
            g = self.flat.groups[key]
            st = optimizer.state[key]
            lo, hi = optimizer._range(g)
            grad_tab, param_tab = self._tabs[key]
            master = st.get("master")
            rc = L.kwu_ddp_adamw_allgather(
                grad_tab, param_tab, self._flag_tab, self._slot_tab, c_int(self.rank), c_int(self.world),
                c_int(self.epoch), c_ll(lo), c_ll(hi - lo), c_ll(g.total), native.ptr(master),
                native.ptr(st["exp_avg"]), native.ptr(st["exp_avg_sq"]), c_int(int(g.dtype == torch.bfloat16)),
                native.ptr(st["seg_start"]), native.ptr(st["seg_wd"]), native.ptr(st["seg_lr"]),
                c_int(len(g.names)), native.ptr(inv_tokens), c_float(max_grad_norm or 0.0), native.ptr(self.norm),
                c_float(lr), c_float(optimizer.betas[0]), c_float(optimizer.betas[1]), c_float(optimizer.eps),
                c_int(optimizer.step_count), native.ptr(self._counter), c_int(int(i == len(keys) - 1)), c_int(1),
                c_ll(self.limit), stream, status)
            native.check(rc, "ddp_adamw_allgather")
        if local_keys:
            # same scale as inside the fused kernel: 1/tokens times the clipping coefficient
            coef = inv_tokens.reshape(1).clone()
            if max_grad_norm:
                coef = coef * torch.clamp(max_grad_norm / (self.norm + 1e-6), max=1.0)
            optimizer.step(grad_scale=coef, zero_grad=True, only=set(local_keys), advance=False)
