"""Whole-model checkpoints for pipeline (and data-parallel, and single-GPU) runs.

File layout (Lightning-shaped so generic tooling can open it)::

    {"state_dict": {whole-model name: tensor},
     "optimizer_states": [{"named_optimizer_state": {whole-model name: {...}}, "step": n}],
     "global_step": int, "epoch": int, "pytorch-lightning_version": "kohakuwupipe", **extra}

Weights AND optimizer state are keyed by the parameter's name in the whole model (stage-local block
index + the stage's first layer), never by rank or position, so a checkpoint written under one
pipeline split loads under any other split, under DDP, or on one GPU. Every rank contributes its
stage through ``all_gather_object``; rank 0 writes. Parameter groups are not stored: each rank rebuilds
them from its own parameters. Reference: src/kohakuwupipe/io/checkpoint.py:18-210.
"""

from __future__ import annotations

import os
from typing import Mapping

import torch
import torch.distributed as dist

FORMAT_TAG = "kohakuwupipe"


class CheckpointError(RuntimeError):
    """The checkpoint file cannot be read (truncated, corrupt, or not a checkpoint of this format)."""


def _world(group=None) -> int:
    return dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1


def _rank(group=None) -> int:
    return dist.get_rank(group) if dist.is_available() and dist.is_initialized() else 0


def local_state_dict(module: torch.nn.Module, names: Mapping[str, str] | None = None) -> dict[str, torch.Tensor]:
    """CPU copy of a module's parameters and persistent buffers under whole-model names."""
    names = names or {}
    out = {}
    for k, v in module.state_dict().items():
        out[names.get(k, k)] = v.detach().to("cpu", copy=True)
    return out


def gather_state_dict(module: torch.nn.Module, names: Mapping[str, str] | None = None, group=None) -> dict:
    """Union of every rank's ``local_state_dict`` (identical on all ranks)."""
    mine = local_state_dict(module, names)
    if _world(group) == 1:
        return mine
    parts: list = [None] * _world(group)
    dist.all_gather_object(parts, mine, group=group)
    merged: dict[str, torch.Tensor] = {}
    for part in parts:
        for k, v in part.items():
            merged.setdefault(k, v)
    return merged


def expert_sharded_names(module: torch.nn.Module) -> set[str]:
    """Names of the parameters of which every rank holds its own slice of the expert dimension."""
    return {n for n, p in module.named_parameters() if getattr(p, "ep_local", False)}


def named_state_of(optimizer, module: torch.nn.Module) -> dict:
    """``{"named_optimizer_state": {local parameter name: state}, "step": n}`` for ANY ``torch.optim.Optimizer``:
    the per-parameter state dicts re-keyed by the parameter's name in ``module`` (a stock optimizer keys its
    state by position, which does not survive another stage split)."""
    id2name = {id(p): n for n, p in module.named_parameters()}
    named, step = {}, 0
    for grp in optimizer.param_groups:
        for p in grp["params"]:
            st = optimizer.state.get(p)
            if st and id(p) in id2name:
                named[id2name[id(p)]] = dict(st)
                s0 = st.get("step", 0)
                step = max(step, int(s0.item()) if torch.is_tensor(s0) else int(s0))
    return {"named_optimizer_state": named, "step": step}


def load_named_state_into(optimizer, module: torch.nn.Module, named: dict) -> None:
    """Inverse of ``named_state_of`` for a stock optimizer: state found under a parameter's name is installed."""
    for n, p in module.named_parameters():
        entry = named.get(n)
        if entry is None:
            continue
        optimizer.state[p] = {k: (v.to(p.device) if torch.is_tensor(v) else v) for k, v in entry.items()
                              if k != "range"}


def gather_optimizer_state(optimizer, names: Mapping[str, str] | None = None, group=None,
                           ep_names: set[str] | frozenset[str] = frozenset(), module: torch.nn.Module | None = None) -> dict:
    """Whole-model-named optimizer state. ``optimizer.state_dict()`` must expose
    ``named_optimizer_state`` keyed by local parameter names (``FlatAdamW`` does). Entries of ``ep_names``
    (expert-parallel parameters: every rank owns a different slice under the same name) are concatenated in
    rank order, which is the order of the expert dimension; all others are merged by their flat ranges."""
    names = names or {}
    sd = optimizer.state_dict()
    if "named_optimizer_state" not in sd:
        if module is None:
            raise ValueError("this optimizer keys its state by position; pass the module so that it can be re-keyed by name")
        sd = named_state_of(optimizer, module)
    mine = {names.get(k, k): {kk: (vv.detach().to("cpu", copy=True) if torch.is_tensor(vv) else vv)
                              for kk, vv in v.items()}
            for k, v in sd["named_optimizer_state"].items()}
    if _world(group) > 1:
        parts: list = [None] * _world(group)
        dist.all_gather_object(parts, mine, group=group)
        merged: dict = {}
        ep_global = {names.get(k, k) for k in ep_names}
        for part in parts:
            for k, v in part.items():
                if k not in merged:
                    merged[k] = v
                elif k in ep_global:
                    merged[k] = _concat_expert_slices(merged[k], v)
                elif "range" in v and "range" in merged[k]:
                    merged[k] = _merge_ranges(merged[k], v)
        mine = merged
    return {"named_optimizer_state": mine, "step": sd.get("step", 0), "hyper": sd.get("hyper", {})}


def _concat_expert_slices(a: dict, b: dict) -> dict:
    """Append rank r+1's state of an expert-parallel parameter to the ranks before it."""
    out = {}
    for k in a:
        if torch.is_tensor(a[k]):
            out[k] = torch.cat([a[k].reshape(-1), b[k].reshape(-1)])
    out["range"] = (0, next(iter(out.values())).numel())
    return out


def _local_expert_slice(entry: dict, local_numel: int, rank: int, world: int) -> dict:
    """This rank's part of a whole-model optimizer entry of an expert-parallel parameter."""
    lo, hi = entry.get("range", (0, None))
    n = next(v for v in entry.values() if torch.is_tensor(v)).numel()
    if lo != 0 or n == local_numel:
        return entry                                  # already a local slice (same layout as saved)
    if n != local_numel * world:
        raise ValueError(f"optimizer state of {n} elements does not split into {world} x {local_numel}")
    out = {k: (v.reshape(-1)[rank * local_numel:(rank + 1) * local_numel].clone() if torch.is_tensor(v) else v)
           for k, v in entry.items()}
    out["range"] = (0, local_numel)
    return out


def _merge_ranges(a: dict, b: dict) -> dict:
    """Concatenate two partial (sharded) states of one parameter into one covering both ranges."""
    first, second = (a, b) if a["range"][0] <= b["range"][0] else (b, a)
    if first["range"][1] != second["range"][0]:
        return first if (first["range"][1] - first["range"][0]) >= (second["range"][1] - second["range"][0]) else second
    out = {"range": (first["range"][0], second["range"][1])}
    for k in first:
        if k != "range" and torch.is_tensor(first[k]):
            out[k] = torch.cat([first[k].reshape(-1), second[k].reshape(-1)])
    return out


def save(path: str, module: torch.nn.Module, optimizer=None, *, names: Mapping[str, str] | None = None,
         global_step: int = 0, epoch: int = 0, extra: dict | None = None, group=None) -> None:
    state = gather_state_dict(module, names, group)
    opt = gather_optimizer_state(optimizer, names, group, module=module) if optimizer is not None else None
    if _rank(group) == 0:
        payload = {"state_dict": state, "optimizer_states": [opt] if opt is not None else [],
                   "global_step": int(global_step), "epoch": int(epoch),
                   "pytorch-lightning_version": FORMAT_TAG}
        payload.update(extra or {})
        tmp = f"{path}.tmp"
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        torch.save(payload, tmp)
        os.replace(tmp, path)
    if _world(group) > 1:
        dist.barrier(group=group)


def read_payload(path: str) -> dict:
    """``torch.load`` of a checkpoint file, with every way a damaged file can fail turned into one
    ``CheckpointError`` that names the file (a write that was cut short leaves a zip archive without its
    central directory; a file of another kind fails in the unpickler)."""
    import pickle
    import zipfile

    try:
        payload = torch.load(path, map_location="cpu", weights_only=False)
    except FileNotFoundError:
        raise
    except (RuntimeError, EOFError, OSError, ValueError, pickle.UnpicklingError, zipfile.BadZipFile) as exc:
        raise CheckpointError(f"checkpoint {path} is unreadable (truncated or corrupt): "
                              f"{type(exc).__name__}: {exc}") from exc
    if not isinstance(payload, dict) or "state_dict" not in payload:
        raise CheckpointError(f"checkpoint {path} holds no 'state_dict': not a checkpoint of this format")
    return payload


def load(path: str, module: torch.nn.Module, optimizer=None, *, names: Mapping[str, str] | None = None,
         strict: bool = True, group=None) -> dict:
    """Load the slice of a whole-model checkpoint that this module (stage) owns. Returns the payload
    without the big tensors (progress, scheduler state, ...)."""
    payload = read_payload(path)
    names = dict(names or {})
    state = payload["state_dict"]
    local = {}
    missing = []
    ep_params = {n: p for n, p in module.named_parameters() if getattr(p, "ep_local", False)}
    world, rank = _world(group), _rank(group)
    for k in module.state_dict().keys():
        g = names.get(k, k)
        if g in state:
            t = state[g]
            if k in ep_params and t.shape[0] != ep_params[k].shape[0]:
                # a whole-model tensor into an expert-parallel module: keep this rank's experts
                n_local = ep_params[k].shape[0]
                if t.shape[0] != n_local * world:
                    raise ValueError(f"{g}: {t.shape[0]} experts do not split into {world} x {n_local}")
                t = t[rank * n_local:(rank + 1) * n_local]
            local[k] = t
        else:
            missing.append(g)
    if missing and strict:
        raise KeyError(f"checkpoint {path} lacks {len(missing)} tensors of this stage, e.g. {missing[:3]}")
    module.load_state_dict(local, strict=False)
    if optimizer is not None and payload.get("optimizer_states"):
        opt = payload["optimizer_states"][0]
        if "named_optimizer_state" not in opt:
            world = _world(group)
            per_rank = payload["optimizer_states"]
            if len(per_rank) != world:
                raise RuntimeError(f"legacy per-rank optimizer state of {len(per_rank)} ranks cannot be loaded "
                                   f"at world size {world}")
            optimizer.load_state_dict(per_rank[_rank(group)])
        else:
            inverse = {v: k for k, v in names.items()}
            named = {inverse.get(g, g): v for g, v in opt["named_optimizer_state"].items()}
            for k, p in ep_params.items():
                if k in named:
                    named[k] = _local_expert_slice(named[k], p.numel(), rank, world)
            if "named_optimizer_state" in optimizer.state_dict():
                optimizer.load_state_dict({"named_optimizer_state": named, "step": opt.get("step", 0)})
            else:
                load_named_state_into(optimizer, module, named)
    return {k: v for k, v in payload.items() if k not in ("state_dict", "optimizer_states")}
