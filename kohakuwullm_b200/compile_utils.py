"""Optional ``torch.compile`` of the framework-level glue. The hot path is hand-written kernels replayed
from CUDA graphs (``TrainEngine``), so compilation is off by default; it remains available for the eager
fallbacks. ``mode``: ``off`` | ``model`` (whole module) | ``module`` (each child named in ``targets``,
compiled IN PLACE so state-dict keys keep no ``_orig_mod.`` prefix).
Reference: src/kohakuwullm/compile_utils.py:19-66."""

from __future__ import annotations

import torch
from torch import nn


def raise_recompile_limit(limit: int = 64) -> None:
    import torch._dynamo as dynamo

    dynamo.config.cache_size_limit = max(dynamo.config.cache_size_limit, limit)
    if hasattr(dynamo.config, "accumulated_cache_size_limit"):
        dynamo.config.accumulated_cache_size_limit = max(dynamo.config.accumulated_cache_size_limit, 4 * limit)


def apply_compile(model: nn.Module, spec: dict | str | None) -> nn.Module:
    if not spec or spec == "off":
        return model
    spec = {"mode": spec} if isinstance(spec, str) else dict(spec)
    mode = spec.pop("mode", "module")
    if mode == "off":
        return model
    targets = spec.pop("targets", ["blocks"])
    exclude = set(spec.pop("exclude", []))
    raise_recompile_limit()
    if mode == "model":
        model.compile(**spec)
        return model
    if mode != "module":
        raise ValueError(f"compile mode must be off, model or module, got {mode!r}")
    for name in targets:
        container = getattr(model, name)
        children = container if isinstance(container, (nn.ModuleList, nn.Sequential)) else [container]
        for i, child in enumerate(children):
            if f"{name}.{i}" in exclude or name in exclude:
                continue
            child.compile(**spec)
    return model
