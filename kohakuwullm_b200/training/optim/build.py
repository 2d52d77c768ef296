"""Parameter grouping and the optimizer factory.

Grouping rules (reference: src/kohakuwullm/training/optim/build.py:17-167):
  * weight decay only on tensors with >= 2 dims that are not a router's ``expert_bias`` / sink logits;
  * the input embedding (a path component ``embed``) never decays unless ``decay_embeddings``;
  * optional ``embed_lr`` group; optional muP groups (``lr * base/fan_in``, ``wd / scale``);
  * Muon takes the hidden matrices (>= 2-D, not under ``embed`` / ``head`` / ``router``); everything else
    goes to its internal AdamW.
``build_optimizer(model, name=...)`` knows ``adamw adam sgd fused_adamw adamw16 muon stochastic_adamw``.
"""

from __future__ import annotations

import torch
from torch import nn

from kohakuwullm_b200.registry import OPTIMIZER
from kohakuwullm_b200.training.optim.adamw16 import AdamW16
from kohakuwullm_b200.training.optim.lowbit_optim import StochasticAdamW
from kohakuwullm_b200.training.optim.muon import MuonW
from kohakuwullm_b200.training.optim.quantized_state import QuantizedStateAdamW
from kohakuwullm_b200.training.optim.torch_fused import FusedAdamW


def is_decay_param(name: str, p: nn.Parameter) -> bool:
    return p.dim() >= 2 and "expert_bias" not in name and not name.endswith("sink")


def is_embedding(name: str) -> bool:
    return "embed" in name.split(".")


def is_hidden_matrix(name: str, p: nn.Parameter) -> bool:
    parts = name.split(".")
    return p.dim() >= 2 and not any(k in parts for k in ("embed", "head", "router"))


def group_parameters(model: nn.Module, weight_decay: float = 0.1, decay_embeddings: bool = False,
                     embed_lr: float | None = None, lr: float = 3e-4, mup_base_dim: int | None = None) -> list[dict]:
    decay, no_decay, embed, mup = [], [], [], {}
    for name, p in model.named_parameters():
        if not p.requires_grad:
            continue
        if is_embedding(name):
            (embed if embed_lr is not None else (decay if decay_embeddings else no_decay)).append(p)
        elif mup_base_dim and is_hidden_matrix(name, p):
            mup.setdefault(p.shape[-1], []).append(p)
        elif is_decay_param(name, p):
            decay.append(p)
        else:
            no_decay.append(p)
    groups = []
    if decay:
        groups.append({"params": decay, "weight_decay": weight_decay})
    if no_decay:
        groups.append({"params": no_decay, "weight_decay": 0.0})
    if embed:
        groups.append({"params": embed, "weight_decay": weight_decay if decay_embeddings else 0.0, "lr": embed_lr})
    for fan_in, ps in sorted(mup.items()):
        scale = mup_base_dim / fan_in
        groups.append({"params": ps, "lr": lr * scale, "weight_decay": weight_decay / scale})
    return groups


def muon_groups(model: nn.Module, lr: float, muon_lr: float, weight_decay: float, embed_lr: float | None = None):
    """Hidden matrices for the orthogonalised step; the rest for the internal AdamW in up to three groups: decayed,
    undecayed, and (with ``embed_lr``) the token-indexed tables (embedding, head) at a rate of their own."""
    hidden, rest_decay, rest_plain, tables = [], [], [], []
    for name, p in model.named_parameters():
        if not p.requires_grad:
            continue
        if is_hidden_matrix(name, p):
            hidden.append(p)
        elif embed_lr is not None and p.dim() >= 2 and (is_embedding(name) or "head" in name.split(".")):
            tables.append(p)
        elif is_decay_param(name, p) and not is_embedding(name):
            rest_decay.append(p)
        else:
            rest_plain.append(p)
    groups = [{"params": rest_decay, "weight_decay": weight_decay}, {"params": rest_plain, "weight_decay": 0.0}]
    if tables:
        groups.append({"params": tables, "weight_decay": 0.0, "lr": embed_lr})
    return hidden, groups


OPTIMIZER.register("adamw", lambda groups, **kw: torch.optim.AdamW(groups, foreach=True, **kw))
OPTIMIZER.register("adam", lambda groups, **kw: torch.optim.Adam(groups, foreach=True, **kw))
OPTIMIZER.register("sgd", lambda groups, **kw: torch.optim.SGD(groups, **kw))
OPTIMIZER.register("fused_adamw", FusedAdamW)
OPTIMIZER.register("adamw16", AdamW16)
OPTIMIZER.register("stochastic_adamw", StochasticAdamW)
# AdamW with quantised moments (the reference takes these three names from an optional package)
for _name, _fmt in (("adamw8bit", "int8"), ("adamw4bit", "int4"), ("adamwfp8", "fp8")):
    OPTIMIZER.register(_name, (lambda fmt: lambda groups, **kw: QuantizedStateAdamW(groups, state_format=fmt, **kw))(_fmt))


def build_optimizer(model: nn.Module, name: str = "fused_adamw", lr: float = 3e-4, weight_decay: float = 0.1,
                    betas=(0.9, 0.95), decay_embeddings: bool = False, embed_lr: float | None = None,
                    mup_base_dim: int | None = None, muon_lr: float | None = None, **kw):
    if name == "muon":
        muon_lr = muon_lr or 0.02
        hidden, rest = muon_groups(model, lr, muon_lr, weight_decay, embed_lr)
        return MuonW(hidden, rest, lr=lr, muon_lr=muon_lr, weight_decay=weight_decay, betas=betas, **kw)
    groups = group_parameters(model, weight_decay, decay_embeddings, embed_lr, lr, mup_base_dim)
    if name == "sgd":
        return OPTIMIZER.get(name)(groups, lr=lr, **kw)
    return OPTIMIZER.get(name)(groups, lr=lr, betas=betas, **kw)


class MainGradOptimizer:
    """Drives an optimizer that reads ``p.grad`` from parameters whose gradients live in flat fp32 ``main_grad``
    buffers (``parallel/flat.py``): ``step`` hands every parameter its gradient (cast to the parameter's dtype for
    16-bit parameters), steps, and clears the flat buffers. ``flat`` is exposed so that the training loops find the
    gradient buffers for the global norm and scale them in place before the step."""

    def __init__(self, optimizer: torch.optim.Optimizer, flat, module: nn.Module):
        self.inner, self.flat, self.module = optimizer, flat, module

    @property
    def param_groups(self):
        return self.inner.param_groups

    @property
    def state(self):
        return self.inner.state

    @torch.no_grad()
    def step(self, closure=None):
        params = [p for p in self.module.parameters() if p.requires_grad and hasattr(p, "main_grad")]
        for p in params:
            g = p.main_grad
            p.grad = g if g.dtype == p.dtype else g.to(p.dtype)
        out = self.inner.step(closure)
        for p in params:
            p.grad = None
        self.flat.zero_grad()
        return out

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.flat.zero_grad()

    def state_dict(self):
        return self.inner.state_dict()

    def load_state_dict(self, sd):
        return self.inner.load_state_dict(sd)
