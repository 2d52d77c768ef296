"""Parameter census of a ladder of presets, MEASURED on models built on the meta device (no memory): total and
active parameters, embedding / head / router counts and the analytic FLOPs per token beside them.
Reference: src/kohakuwullm/bench/model/ladder.py:1-115."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from kohakuwullm_b200.bench.flops_analytic import flop_budget
from kohakuwullm_b200.models import LMBackbone, get_preset
from kohakuwullm_b200.models.presets import KOHAKU_LADDER
from kohakuwullm_b200.utils.misc import count_active_parameters, count_parameters, human_count


@dataclass(frozen=True)
class RungCensus:
    name: str
    dim: int
    depth: int
    heads: int
    kv_heads: int
    num_experts: int
    top_k: int
    total: int
    active: int
    embedding: int
    head: int
    router: int
    train_flops_per_token: float

    @property
    def sparse(self) -> bool:
        return self.num_experts > 0

    @property
    def compute_active(self) -> int:
        """Active parameters that do arithmetic: the embedding table is a gather, the head is a GEMM."""
        return self.active - self.embedding


def census(name: str, **overrides) -> RungCensus:
    cfg = get_preset(name, mxfp8=False, **overrides)
    with torch.device("meta"):
        model = LMBackbone(cfg)
    embedding = model.embed.weight.numel()
    head = 0 if model.head.tied else model.head.weight.numel()
    router = sum(p.numel() for n, p in model.named_parameters() if ".router." in n)
    budget = flop_budget(cfg)
    sparse = any(cfg.moe_layers)
    return RungCensus(name, cfg.dim, cfg.depth, cfg.heads, cfg.kv_heads, cfg.moe_num_experts if sparse else 0,
                      cfg.moe_top_k if sparse else 0, count_parameters(model), count_active_parameters(model),
                      embedding, head, router, budget.total)


def ladder(names=KOHAKU_LADDER) -> list[RungCensus]:
    return [census(n) for n in names]


def render(rows: list[RungCensus]) -> str:
    lines = ["| preset | dim | depth | heads/kv | experts (top-k) | total | active | compute-active | GFLOP/token (train) |",
             "|---|---|---|---|---|---|---|---|---|"]
    for r in rows:
        experts = f"{r.num_experts} ({r.top_k})" if r.sparse else "-"
        lines.append(f"| {r.name} | {r.dim} | {r.depth} | {r.heads}/{r.kv_heads} | {experts} | {human_count(r.total)} | "
                     f"{human_count(r.active)} | {human_count(r.compute_active)} | {r.train_flops_per_token / 1e9:.2f} |")
    return "\n".join(lines)


if __name__ == "__main__":
    print(render(ladder()))
