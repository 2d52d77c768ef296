"""Measured stage costs for the pipeline split.

``measure_costs`` times forward + backward of ONE block per distinct layer kind — the key is
``(is_moe, attention backend, window)`` — at the real micro-batch size, dtype and MXFP8 setting, on a
ragged probe layout of ``doc_len``-token documents, plus the head (loss of final-normed hidden states)
and the embedding. Each figure is the median of ``repeats`` runs after ``warmup`` runs, synchronised on
both sides (CUDA events on the GPU). ``broadcast_costs`` ships rank 0's vector to every rank so all ranks
plan the same split. Reference: src/kohakuwullm/training/parallel/autotune.py:23-258.
"""

from __future__ import annotations

import statistics
import time
from dataclasses import dataclass

import torch
import torch.distributed as dist

from kohakuwullm_b200.models.backbone import build_block
from kohakuwullm_b200.models.head import LMHead
from kohakuwullm_b200.models.presets import LMArchConfig
from kohakuwullm_b200.models.seqinfo import SeqInfo
from kohakuwullm_b200.training.optim.lowbit import cast_parameters_


@dataclass
class LayerCosts:
    layers: list[float]
    embed: float
    head: float

    def to_tensor(self) -> torch.Tensor:
        return torch.tensor([*self.layers, self.embed, self.head], dtype=torch.float64)

    @classmethod
    def from_tensor(cls, t: torch.Tensor) -> "LayerCosts":
        vals = t.tolist()
        return cls(vals[:-2], vals[-2], vals[-1])


def layer_key(config: LMArchConfig, layer: int):
    spec = config.attn_for(layer)
    name = spec if isinstance(spec, str) else (spec.get("name") if isinstance(spec, dict) else repr(spec))
    return (config.moe_layers[layer], name, config.window_for(layer))


def _time_ms(fn, device, warmup: int, repeats: int) -> float:
    for _ in range(warmup):
        fn()
    samples = []
    for _ in range(repeats):
        if device.type == "cuda":
            torch.cuda.synchronize(device)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize(device)
            samples.append(s.elapsed_time(e))
        else:
            t0 = time.perf_counter()
            fn()
            samples.append((time.perf_counter() - t0) * 1e3)
    return statistics.median(samples)


def probe_layout(micro_tokens: int, doc_len: int, device) -> SeqInfo:
    lens = [doc_len] * (micro_tokens // doc_len)
    if micro_tokens % doc_len:
        lens.append(micro_tokens % doc_len)
    return SeqInfo.from_lengths(lens, device=device)


def measure_costs(config: LMArchConfig, micro_tokens: int, device, *, param_dtype=torch.bfloat16,
                  doc_len: int = 2048, warmup: int = 3, repeats: int = 8) -> LayerCosts:
    device = torch.device(device)
    info = probe_layout(micro_tokens, min(doc_len, micro_tokens), device)
    dtype = param_dtype if device.type == "cuda" else torch.float32
    from kohakuwullm_b200.models.components.posenc import RoPE  # noqa: F401  (registration)
    from kohakuwullm_b200.registry import POSENC, build

    posenc = build(config.posenc, POSENC, head_dim=config.head_dim, theta=config.rope_theta,
                   scaling=config.rope_scaling, factor=config.rope_factor, max_position=config.max_position,
                   partial=config.rope_partial).to(device)
    rope = posenc.prepare(info.position_ids)
    by_key: dict = {}
    for layer in range(config.depth):
        key = layer_key(config, layer)
        if key in by_key:
            continue
        torch.manual_seed(0)
        block = build_block(config, layer).to(device)
        for p in block.parameters():
            if p.dim() >= 2:
                torch.nn.init.normal_(p, std=config.init_std)
        if dtype != torch.float32:
            cast_parameters_(block, dtype)
        if config.mxfp8:
            from kohakuwullm_b200.models.mxfp8_swap import swap_mxfp8

            swap_mxfp8(block)
        x = torch.randn(micro_tokens, config.dim, device=device, dtype=dtype, requires_grad=True)

        def run(block=block, x=x):
            y = block(x, info, rope, layer=layer)
            y.float().sum().backward()
            x.grad = None

        by_key[key] = _time_ms(run, device, warmup, repeats)
        del block, x
    head = LMHead(config.dim, config.vocab_size, z_loss_weight=config.z_loss_weight).to(device)
    torch.nn.init.normal_(head.proj.weight, std=config.init_std)
    if dtype != torch.float32:
        cast_parameters_(head, dtype)
    h = torch.randn(micro_tokens, config.dim, device=device, dtype=dtype, requires_grad=True)
    labels = torch.randint(0, config.vocab_size, (micro_tokens,), device=device)

    def run_head():
        loss, _ = head.loss(h, labels, "sum")
        loss.backward()
        h.grad = None

    head_ms = _time_ms(run_head, device, warmup, repeats)
    emb = torch.nn.Embedding(config.vocab_size, config.dim, device=device, dtype=dtype)
    tokens = torch.randint(0, config.vocab_size, (micro_tokens,), device=device)

    def run_embed():
        emb(tokens).float().sum().backward()
        emb.weight.grad = None

    embed_ms = _time_ms(run_embed, device, warmup, repeats)
    return LayerCosts([by_key[layer_key(config, i)] for i in range(config.depth)], embed_ms, head_ms)


def broadcast_costs(costs: LayerCosts | None, depth: int, device, src: int = 0, group=None) -> LayerCosts:
    """Every rank gets rank ``src``'s measurements (fp64 vector of ``depth + 2`` numbers)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        assert costs is not None
        return costs
    t = costs.to_tensor() if costs is not None else torch.zeros(depth + 2, dtype=torch.float64)
    if dist.get_backend(group) == "nccl":
        t = t.to(device)
    dist.broadcast(t, src=src, group=group)
    return LayerCosts.from_tensor(t.cpu())
