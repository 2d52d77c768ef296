"""Text generation: sampling filters, single-process and pipelined generators.

Sampling is done in fp32 with the filters applied in the order top-k -> top-p -> min-p, greedy when
``temperature <= 0``; the generator owns a private per-device RNG (``SAMPLE_SEED``) so sampling never
perturbs the training RNG stream. Rows that have emitted a stop id keep emitting EOS.
``LocalGenerator`` decodes with a static KV cache (``use_cache=False`` recomputes the whole prefix each
step: the reference path used by the equivalence tests). ``PipelineGenerator`` decodes through the stages
of a pipeline: rank 0 embeds and runs its blocks, every rank forwards the ``(rows, S, dim)`` hidden state
to the next with NCCL send/recv, the last rank samples and broadcasts the next token. With
``microbatches=m`` the rows are cut into m chunks, each with a KV cache of its own on every stage, and one
decode step runs the chunks through the stages as a forward-only GPipe wave (sends are asynchronous, so stage
s works on chunk c + 1 while stage s + 1 works on chunk c); the last stage samples all rows at once, so the
tokens do not depend on m. ``max_new_tokens=None`` decodes until every row has stopped or the context is full.
Reference: src/kohakuwullm/generation/engine.py:19-385.
"""

from __future__ import annotations

from typing import Sequence

import torch
import torch.distributed as dist

from kohakuwullm_b200.models.cache import KVCache
from kohakuwullm_b200.models.seqinfo import SeqInfo

SAMPLE_SEED = 20090220


def filter_top_k(logits: torch.Tensor, k: int) -> torch.Tensor:
    if k <= 0 or k >= logits.shape[-1]:
        return logits
    kth = logits.topk(k, dim=-1).values[..., -1:]
    return logits.masked_fill(logits < kth, float("-inf"))


def filter_top_p(logits: torch.Tensor, p: float) -> torch.Tensor:
    if p >= 1.0:
        return logits
    sorted_logits, order = logits.sort(dim=-1, descending=True)
    probs = sorted_logits.softmax(-1)
    cum = probs.cumsum(-1)
    drop = (cum - probs) >= p           # keep the token that crosses the threshold
    sorted_logits = sorted_logits.masked_fill(drop, float("-inf"))
    return torch.full_like(logits, float("-inf")).scatter(-1, order, sorted_logits)


def filter_min_p(logits: torch.Tensor, min_p: float) -> torch.Tensor:
    if min_p <= 0.0:
        return logits
    probs = logits.softmax(-1)
    floor = probs.max(-1, keepdim=True).values * min_p
    return logits.masked_fill(probs < floor, float("-inf"))


def sample(logits: torch.Tensor, temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0,
           min_p: float = 0.0, generator: torch.Generator | None = None) -> torch.Tensor:
    """logits (rows, vocab) -> next ids (rows,)."""
    logits = logits.float()
    if not torch.isfinite(logits).any(-1).all():
        raise FloatingPointError("non-finite logits reached the sampler")
    if temperature <= 0:
        return logits.argmax(-1)
    logits = logits / temperature
    logits = filter_min_p(filter_top_p(filter_top_k(logits, top_k), top_p), min_p)
    return torch.multinomial(logits.softmax(-1), 1, generator=generator).squeeze(-1)


def token_budget(max_new_tokens: int | None, prompt_len: int, max_position: int) -> int:
    """New tokens to decode: the request, cut to what the model's context still holds (None: all of it)."""
    room = max(int(max_position) - int(prompt_len), 0)
    if max_new_tokens is None:
        return room
    # an explicit request is honoured up to the context; a prompt that already fills the context keeps the request
    # (rotary positions extrapolate; the caller asked for it)
    return min(int(max_new_tokens), room) if room else int(max_new_tokens)


def advance(tokens: torch.Tensor, nxt: torch.Tensor, finished: torch.Tensor, stop_ids: Sequence[int], eos: int):
    """Append ``nxt``; rows that already finished are held at EOS. Returns (tokens, finished)."""
    nxt = torch.where(finished, torch.full_like(nxt, eos), nxt)
    hit = torch.zeros_like(finished)
    for s in stop_ids:
        hit |= nxt == s
    return torch.cat([tokens, nxt[:, None]], dim=1), finished | hit


class LocalGenerator:
    def __init__(self, backbone, eos_id: int = 0, stop_ids: Sequence[int] = (), use_cache: bool = True,
                 static_cache: bool = True):
        self.backbone, self.eos = backbone, eos_id
        self.stop_ids = tuple(stop_ids) or (eos_id,)
        self.use_cache, self.static_cache = use_cache, static_cache
        self._rng: dict[str, torch.Generator] = {}

    def rng(self, device) -> torch.Generator:
        key = str(device)
        if key not in self._rng:
            self._rng[key] = torch.Generator(device=device).manual_seed(SAMPLE_SEED)
        return self._rng[key]

    @torch.no_grad()
    def generate(self, prompt: torch.Tensor, max_new_tokens: int | None = 128, **sampling) -> torch.Tensor:
        """prompt (rows, S) of equal-length rows -> (rows, S + new). ``max_new_tokens=None``: until every row has
        stopped or the context is full."""
        bb = self.backbone
        max_new_tokens = token_budget(max_new_tokens, prompt.shape[1], getattr(bb.config, "max_position", 1 << 30))
        was_training = bb.training
        bb.eval()
        tokens = prompt
        rows, S = prompt.shape
        finished = torch.zeros(rows, dtype=torch.bool, device=prompt.device)
        gen = self.rng(prompt.device)
        cache = KVCache.from_config(bb.config, S + max_new_tokens, static=self.static_cache) if self.use_cache else None
        step_in = prompt
        for _ in range(max_new_tokens):
            if cache is not None:
                hidden = bb(step_in, cache.seq_info(step_in), cache=cache)
            else:
                hidden = bb(tokens, SeqInfo.padded(rows, tokens.shape[1], device=tokens.device))
            logits = bb.head.logits(hidden[:, -1])
            nxt = sample(logits, generator=gen, **sampling)
            tokens, finished = advance(tokens, nxt, finished, self.stop_ids, self.eos)
            step_in = tokens[:, -1:]
            if bool(finished.all()):
                break
        bb.train(was_training)
        return tokens


class PipelineGenerator:
    """Forward-only pipelined decode over ``LMStage`` slices: one KV cache per stage and micro-batch."""

    def __init__(self, stage, rank: int, world: int, eos_id: int = 0, stop_ids: Sequence[int] = (), group=None,
                 microbatches: int | None = None):
        self.stage, self.rank, self.world, self.group = stage, rank, world, group
        self.eos = eos_id
        self.stop_ids = tuple(stop_ids) or (eos_id,)
        self.microbatches = microbatches
        self._gen: torch.Generator | None = None

    def _forward(self, step_in, cache, rows, S, device, dtype, pending):
        """One chunk through this rank's blocks. Returns the last stage's logits of the final position."""
        stage = self.stage
        info = cache.seq_info(torch.empty(rows, S, device=device))
        if stage.is_first:
            x = stage.embed(step_in)
            if stage.embed_scale != 1.0:
                x = x * stage.embed_scale
        else:
            x = torch.empty(rows, S, stage.config.dim, device=device, dtype=dtype)
            dist.recv(x, src=self.rank - 1, group=self.group)
        rope = stage.pos_enc.prepare(info.position_ids)
        for i, blk in enumerate(stage.blocks):
            x = blk(x, info, rope, cache=cache, layer=i)
        cache.advance()
        if stage.is_last:
            return stage.head.logits(stage.final_norm(x)[:, -1])
        x = x.contiguous()
        # asynchronous: this rank goes on with its next chunk while the next stage takes this one
        pending.append((dist.isend(x, dst=self.rank + 1, group=self.group), x))
        return None

    @torch.no_grad()
    def generate(self, prompt: torch.Tensor, max_new_tokens: int | None = 128, **sampling) -> torch.Tensor:
        stage = self.stage
        stage.eval()
        device = prompt.device
        dtype = next(p for p in stage.parameters() if p.dim() >= 2).dtype
        rows, S = prompt.shape
        chunks = self.microbatches or 1
        if rows % chunks:
            raise ValueError(f"{rows} rows do not split into {chunks} micro-batches")
        per = rows // chunks
        budget = token_budget(max_new_tokens, S, getattr(stage.config, "max_position", S + (max_new_tokens or 0)))
        caches = [KVCache(len(stage.blocks), S + budget, static=True) for _ in range(chunks)]
        if self._gen is None:
            self._gen = torch.Generator(device=device).manual_seed(SAMPLE_SEED)
        tokens = prompt
        finished = torch.zeros(rows, dtype=torch.bool, device=device)
        step_in = prompt
        last = self.world - 1
        for _ in range(budget):
            pending: list = []
            logits = [self._forward(step_in[c * per:(c + 1) * per], caches[c], per, step_in.shape[1], device, dtype,
                                    pending) for c in range(chunks)]
            for work, _buf in pending:
                work.wait()
            # all rows are sampled in one call: the random stream is consumed as without micro-batches
            nxt = sample(torch.cat(logits), generator=self._gen, **sampling) if self.rank == last else \
                torch.empty(rows, dtype=torch.long, device=device)
            if self.world > 1:
                dist.broadcast(nxt, src=last, group=self.group)
            tokens, finished = advance(tokens, nxt, finished, self.stop_ids, self.eos)
            step_in = tokens[:, -1:]
            if bool(finished.all()):
                break
        return tokens


def build_generator(model, **kw):
    """``LMBackbone`` -> ``LocalGenerator``; an ``LMStage`` needs ``rank`` and ``world`` -> ``PipelineGenerator``."""
    if hasattr(model, "plan"):
        return PipelineGenerator(model, **kw)
    return LocalGenerator(model, **kw)
