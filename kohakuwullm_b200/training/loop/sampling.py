"""Sampler of the in-training previews: one generator object for the life of the trainer, handed the backbone at
each call. It decodes with the key-value cache and draws from a random stream of its own (seeded once with
``SAMPLE_SEED``), so a preview neither disturbs the training stream (dropout, data order) nor repeats the previous
preview's draws. ``texts`` is the whole preview in one call: prompts in, decoded continuations out.
Reference: src/kohakuwullm/training/loop/sampling.py:12-24."""

from __future__ import annotations

from typing import Sequence

import torch

from kohakuwullm_b200.generation.engine import SAMPLE_SEED, LocalGenerator


class PreviewSampler(LocalGenerator):
    def __init__(self, seed: int = SAMPLE_SEED, eos_id: int = 0, use_cache: bool = True, static_cache: bool = True):
        super().__init__(None, eos_id=eos_id, use_cache=use_cache, static_cache=static_cache)
        self.seed = seed

    def rng(self, device) -> torch.Generator:
        key = str(device)
        if key not in self._rng:
            self._rng[key] = torch.Generator(device=device).manual_seed(self.seed)
        return self._rng[key]

    def generate(self, backbone, prompt_ids: torch.Tensor, max_new_tokens: int | None = 64, **sampling) -> torch.Tensor:
        """``(rows, S)`` prompt ids -> ``(rows, S + new)``; the sampling arguments are ``LocalGenerator.generate``'s."""
        self.backbone = backbone
        try:
            return super().generate(prompt_ids, max_new_tokens, **sampling)
        finally:
            self.backbone = None      # the sampler must not keep a stage or a replaced model alive

    def texts(self, backbone, tokenizer, prompts: Sequence[str], max_new_tokens: int | None = 64, count: int = 1,
              **sampling) -> list[list[str]]:
        """``count`` continuations per prompt as text (the prompt itself is not repeated in the result)."""
        device = next(backbone.parameters()).device
        bos = getattr(tokenizer, "bos_token_id", None)
        out = []
        for prompt in prompts:
            ids = ([bos] if bos is not None else []) + list(tokenizer.encode(prompt))
            rows = torch.tensor([ids or [self.eos]] * count, device=device)
            done = self.generate(backbone, rows, max_new_tokens, **sampling)
            out.append([tokenizer.decode(r[len(ids):]) for r in done.tolist()])
        return out
