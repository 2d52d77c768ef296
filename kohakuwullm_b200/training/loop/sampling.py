"""Sampler of the in-training previews: one generator object for the life of the trainer, handed the backbone at
each call. It decodes with the key-value cache and draws from a random stream of its own (seeded once with
``SAMPLE_SEED``), so a preview neither disturbs the training stream (dropout, data order) nor repeats the previous
preview's draws. Reference: src/kohakuwullm/training/loop/sampling.py:12-24."""

from __future__ import annotations

import torch

from kohakuwullm_b200.generation.engine import SAMPLE_SEED, LocalGenerator


class PreviewSampler(LocalGenerator):
    """``generate(backbone, prompt_ids, max_new_tokens, **sampling)``; the sampling arguments are
    ``LocalGenerator.generate``'s."""

    def __init__(self, seed: int = SAMPLE_SEED, eos_id: int = 0, use_cache: bool = True, static_cache: bool = True):
        super().__init__(None, eos_id=eos_id, use_cache=use_cache, static_cache=static_cache)
        self.seed = seed

    def rng(self, device) -> torch.Generator:
        key = str(device)
        if key not in self._rng:
            self._rng[key] = torch.Generator(device=device).manual_seed(self.seed)
        return self._rng[key]

    def generate(self, backbone, prompt_ids: torch.Tensor, max_new_tokens: int | None = 64, **sampling) -> torch.Tensor:
        self.backbone = backbone
        try:
            return super().generate(prompt_ids, max_new_tokens, **sampling)
        finally:
            self.backbone = None      # the sampler must not keep a stage or a replaced model alive
