"""Language-model callbacks for the pipeline trainer (the trainer itself knows nothing about tokens).

``RouterBiasSchedule`` scales every router's aux-loss-free bias update rate by a schedule factor of the
step: the factor multiplies the rate the routers were BUILT with (no compounding), a factor of zero
freezes the biases while the load statistics keep reporting, and a resumed run re-applies the factor of
the restored step.

``SamplePreview`` generates completions every N steps and hands them to a ``report(step, rows)`` function
on rank 0. It is collective: by default the stages' weights are gathered under whole-model names, rank 0
rebuilds the full model and decodes locally (one gather per preview, no per-token pipeline traffic); with
``local=False`` every rank drives a pipelined forward-only decode instead. Prompts are fixed
``(name, text)`` pairs and, with ``from_batch``, documents cut out of the batch that was just trained on.
Reference behaviour: src/kohakuwullm/training/parallel/uwupipe_callbacks.py:32-337.
"""

from __future__ import annotations

from typing import Callable, Sequence

import torch
import torch.distributed as dist

from kohakuwullm_b200.data.preview import prompts_from_batch
from kohakuwullm_b200.pipe.hooks import Callback
from kohakuwullm_b200.utils.schedule import build_schedule


def _routers(module) -> list:
    found = []
    for stage in getattr(module, "stages", [module]):
        for m in stage.modules():
            if hasattr(m, "bias_update_rate") and hasattr(m, "expert_bias"):
                found.append(m)
    return found


from kohakuwullm_b200.utils.logging import get_logger  # noqa: E402

_log = get_logger("preview")


class RouterBiasSchedule(Callback):
    def __init__(self, module, schedule: dict | Callable[[int], float]):
        self.module = module
        self.schedule = schedule if callable(schedule) else build_schedule(dict(schedule))
        self.base: list[float] | None = None
        self.factor = 1.0

    def apply(self, step: int) -> None:
        if self.base is None:
            return
        self.factor = float(self.schedule(step))
        for router, base in zip(_routers(self.module), self.base):
            router.bias_update_rate = base * self.factor

    def on_train_start(self, loop) -> None:
        self.base = [r.bias_update_rate for r in _routers(self.module)]
        self.apply(getattr(loop, "global_step", 0))

    def on_train_batch_end(self, loop, out=None, batch=None, batch_idx: int = 0) -> None:
        self.apply(getattr(out, "index", getattr(loop, "global_step", 0)))

    def state_dict(self) -> dict:
        return {"base": self.base}

    def load_state_dict(self, state: dict) -> None:
        if state.get("base") is not None:
            self.base = list(state["base"])


class SamplePreview(Callback):
    def __init__(self, module, tokenizer, prompts: Sequence[tuple[str, str]] = (), *, every_n_steps: int = 1000,
                 at_start: bool = True, samples: int = 4, report: Callable | None = None,
                 max_new_tokens: int = 64, temperature: float = 0.35, top_p: float = 0.95, top_k: int = 0,
                 min_p: float = 0.0, local: bool = True, from_batch: int = 0, prefix_frac: float = 0.25,
                 prefix_tokens: int = 768, turns_only: bool = True, stop_ids: Sequence[int] = (), group=None):
        self.module, self.tokenizer = module, tokenizer
        self.prompts = list(prompts)
        self.every, self.at_start, self.samples = every_n_steps, at_start, samples
        self.report = report
        self.sampling = dict(temperature=temperature, top_p=top_p, top_k=top_k, min_p=min_p)
        self.max_new_tokens = max_new_tokens
        self.local, self.from_batch = local, from_batch
        self.prefix_frac, self.prefix_tokens, self.turns_only = prefix_frac, prefix_tokens, turns_only
        self.stop_ids = tuple(stop_ids)
        self.group = group
        self.history: list[tuple[int, list]] = []

    # ------------------------------------------------------------------ helpers
    def _rank(self) -> int:
        return dist.get_rank(self.group) if dist.is_available() and dist.is_initialized() else 0

    def _encode(self, text: str) -> torch.Tensor:
        ids = self.tokenizer(text) if callable(self.tokenizer) else self.tokenizer.encode(text)
        if isinstance(ids, dict):
            ids = ids["input_ids"]
        return torch.as_tensor(list(ids), dtype=torch.long)

    def _full_model(self):
        """Whole model on rank 0 from the stages' gathered weights (None elsewhere). Collective."""
        from kohakuwullm_b200.models import LMBackbone
        from kohakuwullm_b200.pipe.checkpoint import gather_state_dict

        module = self.module
        if not hasattr(module, "stages"):
            return module if self._rank() == 0 else None     # a plain backbone: nothing to gather
        merged: dict = {}
        for stage in module.stages:
            merged.update(gather_state_dict(stage, stage.global_names(), group=self.group))
        if self._rank() != 0:
            return None
        device = module.device
        with torch.device(device):
            full = LMBackbone(module.config.replace(mxfp8=False), init=False)
        dtype = next(iter(module.stages[0].parameters())).dtype
        full.to(dtype)
        full.load_state_dict({k: v.to(device) for k, v in merged.items()}, strict=False)
        return full.eval()

    def _decode_rows(self, model, named_prompts):
        from kohakuwullm_b200.generation.engine import LocalGenerator

        gen = LocalGenerator(model, eos_id=getattr(self.tokenizer, "eos_id", 0), stop_ids=self.stop_ids)
        device = next(model.parameters()).device
        rows = []
        for name, ids in named_prompts:
            prompt = ids.to(device)[None, :].expand(self.samples, -1).contiguous()
            out = gen.generate(prompt, self.max_new_tokens, **self.sampling)
            for i in range(self.samples):
                new = out[i, ids.numel():].tolist()
                text = self.tokenizer.decode(new) if hasattr(self.tokenizer, "decode") else str(new)
                prompt_text = self.tokenizer.decode(ids.tolist()) if hasattr(self.tokenizer, "decode") else ""
                rows.append((name, prompt_text, i, text))
        return rows

    def preview(self, step: int, batch=None, silent: bool = False):
        named = [(n, self._encode(t)) for n, t in self.prompts]
        if self.from_batch and batch is not None:
            # the fixed prompts stay comparable from preview to preview; the batch prompts show the current data
            named = named + prompts_from_batch(batch, self.from_batch, seed=step, prefix_frac=self.prefix_frac,
                                               prefix_tokens=self.prefix_tokens, turns_only=self.turns_only)
        if not named:
            return []
        if self.local:
            model = self._full_model()
            rows = self._decode_rows(model, named) if model is not None else []
        else:
            from kohakuwullm_b200.generation.engine import PipelineGenerator

            world = dist.get_world_size(self.group) if dist.is_available() and dist.is_initialized() else 1
            gen = PipelineGenerator(self.module.stages[0], self._rank(), world, group=self.group)
            rows = []
            for name, ids in named:
                out = gen.generate(ids.to(self.module.device)[None, :].expand(self.samples, -1).contiguous(),
                                   self.max_new_tokens, **self.sampling)
                if self._rank() == 0:
                    for i in range(self.samples):
                        rows.append((name, "", i, self.tokenizer.decode(out[i, ids.numel():].tolist())))
        if self._rank() == 0 and not silent:
            self.history.append((step, rows))
            for name, prompt_text, i, text in rows:
                _log.info("sample", step=step, name=name, n=i, prompt=prompt_text[:40].replace("\n", "\\n"),
                          text=text[:200].replace("\n", "\\n"))
            if self.report is not None:
                self.report(step, rows)
        return rows

    # ------------------------------------------------------------------ hooks
    def on_train_start(self, loop) -> None:
        if self.at_start and self.every:
            # a decode path that is broken should say so now, not at the first real preview
            saved, self.prompts = self.prompts, [("validate", "hello")]
            keep_new, self.max_new_tokens = self.max_new_tokens, min(self.max_new_tokens, 8)
            try:
                self.preview(getattr(loop, "global_step", 0), silent=True)
            finally:
                self.prompts, self.max_new_tokens = saved, keep_new

    def on_train_batch_end(self, loop, out=None, batch=None, batch_idx: int = 0) -> None:
        step = getattr(out, "index", getattr(loop, "global_step", 0))
        if self.every and step > 0 and step % self.every == 0:
            self.preview(step, batch)
