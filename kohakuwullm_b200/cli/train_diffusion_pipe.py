"""Flow-matching diffusion trained on the pipeline engine: the second user of ``kohakuwullm_b200.pipe``, which
shows that the engine knows nothing about language models.

    torchrun --nproc-per-node 2 -m kohakuwullm_b200.cli.train_diffusion_pipe --set MAX_STEPS=50
    python -m kohakuwullm_b200.cli.train_diffusion_pipe --set BACKEND=gloo      # one process, one stage

What differs from the LM adapter and is exercised here: the first stage takes TWO inputs prepared on the fly
(the noised sample and its time), TWO tensors cross every stage boundary (hidden state and time embedding),
the target is a STRUCTURE (``{"velocity", "weight"}``) that never leaves the last rank, the loss is a weighted
mean-squared error normalised by the number of samples of the step, and validation runs the stages forward
only. Model: a residual MLP with adaptive (time-conditioned) layer scaling; data: a fixed mixture of Gaussians.
Objective: with ``x_t = (1 - t) x_0 + t eps`` the network predicts the velocity ``eps - x_0``.
Reference: scripts/train/diffusion_pipe.py:1-515.
"""

from __future__ import annotations

import math
import sys
from dataclasses import dataclass

import torch
from torch import nn

DIM = 256
DEPTH = 8
DATA_DIM = 32
BATCH = 256
NUM_MICROBATCHES = 4
SCHEDULE = "1f1b"
LR = 1e-3
WEIGHT_DECAY = 0.0
GRAD_CLIP = 1.0
MAX_STEPS = 200
VAL_EVERY = 50
LOG_INTERVAL = 10
SEED = 1234
BACKEND: str | None = None
CKPT_DIR = ""


@dataclass
class DiffusionStep:
    """One optimizer step: ``NUM_MICROBATCHES`` micro-batches of clean samples (every rank draws the same)."""

    clean: list


class TimeEmbedding(nn.Module):
    def __init__(self, dim: int):
        super().__init__()
        self.dim = dim
        self.mlp = nn.Sequential(nn.Linear(dim, dim), nn.SiLU(), nn.Linear(dim, dim))

    def forward(self, t: torch.Tensor) -> torch.Tensor:
        half = self.dim // 2
        freqs = torch.exp(-math.log(1000.0) * torch.arange(half, device=t.device) / half)
        ang = t[:, None] * 1000.0 * freqs[None]
        return self.mlp(torch.cat([ang.sin(), ang.cos()], dim=-1))


class Block(nn.Module):
    """Residual MLP block whose normalised input is scaled and shifted by the time embedding."""

    def __init__(self, dim: int):
        super().__init__()
        self.norm = nn.LayerNorm(dim, elementwise_affine=False)
        self.mod = nn.Linear(dim, 2 * dim)
        self.ff = nn.Sequential(nn.Linear(dim, 4 * dim), nn.GELU(), nn.Linear(4 * dim, dim))
        nn.init.zeros_(self.mod.weight)
        nn.init.zeros_(self.mod.bias)

    def forward(self, x, temb):
        scale, shift = self.mod(temb).chunk(2, dim=-1)
        return x + self.ff(self.norm(x) * (1 + scale) + shift)


class DiffusionStage(nn.Module):
    def __init__(self, plan, dim: int, data_dim: int):
        super().__init__()
        self.plan = plan
        self.is_first, self.is_last = plan.is_first, plan.is_last
        if self.is_first:
            self.inp = nn.Linear(data_dim, dim)
            self.time = TimeEmbedding(dim)
        self.blocks = nn.ModuleList(Block(dim) for _ in range(plan.start_layer, plan.end_layer))
        if self.is_last:
            self.out = nn.Linear(dim, data_dim)
        self._inputs: list = []

    def set_inputs(self, inputs) -> None:
        self._inputs = list(inputs)

    def forward_micro(self, mb: int, *inputs):
        if self.is_first:
            noised, t = self._inputs[mb]
            x, temb = self.inp(noised), self.time(t)
        else:
            x, temb = inputs
        for blk in self.blocks:
            x = blk(x, temb)
        if self.is_last:
            return self.out(x)
        return x, temb

    def global_names(self) -> dict:
        out = {}
        for name, _ in list(self.named_parameters()) + list(self.named_buffers()):
            parts = name.split(".")
            if parts[0] == "blocks":
                parts[1] = str(int(parts[1]) + self.plan.start_layer)
            out[name] = ".".join(parts)
        return out


def sample_data(n: int, data_dim: int, gen: torch.Generator) -> torch.Tensor:
    """A fixed mixture of four Gaussians (what the model should learn to denoise towards)."""
    centres = torch.tensor([[2.0, 0.0], [-2.0, 0.0], [0.0, 2.0], [0.0, -2.0]]).repeat(1, data_dim // 2)
    which = torch.randint(0, 4, (n,), generator=gen)
    return centres[which] + 0.3 * torch.randn(n, data_dim, generator=gen)


def build_module(dim=DIM, depth=DEPTH, data_dim=DATA_DIM, micro_rows=BATCH // NUM_MICROBATCHES, lr=LR, seed=SEED):
    from kohakuwullm_b200.pipe.module import PipelineModule

    class DiffusionModule(PipelineModule):
        def __init__(self):
            super().__init__()
            self._targets: list = []
            self._gen = torch.Generator().manual_seed(seed + 1)

        def configure_model(self, plan, rank, world, device):
            torch.manual_seed(seed + plan.index)
            return DiffusionStage(plan, dim, data_dim).to(device)

        def configure_optimizers(self):
            params = [p for s in self.stages for p in s.parameters()]
            return torch.optim.AdamW(params, lr=lr, weight_decay=WEIGHT_DECAY)

        def boundary_example(self, plan):
            z = torch.zeros(micro_rows, dim, device=self.device)
            return (z, z.clone())

        def global_names(self):
            return self.stages[0].global_names()

        # -------------------------------------------------------------- per step
        def set_batch(self, batch: DiffusionStep) -> None:
            """Noise the clean samples on the fly (the same draw on every rank: one shared generator), give the
            first stage its two inputs and keep the structured target on the last."""
            inputs, targets = [], []
            for clean in batch.clean:
                t = torch.rand(clean.shape[0], generator=self._gen)
                eps = torch.randn(clean.shape, generator=self._gen)
                noised = (1 - t[:, None]) * clean + t[:, None] * eps
                inputs.append((noised.to(self.device), t.to(self.device)))
                targets.append({"velocity": (eps - clean).to(self.device),
                                "weight": (1.0 / (0.05 + t * (1 - t))).clamp(max=10.0).to(self.device)})
            for stage in self.stages:
                if stage.is_first:
                    stage.set_inputs(inputs)
            self._targets = targets

        def num_microbatches(self, batch) -> int:
            return len(batch.clean)

        def step_tokens(self, batch) -> int:
            return sum(c.shape[0] for c in batch.clean)       # the loss is a mean over samples

        def loss(self, output, micro_index: int) -> torch.Tensor:
            tgt = self._targets[micro_index]
            per_sample = ((output - tgt["velocity"]) ** 2).mean(dim=-1)
            self.log("mse", per_sample.mean())
            return (per_sample * tgt["weight"]).sum()

        def forward_backward(self, schedule, batch, n_micro):
            return schedule.step(n_micro)

    return DiffusionModule()


def stream(batch: int, n_micro: int, data_dim: int, seed: int):
    gen = torch.Generator().manual_seed(seed)
    while True:
        yield DiffusionStep([sample_data(batch // n_micro, data_dim, gen) for _ in range(n_micro)])


def main():
    from kohakuwullm_b200.pipe import LossLog, Throughput, describe, init_pipeline, plan_stages, shutdown
    from kohakuwullm_b200.pipe.trainer import PipelineTrainer
    from kohakuwullm_b200.utils.logging import get_logger

    log = get_logger("diffusion_pipe")
    ranks = init_pipeline(BACKEND)
    plans = plan_stages([1.0] * DEPTH, ranks.world_size, head_cost=0.2)
    log.info("plan", text="\n" + describe(plans))
    module = build_module()
    trainer = PipelineTrainer(module, plans, rank=ranks.rank, world=ranks.world_size, device=ranks.device,
                              n_micro=NUM_MICROBATCHES, schedule=SCHEDULE, max_grad_norm=GRAD_CLIP,
                              callbacks=[LossLog(LOG_INTERVAL), Throughput(LOG_INTERVAL)])
    outs = trainer.fit(stream(BATCH, NUM_MICROBATCHES, DATA_DIM, SEED), MAX_STEPS)
    if CKPT_DIR:
        import os

        trainer.save_checkpoint(os.path.join(CKPT_DIR, "last.ckpt"))
    if outs and ranks.rank == 0:
        log.info("done", first_loss=float(outs[0].loss), last_loss=float(outs[-1].loss))
    shutdown()
    return outs


if __name__ == "__main__":
    from kohakuwullm_b200.utils.config import configure

    configure(sys.modules[__name__], sys.argv[1:])
    main()
