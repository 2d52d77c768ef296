"""Run state that a checkpoint carries besides weights and optimizer state: global token / FLOP totals,
elapsed time, EMA loss, RNG states (python, numpy, torch, cuda) and the loader position. Everything is
encoded as tensors / plain containers so the file loads with ``weights_only=True``.
Reference: src/kohakuwullm/training/loop/resume.py:13-76, trainer.py:329-401."""

from __future__ import annotations

import pickle
import random

import numpy as np
import torch

RESUME_KEY = "kohakuwullm"


def capture_rng() -> dict:
    state = {"python": torch.tensor(list(pickle.dumps(random.getstate())), dtype=torch.uint8),
             "numpy": torch.tensor(list(pickle.dumps(np.random.get_state())), dtype=torch.uint8),
             "torch": torch.get_rng_state()}
    if torch.cuda.is_available():
        state["cuda"] = torch.cuda.get_rng_state_all()
    return state


def restore_rng(state: dict) -> None:
    random.setstate(pickle.loads(bytes(state["python"].tolist())))  # noqa: S301  own checkpoint
    np.random.set_state(pickle.loads(bytes(state["numpy"].tolist())))  # noqa: S301
    torch.set_rng_state(state["torch"])
    if "cuda" in state and torch.cuda.is_available() and len(state["cuda"]) == torch.cuda.device_count():
        torch.cuda.set_rng_state_all(state["cuda"])


def pack_state(snapshot, ema_loss, loader_state, global_step: int) -> dict:
    return {"seen": snapshot.seen, "trained": snapshot.trained, "model_flops": snapshot.model_flops,
            "hardware_flops": snapshot.hardware_flops, "elapsed": snapshot.elapsed, "ema_loss": ema_loss,
            "rng": capture_rng(), "loader": loader_state, "global_step": global_step}


def unpack_state(state: dict):
    from kohakuwullm_b200.training.loop.tokens import TokenSnapshot

    snap = TokenSnapshot(int(state["seen"]), int(state["trained"]), float(state["model_flops"]),
                         float(state["hardware_flops"]), float(state["elapsed"]))
    return snap, state.get("ema_loss"), state.get("loader"), int(state.get("global_step", 0))
