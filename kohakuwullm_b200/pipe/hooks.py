"""Callback protocol of the pipeline trainer: Lightning-named hooks, dispatched to a list.

Calling a hook name that does not exist raises (a typo must not turn into a silent no-op).
Reference: src/kohakuwupipe/training/hooks.py:11-127.
"""

from __future__ import annotations

HOOKS = (
    "setup", "teardown", "on_fit_start", "on_fit_end", "on_train_start", "on_train_end",
    "on_train_epoch_start", "on_train_epoch_end", "on_train_batch_start", "on_train_batch_end",
    "on_before_backward", "on_after_backward", "on_before_optimizer_step", "on_before_zero_grad",
    "on_validation_start", "on_validation_end", "on_validation_batch_start", "on_validation_batch_end",
    "on_save_checkpoint", "on_load_checkpoint", "on_exception", "state_dict", "load_state_dict",
)


class Callback:
    """Base class: every hook is a no-op; ``state_dict`` returns ``{}``."""

    def state_dict(self) -> dict:
        return {}

    def load_state_dict(self, state: dict) -> None:
        pass


def _noop(self, *args, **kwargs):
    return None


for _name in HOOKS:
    if not hasattr(Callback, _name):
        setattr(Callback, _name, _noop)


class CallbackList:
    def __init__(self, callbacks=()):
        self.callbacks = list(callbacks)

    def call(self, hook: str, *args, **kwargs) -> list:
        if hook not in HOOKS:
            raise AttributeError(f"unknown hook {hook!r}; known hooks: {', '.join(HOOKS)}")
        return [getattr(cb, hook)(*args, **kwargs) for cb in self.callbacks]

    def __getattr__(self, hook: str):
        if hook in HOOKS:
            return lambda *a, **k: self.call(hook, *a, **k)
        raise AttributeError(f"unknown hook {hook!r}; known hooks: {', '.join(HOOKS)}")

    def state_dict(self) -> dict:
        return {f"{type(cb).__name__}:{i}": cb.state_dict() for i, cb in enumerate(self.callbacks)}

    def load_state_dict(self, state: dict) -> None:
        for i, cb in enumerate(self.callbacks):
            key = f"{type(cb).__name__}:{i}"
            if key in state:
                cb.load_state_dict(state[key])
