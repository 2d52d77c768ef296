"""Config runner in the style of ``kogine run script.py --config file.py --set KEY=VALUE``.

A training script declares its knobs as UPPER_CASE module globals. A config is a Python file whose
UPPER_CASE globals (or the dict returned by its ``config_gen()``) overwrite the script's same-named
globals (names with a leading underscore are the config's own helpers and are ignored); ``--set KEY=VALUE`` (a Python literal) overwrites one more. Unknown keys are an error, so a typo
never silently trains the default. Reference: configs/lm/README.md:1-25, docs/guides/writing-configs.md.
"""

from __future__ import annotations

import argparse
import ast
import importlib.util
import runpy
from types import ModuleType
from typing import Any


def _is_knob(name: str) -> bool:
    """UPPER_CASE and not private: a config may keep helpers of its own under a leading underscore."""
    return name.isupper() and not name.startswith("_")


def load_config_file(path: str) -> dict[str, Any]:
    ns = runpy.run_path(path)
    if callable(ns.get("config_gen")):
        out = ns["config_gen"]()
        if not isinstance(out, dict):
            raise TypeError(f"{path}: config_gen() must return a dict")
        return {k: v for k, v in out.items() if _is_knob(k)}
    return {k: v for k, v in ns.items() if _is_knob(k)}


def parse_value(text: str) -> Any:
    try:
        return ast.literal_eval(text)
    except (ValueError, SyntaxError):
        return text


def apply_overrides(module: ModuleType | dict, overrides: dict[str, Any], source: str = "config") -> None:
    target = module if isinstance(module, dict) else vars(module)
    known = {k for k in target if k.isupper()}
    for key, value in overrides.items():
        if key not in known:
            raise KeyError(f"{source}: unknown knob {key!r}; the script declares {sorted(known)}")
        if isinstance(target[key], dict) and isinstance(value, dict):
            target[key] = {**target[key], **value}
        else:
            target[key] = value


def configure(module: ModuleType | dict, argv: list[str] | None = None) -> argparse.Namespace:
    """Parse ``--config FILE`` (repeatable) and ``--set KEY=VALUE`` (repeatable) and apply them in order."""
    ap = argparse.ArgumentParser(add_help=True)
    ap.add_argument("--config", action="append", default=[])
    ap.add_argument("--set", action="append", default=[], metavar="KEY=VALUE")
    args, rest = ap.parse_known_args(argv)
    for path in args.config:
        apply_overrides(module, load_config_file(path), path)
    for item in args.set:
        if "=" not in item:
            raise ValueError(f"--set expects KEY=VALUE, got {item!r}")
        k, v = item.split("=", 1)
        apply_overrides(module, {k.strip(): parse_value(v)}, "--set")
    args.rest = rest
    return args


def run_script(script_path: str, argv: list[str] | None = None):
    """``python -m kohakuwullm_b200.cli.run script.py --config ... --set ...``: import, configure, ``main()``."""
    spec = importlib.util.spec_from_file_location("__kwu_script__", script_path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    configure(module, argv)
    return module.main()
