"""Reading a directory of end-to-end result files (one JSON per run, as ``step_throughput`` and ``bench.py``
print them): every row is ``clean``, ``contended`` or ``oom``; a configuration that was never run has NO row,
which must stay different from a zero. Reference: src/kohakuwullm/bench/analysis/sweep.py:1-175."""

from __future__ import annotations

import glob
import json
import os

DTYPES = ("fp32", "bf16", "fp16")
OPTIMIZERS = ("adamw", "muon")
FLAGS = ("ckpt", "micro", "compiled", "mxfp8", "graphs", "fused")


def parse_tag(tag: str) -> dict:
    """``dp8_bf16_mxfp8_ckpt`` -> strategy dp8 (dp8_ckpt with checkpointing), dtype, optimizer, flags; parts that
    are none of these are reported as ``unknown`` rather than guessed at."""
    parts = tag.split("_")
    out = {"strategy": parts[0], "dtype": None, "optimizer": None, "flags": [], "unknown": []}
    for p in parts[1:]:
        if p in DTYPES:
            out["dtype"] = p
        elif p in OPTIMIZERS:
            out["optimizer"] = p
        elif p in FLAGS:
            out["flags"].append(p)
        else:
            out["unknown"].append(p)
    if "ckpt" in out["flags"]:
        out["strategy"] = f"{parts[0]}_ckpt"
    return out


def classify(row: dict, max_spread: float = 0.1) -> str:
    if not row.get("ok", True) or row.get("oom"):
        return "oom"
    if row.get("step_spread", 0.0) > max_spread or row.get("contended_fraction", 0.0) > 0.01:
        return "contended"
    clocks = row.get("clocks") or {}
    if any(r in ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown") for r in clocks.get("reasons", [])):
        return "contended"
    return "clean"


def load_rows(directory: str, pattern: str = "*.json") -> list[dict]:
    rows = []
    for path in sorted(glob.glob(os.path.join(directory, pattern))):
        with open(path) as fh:
            text = fh.read().strip()
        for line in text.splitlines() if not text.startswith("{") or "\n{" in text else [text]:
            line = line.strip()
            if not line.startswith("{"):
                continue
            try:
                payload = json.loads(line)
            except ValueError:
                continue
            payload["file"] = os.path.basename(path)
            payload["status"] = classify(payload)
            rows.append(payload)
    return rows


def table(rows: list[dict], key: str = "tokens_per_s") -> str:
    lines = ["| file | model | GPUs | status | " + key + " |", "|---|---|---|---|---|"]
    for r in rows:
        value = r.get(key, r.get("value"))
        model = r.get("preset") or (r.get("config") or {}).get("model", "?")
        shown = f"{value:,.0f}" if isinstance(value, (int, float)) and r["status"] != "oom" else "-"
        lines.append(f"| {r['file']} | {model} | {r.get('n_gpus', '?')} | {r['status']} | {shown} |")
    return "\n".join(lines)
