"""Post-initialisation MXFP8 conversion of a built model.

``swap_mxfp8(model)`` walks the module tree and turns on MXFP8 for the linear layers selected BY THE
TYPE OF THEIR PARENT: the q/k/v/o projections of attention layers and the projections of the dense
MLPs (gated or not). Everything else (embedding, head, router gates, norms) stays 16-bit. A layer is
rejected when it has a bias or when either feature dimension is not a multiple of 128; rejections
inside a selected parent are reported as ``blocking`` so a caller can refuse a partial conversion.
Bare-parameter matmuls (stacked expert weights) are declared by their module through
``mxfp8_matmuls()`` and switched on through ``enable_mxfp8()``.

The report also carries a CENSUS of the model's matmul work per token (multiply-accumulates, MoE layers
counted at their active experts) in four buckets: ``fp8`` (converted), ``skipped`` (selected but refused: a
bias, a width that is not a multiple of 128), ``unreached`` (declared convertible but nothing converted it)
and ``never`` (16-bit by design: the vocabulary head, router gates, anything outside ``scope``), and a CLOSING
SWEEP lists every parameter of two or more dimensions that no rule and no declaration claimed
(``unaccounted``): a matmul that silently stayed 16-bit shows up there instead of nowhere.

``refresh_mxfp8_weights(model)`` re-quantises every converted weight (call it after each optimizer
step) and returns how many modules it reached. Reference: src/kohakuwullm/models/mxfp8_swap.py:22-343.
"""

from __future__ import annotations

from dataclasses import dataclass, field

from torch import nn

from kohakuwullm_b200.models.components.attention import Attention
from kohakuwullm_b200.models.components.mlp import GELUMLP, GLUMLP, Linear

PARENT_LINEARS = {
    Attention: ("qkv_proj", "o_proj"),
    GLUMLP: ("w_in", "w_out"),
    GELUMLP: ("fc1", "fc2"),
}


BUCKETS = ("fp8", "skipped", "unreached", "never")


@dataclass
class SwapReport:
    modules: list[str] = field(default_factory=list)      # converted
    skipped: dict[str, str] = field(default_factory=dict)  # out of scope, with the reason
    blocking: dict[str, str] = field(default_factory=dict)  # selected but not convertible
    declared: list[str] = field(default_factory=list)      # bare-parameter matmuls switched on
    unreached: dict[str, str] = field(default_factory=dict)  # declared convertible, not converted, with the reason
    by_design: list[str] = field(default_factory=list)     # 16-bit on purpose (head, router gates, embeddings)
    unaccounted: list[str] = field(default_factory=list)   # >= 2-D parameters nobody claimed (closing sweep)
    mac: dict[str, int] = field(default_factory=lambda: {b: 0 for b in BUCKETS})  # per-token multiply-accumulates

    def share(self, bucket: str) -> float:
        total = sum(self.mac.values())
        return self.mac[bucket] / total if total else 0.0

    def __str__(self) -> str:
        lines = [f"mxfp8: {len(self.modules)} linears + {len(self.declared)} declared matmuls converted, "
                 f"{len(self.skipped)} skipped, {len(self.blocking)} blocking"]
        lines.append("  per-token MAC: " + ", ".join(f"{b} {self.share(b):.1%}" for b in BUCKETS))
        if self.unreached:
            lines.append(f"  unreached: {sorted(self.unreached)}")
        if self.unaccounted:
            lines.append(f"  UNACCOUNTED matmul-shaped parameters: {self.unaccounted}")
        return "\n".join(lines)


def _reject(lin: Linear) -> str | None:
    if lin.bias is not None:
        return "has a bias"
    if lin.in_features % 128 or lin.out_features % 128:
        return f"features {lin.in_features}->{lin.out_features} are not multiples of 128"
    return None


def _in_scope(name: str, scope) -> bool:
    return scope is None or any(name.startswith(s) or f".{s}." in f".{name}." for s in scope)


def _declared_mac(module, names) -> dict[str, int]:
    """Per-token multiply-accumulates of a module's declared bare-parameter matmuls (stacked expert weights
    count at the experts a token is routed to)."""
    out = {}
    top_k = int(getattr(module, "top_k", 1))
    for n in names:
        w = getattr(module, n, None)
        if w is None:
            continue
        per = w[0].numel() if w.dim() == 3 else w.numel()
        out[n] = per * (top_k if w.dim() == 3 else 1)
    return out


def swap_mxfp8(model: nn.Module, scope: tuple[str, ...] | None = None, convert_declared: bool = True) -> SwapReport:
    from kohakuwullm_b200.models.head import LMHead

    report = SwapReport()
    accounted: set[int] = set()
    for mod_name, module in model.named_modules():
        wanted = None
        for parent_type, children in PARENT_LINEARS.items():
            if isinstance(module, parent_type):
                wanted = children
                break
        if wanted is not None:
            for child in wanted:
                lin = getattr(module, child, None)
                if not isinstance(lin, Linear):
                    continue
                full = f"{mod_name}.{child}" if mod_name else child
                mac = lin.in_features * lin.out_features
                accounted.add(id(lin.weight))
                if not _in_scope(full, scope):
                    report.skipped[full] = "outside scope"
                    report.mac["never"] += mac
                    continue
                if lin.mxfp8:                      # a second pass over an already converted model
                    report.modules.append(full)
                    report.mac["fp8"] += mac
                    continue
                why = _reject(lin)
                if why:
                    report.blocking[full] = why
                    report.mac["skipped"] += mac
                    continue
                lin.mxfp8 = True
                lin._qweight = None
                report.modules.append(full)
                report.mac["fp8"] += mac
        # 16-bit by design: the vocabulary head (a contraction into the vocabulary, kept in bf16), embeddings
        # (a gather, no matmul) and router gates (fp32 selection logic)
        if isinstance(module, LMHead):
            proj = getattr(module, "proj", None)
            w = proj.weight if proj is not None else (module._tied[0] if getattr(module, "_tied", None) else None)
            if w is not None:
                accounted.add(id(w))
                report.by_design.append(f"{mod_name}.proj.weight" if mod_name else "proj.weight")
                report.mac["never"] += w.numel()
        elif isinstance(module, nn.Embedding):
            accounted.add(id(module.weight))
            report.by_design.append(f"{mod_name}.weight")
        router = getattr(module, "router", None)
        if router is not None and isinstance(getattr(router, "weight", None), nn.Parameter):
            if id(router.weight) not in accounted:
                accounted.add(id(router.weight))
                report.by_design.append(f"{mod_name}.router.weight")
                report.mac["never"] += router.weight.numel()
        if hasattr(module, "mxfp8_matmuls"):
            stacked = [n for n in ("w_in", "w_out") if isinstance(getattr(module, n, None), nn.Parameter)]
            names = list(module.mxfp8_matmuls())
            macs = _declared_mac(module, set(names) | set(stacked))
            for n in set(names) | set(stacked):
                accounted.add(id(getattr(module, n)))
            refused = [n for n in stacked if n not in names]
            for n in refused:
                report.blocking[f"{mod_name}.{n}"] = "expert width is not a multiple of 128"
                report.mac["skipped"] += macs.get(n, 0)
            if not names:
                continue
            if not _in_scope(mod_name, scope):
                for n in names:
                    report.skipped[f"{mod_name}.{n}"] = "outside scope"
                    report.mac["never"] += macs.get(n, 0)
                continue
            if convert_declared and hasattr(module, "enable_mxfp8"):
                for n in names:
                    report.declared.append(f"{mod_name}.{n}")
                    report.mac["fp8"] += macs.get(n, 0)
                module.enable_mxfp8()
            else:
                why = ("the caller passed convert_declared=False" if not convert_declared else
                       f"{type(module).__name__} declares it convertible but has no enable_mxfp8()")
                for n in names:
                    report.unreached[f"{mod_name}.{n}"] = why
                    report.mac["unreached"] += macs.get(n, 0)
    # closing sweep: a parameter of two or more dimensions is a matmul operand unless somebody said otherwise
    for name, p in model.named_parameters():
        if p.dim() >= 2 and id(p) not in accounted:
            report.unaccounted.append(f"{name}{tuple(p.shape)}")
    return report


def wire_fused_quantisation(backbone: nn.Module) -> int:
    """Tell every RMSNorm whose output (or whose input gradient) feeds an MXFP8 linear to write the fp8 copy
    itself: ``norm_attn -> qkv_proj``, ``norm_mlp -> w_in`` in the forward pass; in the backward pass the
    gradient leaving ``norm_mlp`` is the ``dy`` of ``attn.o_proj`` and the one leaving the NEXT block's
    ``norm_attn`` (or the final norm) is the ``dy`` of ``mlp.w_out``. Returns the number of flags set."""
    from kohakuwullm_b200.models.components.norm import RMSNorm

    def is_mx(module, name):
        lin = getattr(module, name, None)
        return isinstance(lin, Linear) and lin.mxfp8

    blocks = list(getattr(backbone, "blocks", []))
    n = 0
    for i, blk in enumerate(blocks):
        plain = getattr(blk, "post_attn", None) is None and getattr(blk, "residual_scale", 1.0) == 1.0
        if isinstance(blk.norm_attn, RMSNorm):
            blk.norm_attn.emit_mx = is_mx(blk.attn, "qkv_proj")
            prev_out = i > 0 and plain and is_mx(blocks[i - 1].mlp, "w_out")
            blk.norm_attn.emit_mx_grad = bool(prev_out)
            n += int(blk.norm_attn.emit_mx) + int(blk.norm_attn.emit_mx_grad)
        if isinstance(blk.norm_mlp, RMSNorm):
            blk.norm_mlp.emit_mx = is_mx(blk.mlp, "w_in")
            blk.norm_mlp.emit_mx_grad = plain and is_mx(blk.attn, "o_proj")
            n += int(blk.norm_mlp.emit_mx) + int(blk.norm_mlp.emit_mx_grad)
    final = getattr(backbone, "final_norm", None)
    if blocks and isinstance(final, RMSNorm):
        last = blocks[-1]
        plain = getattr(last, "post_mlp", None) is None and getattr(last, "residual_scale", 1.0) == 1.0
        final.emit_mx_grad = plain and is_mx(last.mlp, "w_out")
        n += int(final.emit_mx_grad)
    return n


def refresh_mxfp8_weights(model: nn.Module) -> int:
    count = 0
    for module in model.modules():
        if isinstance(module, Linear) and module.mxfp8:
            module.refresh_quantized_weight()
            count += 1
        elif hasattr(module, "refresh_mxfp8") and not isinstance(module, type(model)):
            count += int(bool(module.refresh_mxfp8()))
    return count
