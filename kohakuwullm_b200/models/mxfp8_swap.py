"""Post-initialisation MXFP8 conversion of a built model.

``swap_mxfp8(model)`` walks the module tree and turns on MXFP8 for the linear layers selected BY THE
TYPE OF THEIR PARENT: the q/k/v/o projections of attention layers and the projections of the dense
MLPs (gated or not). Everything else (embedding, head, router gates, norms) stays 16-bit. A layer is
rejected when it has a bias or when either feature dimension is not a multiple of 128; rejections
inside a selected parent are reported as ``blocking`` so a caller can refuse a partial conversion.
Bare-parameter matmuls (stacked expert weights) are declared by their module through
``mxfp8_matmuls()`` and switched on through ``enable_mxfp8()``.

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


@dataclass
class SwapReport:
    modules: list[str] = field(default_factory=list)      # converted
    skipped: dict[str, str] = field(default_factory=dict)  # out of scope, with the reason
    blocking: dict[str, str] = field(default_factory=dict)  # selected but not convertible
    declared: list[str] = field(default_factory=list)      # bare-parameter matmuls switched on

    def __str__(self) -> str:
        return (f"mxfp8: {len(self.modules)} linears + {len(self.declared)} declared matmuls converted, "
                f"{len(self.skipped)} skipped, {len(self.blocking)} blocking")


def _reject(lin: Linear) -> str | None:
    if lin.bias is not None:
        return "has a bias"
    if lin.in_features % 128 or lin.out_features % 128:
        return f"features {lin.in_features}->{lin.out_features} are not multiples of 128"
    return None


def _in_scope(name: str, scope) -> bool:
    return scope is None or any(name.startswith(s) or f".{s}." in f".{name}." for s in scope)


def swap_mxfp8(model: nn.Module, scope: tuple[str, ...] | None = None, convert_declared: bool = True) -> SwapReport:
    report = SwapReport()
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
                if not _in_scope(full, scope):
                    report.skipped[full] = "outside scope"
                    continue
                why = _reject(lin)
                if why:
                    report.blocking[full] = why
                    continue
                lin.mxfp8 = True
                lin._qweight = None
                report.modules.append(full)
        if convert_declared and hasattr(module, "mxfp8_matmuls") and hasattr(module, "enable_mxfp8"):
            if _in_scope(mod_name, scope):
                for decl in module.mxfp8_matmuls():
                    report.declared.append(f"{mod_name}.{decl}")
                module.enable_mxfp8()
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
