"""``LMArchConfig`` — every knob of the architecture — and the table of named presets.

Component fields (``norm``, ``mlp``, ``attn``, ``posenc``, ``moe_router``) are *specs* resolved
once by :func:`kohakuwullm_b200.registry.build`. Field names follow the reference's
``LMArchConfig`` (src/kohakuwullm/models/presets.py:12-152) so that a config written for it
loads here unchanged; the preset names of its ladder are kept as well (``:157-398``), and the
five benchmark shapes this framework is measured on are added under ``B200-*``.
"""

from __future__ import annotations

from dataclasses import dataclass, field, fields
from typing import Any


@dataclass
class LMArchConfig:
    # shape
    vocab_size: int = 65536
    dim: int = 1024
    depth: int = 24
    heads: int = 16
    kv_heads: int | None = 4
    head_dim: int | None = None
    mlp_ratio: float = 4.0
    mlp_hidden: int | None = None
    mlp_multiple_of: int = 128
    max_position: int = 8192
    # components (specs)
    norm: Any = "rmsnorm"
    mlp: Any = "swiglu"
    attn: Any = "flash"
    attn_sliding: Any = None          # backend used only by sliding-window layers (None: same as attn)
    posenc: Any = "rope"
    norm_eps: float = 1e-6
    # attention detail
    qk_norm: bool = True
    qk_norm_affine: bool = True
    attn_bias: bool = False
    attn_sink: bool = False
    attn_num_sinks: int = 1           # learned sink logits per head (the reference has exactly one)
    sliding_window: int | None = None
    global_layer_every: int = 0
    window_pattern: list[int | None] | None = None
    rope_theta: float = 10000.0
    rope_scaling: str | None = None   # None | "linear" | "ntk" | "yarn"
    rope_factor: float = 1.0
    rope_partial: float = 1.0
    # mixture of experts (inactive while moe_every == 0)
    moe_every: int = 0
    moe_first_dense: int = 0
    moe_num_experts: int = 64
    moe_top_k: int = 8
    moe_num_shared: int = 1
    moe_hidden: int | None = None
    moe_ratio: float = 4.0
    moe_router: Any = "topk"
    moe_router_kwargs: dict = field(default_factory=dict)
    moe_mlp: str | None = None
    moe_mlp_kwargs: dict = field(default_factory=dict)
    # head / embedding
    tie_embeddings: bool = False
    embedding_scale: bool = False
    logit_soft_cap: float | None = None
    z_loss_weight: float = 0.0
    # residual / init
    post_norm: bool = False
    scale_residual_by_depth: bool = False
    init_std: float = 0.02
    mup_base_dim: int | None = None
    # runtime
    grad_ckpt: bool = False
    mxfp8: bool = False

    def __post_init__(self) -> None:
        if self.head_dim is None:
            if self.dim % self.heads:
                raise ValueError(f"dim {self.dim} is not a multiple of heads {self.heads}; give head_dim")
            self.head_dim = self.dim // self.heads
        if self.kv_heads is None:
            self.kv_heads = self.heads
        if self.heads % self.kv_heads:
            raise ValueError(f"heads {self.heads} must be a multiple of kv_heads {self.kv_heads}")

    # ------------------------------------------------------------------ derived per-layer views
    @property
    def windows(self) -> list[int | None]:
        """Window width of each layer (``None`` = full causal). The last layer is always global."""
        n = self.depth
        if self.window_pattern is not None:
            pat = list(self.window_pattern)
            out = [pat[i % len(pat)] for i in range(n)]
        elif self.sliding_window is None:
            return [None] * n
        elif self.global_layer_every <= 0:
            return [self.sliding_window] * n
        else:
            out = [None if (i + 1) % self.global_layer_every == 0 else self.sliding_window for i in range(n)]
        out[-1] = None
        return out

    @property
    def layer_types(self) -> list[str]:
        return ["sliding" if w is not None else "full" for w in self.windows]

    @property
    def moe_layers(self) -> list[bool]:
        if self.moe_every <= 0:
            return [False] * self.depth
        first = self.moe_first_dense
        return [i >= first and (i - first) % self.moe_every == 0 for i in range(self.depth)]

    def window_for(self, layer: int) -> int | None:
        return self.windows[layer]

    def attn_for(self, layer: int) -> Any:
        if self.attn_sliding is not None and self.windows[layer] is not None:
            return self.attn_sliding
        return self.attn

    @property
    def residual_scale(self) -> float:
        return self.depth ** -0.5 if self.scale_residual_by_depth else 1.0

    def replace(self, **changes: Any) -> "LMArchConfig":
        base = {f.name: getattr(self, f.name) for f in fields(self)}
        base.update(changes)
        return LMArchConfig(**base)


def _dense(dim, depth, heads, kv, hd=64, **kw):
    return dict(dim=dim, depth=depth, heads=heads, kv_heads=kv, head_dim=hd, **kw)


def _sparse(dim, depth, heads, kv, experts, top_k, hidden, first_dense=1, shared=1, **kw):
    return dict(dim=dim, depth=depth, heads=heads, kv_heads=kv, head_dim=64, moe_every=1,
                moe_first_dense=first_dense, moe_num_experts=experts, moe_top_k=top_k,
                moe_num_shared=shared, moe_hidden=hidden, **kw)


PRESETS: dict[str, dict[str, Any]] = {
    # retired dense ladder
    "Nano-25M": _dense(384, 8, 6, 2),
    "Nano-100M": _dense(640, 14, 10, 2),
    "Nano-200M": _dense(896, 16, 14, 2),
    "Nano-200M-wide": _dense(1152, 10, 18, 3),
    "Nano-200M-deep": _dense(704, 26, 11, 1),
    "Nano-500M": _dense(1280, 20, 20, 4),
    "Nano-500M-wide": _dense(1664, 12, 26, 2),
    "Nano-500M-deep": _dense(1024, 32, 16, 2),
    "Nano-1B": _dense(1792, 26, 28, 4),
    "Nano-1B-wide": _dense(2304, 16, 18, 3, hd=128),
    "Nano-1B-deep": _dense(1408, 42, 22, 2),
    # retired sparse ladder
    "MoE-1B-A120M": _sparse(640, 18, 10, 2, 64, 3, 448),
    "MoE-1B-A280M": _sparse(1024, 20, 16, 4, 32, 4, 512),
    "MoE-2B-A370M": _sparse(1152, 24, 18, 3, 48, 4, 512, first_dense=2),
    "MoE-3B-A500M": _sparse(1280, 28, 20, 4, 64, 6, 448, first_dense=2),
    "MoE-3B-A500M-wide": _sparse(1792, 16, 28, 4, 48, 4, 704),
    "MoE-3B-A500M-deep": _sparse(1024, 40, 16, 2, 80, 7, 320, first_dense=2),
    "MoE-8B-A1B": _sparse(1536, 32, 24, 4, 96, 8, 576, first_dense=2),
    # Kohaku dense
    "Kohaku-200M": _dense(768, 17, 12, 2, mlp_hidden=2048),
    "Kohaku-500M": _dense(1280, 22, 20, 4, mlp_hidden=3456),
    "Kohaku-1B": _dense(1536, 32, 24, 4, mlp_hidden=4096),
    "Kohaku-1.5B": _dense(1792, 39, 28, 4, mlp_hidden=4736),
    # Kohaku sparse
    "Kohaku-MoE-1B": _sparse(768, 16, 12, 2, 64, 8, 384, mlp_hidden=2048),
    "Kohaku-MoE-2B": _sparse(896, 21, 14, 2, 64, 8, 512, mlp_hidden=2432),
    "Kohaku-MoE-3B": _sparse(1024, 27, 16, 2, 64, 8, 512, shared=2, mlp_hidden=2688),
    "Kohaku-MoE-5B": _sparse(1280, 30, 20, 4, 64, 8, 640, mlp_hidden=3456),
    "Kohaku-MoE-8B": _sparse(1536, 33, 24, 4, 128, 16, 384, mlp_hidden=4096),
    # benchmark shapes measured on B200
    "B200-smoke": _dense(256, 4, 4, 2, mlp_hidden=704, rope_theta=10000.0, z_loss_weight=1e-4),
    "B200-dense-546M": _dense(1280, 24, 20, 4, mlp_hidden=3584, rope_theta=500000.0, mxfp8=True),
    "B200-moe-991M": _sparse(1024, 16, 16, 4, 64, 6, 384, shared=2, mlp_hidden=2816,
                             moe_router_kwargs={"score": "sigmoid"}, mxfp8=True),
    "B200-sliding-1B": _dense(1536, 28, 24, 8, mlp_hidden=4096, sliding_window=1024,
                              global_layer_every=4, attn_sink=True, attn_num_sinks=4,
                              rope_scaling="yarn", rope_factor=4.0, max_position=4096),
}

KOHAKU_LADDER: tuple[str, ...] = (
    "Kohaku-200M", "Kohaku-MoE-1B", "Kohaku-500M", "Kohaku-MoE-2B", "Kohaku-1B",
    "Kohaku-MoE-3B", "Kohaku-1.5B", "Kohaku-MoE-5B", "Kohaku-MoE-8B",
)


def get_preset(name: str, **overrides: Any) -> LMArchConfig:
    if name not in PRESETS:
        raise KeyError(f"unknown preset {name!r}; available: {sorted(PRESETS)}")
    return LMArchConfig(**{**PRESETS[name], **overrides})
