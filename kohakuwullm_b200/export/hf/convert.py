"""Framework checkpoint / live model -> Hugging Face repository (config, weights, modeling code)."""

from __future__ import annotations

import os
import shutil

import torch


def _name(spec) -> str:
    return spec if isinstance(spec, str) else (spec.get("name") if isinstance(spec, dict) else getattr(spec, "__name__", str(spec)))


NORMS = {"rmsnorm": False, "rmsnorm_native": False, "rmsnorm_triton": False, "gemma_rmsnorm": True}     # name -> scale is 1 + weight
MLPS = {"swiglu": "silu", "swiglu_native": "silu", "swiglu_triton": "silu", "geglu": "gelu_tanh"}


def unsupported_options(cfg) -> list[str]:
    """Architecture options the exported modelling code does not implement. Some of them keep every parameter name
    (a routing variant, a residual rule), so loading the weights would succeed and the exported model would silently
    compute something else: the export refuses them instead."""
    bad = []
    if _name(cfg.norm) not in NORMS:
        bad.append(f"norm={_name(cfg.norm)!r}")
    if _name(cfg.mlp) not in MLPS:
        bad.append(f"mlp={_name(cfg.mlp)!r}")
    if _name(cfg.posenc) != "rope":
        bad.append(f"posenc={_name(cfg.posenc)!r}")
    if cfg.post_norm:
        bad.append("post_norm")
    if cfg.attn_bias:
        bad.append("attn_bias")
    if cfg.qk_norm and not cfg.qk_norm_affine:
        bad.append("qk_norm_affine=False")
    if any(cfg.moe_layers):
        if _name(cfg.moe_router) != "topk":
            bad.append(f"moe_router={_name(cfg.moe_router)!r}")
        if cfg.moe_mlp not in (None, "moe"):
            bad.append(f"moe_mlp={cfg.moe_mlp!r}")
    return bad


def to_hf_config(cfg):
    from kohakuwullm_b200.export.hf.configuration_kohaku import KohakuConfig

    from kohakuwullm_b200.models.components.mlp import resolve_hidden

    rk = cfg.moe_router_kwargs or {}
    # the widths the model itself resolves (an explicit value, else ratio * dim * 2/3 rounded up to the multiple)
    dense_hidden = resolve_hidden(cfg.dim, cfg.mlp_ratio, cfg.mlp_hidden, cfg.mlp_multiple_of, glu=True)
    expert_hidden = resolve_hidden(cfg.dim, cfg.moe_ratio, cfg.moe_hidden, cfg.mlp_multiple_of, glu=True) \
        if any(cfg.moe_layers) else 0
    return KohakuConfig(
        vocab_size=cfg.vocab_size, hidden_size=cfg.dim, num_hidden_layers=cfg.depth, num_attention_heads=cfg.heads,
        num_key_value_heads=cfg.kv_heads, head_dim=cfg.head_dim,
        intermediate_size=dense_hidden,
        rms_norm_eps=cfg.norm_eps, kohaku_rope_theta=cfg.rope_theta, kohaku_rope_scaling=cfg.rope_scaling,
        kohaku_rope_factor=cfg.rope_factor,
        max_position_embeddings=cfg.max_position, qk_norm=cfg.qk_norm, windows=cfg.windows,
        num_sinks=cfg.attn_num_sinks if cfg.attn_sink else 0, moe_layers=cfg.moe_layers,
        moe_num_experts=cfg.moe_num_experts if any(cfg.moe_layers) else 0, moe_top_k=cfg.moe_top_k,
        moe_num_shared=cfg.moe_num_shared, moe_intermediate_size=expert_hidden, moe_score=rk.get("score", "sigmoid"),
        moe_norm_topk_prob=rk.get("norm_topk_prob", True), moe_scaling=rk.get("routed_scaling_factor", 1.0),
        tie_word_embeddings=cfg.tie_embeddings, embedding_scale=cfg.embedding_scale, logit_soft_cap=cfg.logit_soft_cap,
        hidden_act=MLPS.get(_name(cfg.mlp), "silu"), residual_scale=cfg.residual_scale, rope_partial=cfg.rope_partial)


def convert_state_dict(state: dict, cfg) -> dict:
    out = {}
    for k, v in state.items():
        if k.endswith("load_accum"):
            continue
        k = k.replace("head.proj.weight", "lm_head.weight").replace(".mlp.router.weight", ".mlp.router.weight")
        k = k.replace(".mlp.router.expert_bias", ".mlp.expert_bias")
        k = k.replace(".mlp.shared.w_in.weight", ".mlp.shared.w_in.weight")
        out[k] = v
    if cfg.tie_embeddings:
        out["lm_head.weight"] = out["embed.weight"]
    if NORMS.get(_name(cfg.norm), False):
        # the model scales by 1 + weight (zero-initialised weight); the exported norm scales by its weight
        for k in list(out):
            if k.endswith(("norm_attn.weight", "norm_mlp.weight", "final_norm.weight")):
                out[k] = out[k].float() + 1.0
    return out


def export_hf(backbone_or_state, cfg, out_dir: str, dtype=torch.bfloat16):
    from kohakuwullm_b200.export.hf.modeling_kohaku import KohakuForCausalLM

    state = backbone_or_state.state_dict() if hasattr(backbone_or_state, "state_dict") else backbone_or_state
    bad = unsupported_options(cfg)
    if bad:
        raise ValueError("the exported modelling code does not implement: " + ", ".join(bad))
    hf_cfg = to_hf_config(cfg)
    hf_cfg.auto_map = {"AutoConfig": "configuration_kohaku.KohakuConfig",
                       "AutoModelForCausalLM": "modeling_kohaku.KohakuForCausalLM"}
    model = KohakuForCausalLM(hf_cfg)
    missing, unexpected = model.load_state_dict(convert_state_dict(state, cfg), strict=False)
    if unexpected or [m for m in missing if "inv_freq" not in m]:
        raise RuntimeError(f"export mismatch: missing {missing[:5]} unexpected {unexpected[:5]}")
    model.to(dtype).save_pretrained(out_dir, safe_serialization=True)
    here = os.path.dirname(__file__)
    for f in ("configuration_kohaku.py", "modeling_kohaku.py"):
        shutil.copy(os.path.join(here, f), os.path.join(out_dir, f))
    return model
