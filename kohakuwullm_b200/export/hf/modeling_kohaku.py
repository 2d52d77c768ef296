"""Stand-alone Hugging Face implementation of an exported model: plain PyTorch, no dependency on the
training framework, so the exported repository works with ``trust_remote_code``. Architecture: pre-norm
blocks, fused-qkv attention with per-head QK-RMSNorm, rotary embedding (none / linear / NTK / YaRN),
GQA, sliding windows, sink logits, SwiGLU MLP, and DeepSeekMoE layers with stacked experts, score
function and selection bias. Reference: src/kohakuwullm/export/hf/modeling_kohaku.py:23-321."""

import math

import torch
from torch import nn
from transformers import PreTrainedModel
from transformers.modeling_outputs import CausalLMOutputWithPast

from .configuration_kohaku import KohakuConfig


def _rms(x, w, eps):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (y * w.float() if w is not None else y).to(x.dtype)


class KohakuRMSNorm(nn.Module):
    def __init__(self, dim, eps):
        super().__init__()
        self.weight, self.eps = nn.Parameter(torch.ones(dim)), eps

    def forward(self, x):
        return _rms(x, self.weight, self.eps)


def _inv_freq(cfg: KohakuConfig):
    d = int(cfg.head_dim * getattr(cfg, "rope_partial", 1.0)) // 2 * 2      # only the first d channels of a head rotate
    theta, f = cfg.kohaku_rope_theta, cfg.kohaku_rope_factor
    idx = torch.arange(0, d, 2, dtype=torch.float64)
    scale = 1.0
    if cfg.kohaku_rope_scaling in (None, "none", "linear"):
        inv = theta ** (-idx / d)
    elif cfg.kohaku_rope_scaling == "ntk":
        inv = (theta * f ** (d / max(d - 2, 1))) ** (-idx / d)
    else:  # yarn
        ex = theta ** (-idx / d)

        def corr(rot):
            return d * math.log(cfg.max_position_embeddings / (rot * 2 * math.pi)) / (2 * math.log(theta))

        lo, hi = max(math.floor(corr(32.0)), 0), min(math.ceil(corr(1.0)), d // 2 - 1)
        ramp = ((torch.arange(d // 2, dtype=torch.float64) - lo) / max(hi - lo, 1e-3)).clamp(0, 1)
        inv = ex / f * ramp + ex * (1 - ramp)
        scale = 0.1 * math.log(f) + 1.0 if f > 1 else 1.0
    pos_scale = 1.0 / f if cfg.kohaku_rope_scaling == "linear" else 1.0
    return inv.float(), pos_scale, scale


class KohakuAttention(nn.Module):
    def __init__(self, cfg: KohakuConfig, layer: int):
        super().__init__()
        self.cfg, self.layer = cfg, layer
        H, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        self.qkv_proj = nn.Linear(cfg.hidden_size, (H + 2 * Hkv) * D, bias=False)
        self.o_proj = nn.Linear(H * D, cfg.hidden_size, bias=False)
        self.q_norm = nn.Parameter(torch.ones(D)) if cfg.qk_norm else None
        self.k_norm = nn.Parameter(torch.ones(D)) if cfg.qk_norm else None
        self.sink = nn.Parameter(torch.zeros(H, cfg.num_sinks)) if cfg.num_sinks else None
        self.window = cfg.windows[layer]

    def forward(self, x, cos, sin, q_pos, past):
        cfg = self.cfg
        B, S, _ = x.shape
        H, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        qkv = self.qkv_proj(x)
        q = qkv[..., : H * D].view(B, S, H, D)
        k = qkv[..., H * D:(H + Hkv) * D].view(B, S, Hkv, D)
        v = qkv[..., (H + Hkv) * D:].view(B, S, Hkv, D)
        if cfg.qk_norm:
            q, k = _rms(q, self.q_norm, cfg.rms_norm_eps), _rms(k, self.k_norm, cfg.rms_norm_eps)

        def rot(t):
            half = cos.shape[-1]
            tf = t.float()
            a, b, tail = tf[..., :half], tf[..., half:2 * half], tf[..., 2 * half:]
            c, s = cos[:, :, None, :], sin[:, :, None, :]
            return torch.cat([a * c - b * s, b * c + a * s, tail], -1).to(t.dtype)

        q, k = rot(q), rot(k)
        if past is not None:
            pk, pv, ppos = past
            k, v = torch.cat([pk, k], 1), torch.cat([pv, v], 1)
            k_pos = torch.cat([ppos, q_pos], 1)
        else:
            k_pos = q_pos
        new_past = (k, v, k_pos)
        g = H // Hkv
        qf = q.float().permute(0, 2, 1, 3)
        kf = k.float().permute(0, 2, 1, 3).repeat_interleave(g, 1)
        vf = v.float().permute(0, 2, 1, 3).repeat_interleave(g, 1)
        scores = qf @ kf.transpose(-1, -2) / math.sqrt(D)
        ok = k_pos[:, None, :] <= q_pos[:, :, None]
        if self.window is not None:
            ok &= (q_pos[:, :, None] - k_pos[:, None, :]) < self.window
        scores = scores.masked_fill(~ok[:, None], float("-inf"))
        lse = torch.logsumexp(scores, -1)
        if self.sink is not None:
            lse = torch.logaddexp(lse, torch.logsumexp(self.sink.float(), -1)[None, :, None])
        out = (torch.exp(scores - lse[..., None]) @ vf).permute(0, 2, 1, 3).reshape(B, S, H * D)
        return self.o_proj(out.to(x.dtype)), new_past


class KohakuMLP(nn.Module):
    def __init__(self, dim, hidden, act="silu"):
        super().__init__()
        self.w_in = nn.Linear(dim, 2 * hidden, bias=False)
        self.w_out = nn.Linear(hidden, dim, bias=False)
        self.act = act

    def forward(self, x):
        g, v = self.w_in(x).chunk(2, -1)
        g = torch.nn.functional.gelu(g, approximate="tanh") if self.act == "gelu_tanh" else torch.nn.functional.silu(g)
        return self.w_out(g * v)


class KohakuMoE(nn.Module):
    def __init__(self, cfg: KohakuConfig):
        super().__init__()
        E, Hd, D = cfg.moe_num_experts, cfg.moe_intermediate_size, cfg.hidden_size
        self.cfg = cfg
        self.router = nn.Linear(D, E, bias=False)
        self.register_buffer("expert_bias", torch.zeros(E))
        self.w_in = nn.Parameter(torch.empty(E, 2 * Hd, D))
        self.w_out = nn.Parameter(torch.empty(E, D, Hd))
        self.shared = KohakuMLP(D, Hd * cfg.moe_num_shared) if cfg.moe_num_shared else None

    def forward(self, x):
        cfg = self.cfg
        flat = x.reshape(-1, x.shape[-1])
        logits = self.router(flat.float().to(self.router.weight.dtype)).float()
        s = torch.sigmoid(logits) if cfg.moe_score == "sigmoid" else (
            torch.softmax(logits, -1) if cfg.moe_score == "softmax" else torch.sqrt(torch.nn.functional.softplus(logits)))
        idx = (s + self.expert_bias).topk(cfg.moe_top_k, -1).indices
        w = s.gather(1, idx)
        if cfg.moe_norm_topk_prob:
            w = w / (w.sum(-1, keepdim=True) + 1e-20)
        w = w * cfg.moe_scaling
        out = torch.zeros_like(flat, dtype=torch.float32)
        for e in range(cfg.moe_num_experts):
            tok, slot = (idx == e).nonzero(as_tuple=True)
            if tok.numel():
                g, v = (flat[tok] @ self.w_in[e].t()).chunk(2, -1)
                y = (torch.nn.functional.silu(g) * v) @ self.w_out[e].t()
                out.index_add_(0, tok, y.float() * w[tok, slot][:, None])
        out = out.to(x.dtype)
        if self.shared is not None:
            out = out + self.shared(flat)
        return out.reshape(x.shape)


class KohakuBlock(nn.Module):
    def __init__(self, cfg: KohakuConfig, layer: int):
        super().__init__()
        self.norm_attn = KohakuRMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.attn = KohakuAttention(cfg, layer)
        self.norm_mlp = KohakuRMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.mlp = KohakuMoE(cfg) if cfg.moe_layers[layer] else \
            KohakuMLP(cfg.hidden_size, cfg.intermediate_size, getattr(cfg, "hidden_act", "silu"))
        self.scale = float(getattr(cfg, "residual_scale", 1.0))

    def forward(self, x, cos, sin, pos, past):
        a, past = self.attn(self.norm_attn(x), cos, sin, pos, past)
        x = x + a * self.scale
        return x + self.mlp(self.norm_mlp(x)) * self.scale, past


class KohakuForCausalLM(PreTrainedModel):
    config_class = KohakuConfig
    _no_split_modules = ["KohakuBlock"]

    def __init__(self, config: KohakuConfig):
        super().__init__(config)
        self.embed = nn.Embedding(config.vocab_size, config.hidden_size)
        self.blocks = nn.ModuleList(KohakuBlock(config, i) for i in range(config.num_hidden_layers))
        self.final_norm = KohakuRMSNorm(config.hidden_size, config.rms_norm_eps)
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)
        inv, self.pos_scale, self.attn_scale = _inv_freq(config)
        self.register_buffer("inv_freq", inv, persistent=False)
        self.post_init()

    def get_input_embeddings(self):
        return self.embed

    def get_output_embeddings(self):
        return self.lm_head

    def forward(self, input_ids, past_key_values=None, labels=None, use_cache=False, **_unused):
        B, S = input_ids.shape
        start = 0 if not past_key_values else past_key_values[0][2].shape[1]
        pos = torch.arange(start, start + S, device=input_ids.device)[None].expand(B, S)
        ang = pos[..., None].float() * self.pos_scale * self.inv_freq[None, None, :]
        cos, sin = ang.cos() * self.attn_scale, ang.sin() * self.attn_scale
        x = self.embed(input_ids)
        if self.config.embedding_scale:
            x = x * math.sqrt(self.config.hidden_size)
        new_past = []
        for i, blk in enumerate(self.blocks):
            x, p = blk(x, cos, sin, pos, past_key_values[i] if past_key_values else None)
            new_past.append(p)
        logits = self.lm_head(self.final_norm(x)).float()
        if self.config.logit_soft_cap:
            logits = self.config.logit_soft_cap * torch.tanh(logits / self.config.logit_soft_cap)
        loss = None
        if labels is not None:
            loss = torch.nn.functional.cross_entropy(logits[:, :-1].reshape(-1, logits.shape[-1]), labels[:, 1:].reshape(-1),
                                                     ignore_index=-100)
        return CausalLMOutputWithPast(loss=loss, logits=logits, past_key_values=tuple(new_past) if use_cache else None)
