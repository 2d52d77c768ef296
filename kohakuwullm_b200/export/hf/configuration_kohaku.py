"""Hugging Face configuration of an exported model (shipped into the exported repository).
Reference: src/kohakuwullm/export/hf/configuration_kohaku.py."""

from transformers import PretrainedConfig


class KohakuConfig(PretrainedConfig):
    model_type = "kohaku"

    def __init__(self, vocab_size=65536, hidden_size=1024, num_hidden_layers=24, num_attention_heads=16,
                 num_key_value_heads=4, head_dim=64, intermediate_size=2816, rms_norm_eps=1e-6, kohaku_rope_theta=10000.0,
                 kohaku_rope_scaling=None, kohaku_rope_factor=1.0, max_position_embeddings=8192, qk_norm=True, windows=None,
                 num_sinks=0, moe_layers=None, moe_num_experts=0, moe_top_k=0, moe_num_shared=0,
                 moe_intermediate_size=0, moe_score="sigmoid", moe_norm_topk_prob=True, moe_scaling=1.0,
                 tie_word_embeddings=False, embedding_scale=False, logit_soft_cap=None, hidden_act="silu",
                 residual_scale=1.0, rope_partial=1.0, **kwargs):
        self.vocab_size, self.hidden_size, self.num_hidden_layers = vocab_size, hidden_size, num_hidden_layers
        self.num_attention_heads, self.num_key_value_heads, self.head_dim = num_attention_heads, num_key_value_heads, head_dim
        self.intermediate_size, self.rms_norm_eps = intermediate_size, rms_norm_eps
        # prefixed so that transformers does not reinterpret them as its own rope_scaling / rope_parameters dicts
        self.kohaku_rope_theta, self.kohaku_rope_scaling, self.kohaku_rope_factor = kohaku_rope_theta, kohaku_rope_scaling, kohaku_rope_factor
        self.max_position_embeddings, self.qk_norm = max_position_embeddings, qk_norm
        self.windows = windows or [None] * num_hidden_layers
        self.num_sinks = num_sinks
        self.moe_layers = moe_layers or [False] * num_hidden_layers
        self.moe_num_experts, self.moe_top_k, self.moe_num_shared = moe_num_experts, moe_top_k, moe_num_shared
        self.moe_intermediate_size, self.moe_score = moe_intermediate_size, moe_score
        self.moe_norm_topk_prob, self.moe_scaling = moe_norm_topk_prob, moe_scaling
        self.embedding_scale, self.logit_soft_cap = embedding_scale, logit_soft_cap
        # gate activation of the dense MLPs ("silu" or "gelu_tanh"), multiplier of every branch output, rotated share of a head
        self.hidden_act, self.residual_scale, self.rope_partial = hidden_act, residual_scale, rope_partial
        super().__init__(tie_word_embeddings=tie_word_embeddings, **kwargs)
