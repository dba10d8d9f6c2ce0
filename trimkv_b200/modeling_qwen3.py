"""Qwen3 decoder with retention gates: the caller of the cache hot path.

Mirrors the inference path of the reference model (src/trimkv/models/qwen3/modeling_trimkv_qwen3.py):
separate q/k/v projections with an RMSNorm over each head's q and k (:315-323), SwiGLU MLP (:109-122),
``compress`` called with ``alpha_threshold`` (:751-760).  Parameter names follow the reference so its state
dicts load.  The shared forward order, gates, ``from_pretrained`` and ``generate`` are in modeling_trimkv.py.
"""
from __future__ import annotations

from torch import nn
from transformers.models.qwen3.configuration_qwen3 import Qwen3Config

from .modeling_trimkv import (GatedMLP, RMSNorm, RetentionGate, RetentionGate2, RetentionGate3, RotaryEmbedding,  # noqa: F401
                              TrimKVAttention, TrimKVDecoderLayer, TrimKVForCausalLM, TrimKVModel,
                              apply_rotary_pos_emb, rotate_half, set_trimkv_flags)

Qwen3RMSNorm = RMSNorm
Qwen3RotaryEmbedding = RotaryEmbedding
Qwen3MLP = GatedMLP


class TrimKVQwen3Config(Qwen3Config):
    """Flag surface and defaults of ``TrimKVQwen3Config`` (configuration_trimkv_qwen3.py:10-47).  The shape
    defaults are those of the Qwen3-1.7B architecture; ``attn_implementation`` defaults to this library's kernels."""

    _flags = dict(retention_gate_bias_init=10.0, retention_weight=1.0, memory_size=1024, retention_gate="rg",
                  base_loss="fwkl", attn_impl="rg_attn_flex", compress_memory=True, compress_strategy="alpha",
                  floor_budget_ratio=0.0, alpha_threshold=0.0, buffer_size=128, trainable_params=None,
                  max_seq_len=131072, retention_gate_intermediate_size=512, logit_block_size=-1)
    _shape = dict(vocab_size=151936, hidden_size=2048, intermediate_size=6144, num_hidden_layers=28,
                  num_attention_heads=16, num_key_value_heads=8, head_dim=128, max_position_embeddings=40960,
                  rope_theta=1000000.0, tie_word_embeddings=False)

    def __init__(self, **kwargs):
        rest = set_trimkv_flags(self, self._flags, kwargs)
        rest.setdefault("attn_implementation", "tkv_b200")
        super().__init__(**{**self._shape, **rest})


class TrimKVQwen3Attention(TrimKVAttention):
    def __init__(self, config, layer_idx):
        super().__init__(config, layer_idx)
        h, d, bias = config.hidden_size, self.head_dim, config.attention_bias
        self.q_proj = nn.Linear(h, config.num_attention_heads * d, bias=bias)
        self.k_proj = nn.Linear(h, config.num_key_value_heads * d, bias=bias)
        self.v_proj = nn.Linear(h, config.num_key_value_heads * d, bias=bias)
        self.o_proj = nn.Linear(config.num_attention_heads * d, h, bias=bias)
        self.q_norm = RMSNorm(d, eps=config.rms_norm_eps)
        self.k_norm = RMSNorm(d, eps=config.rms_norm_eps)

    def project(self, hidden_states, hidden_shape):
        return (self.q_norm(self.q_proj(hidden_states).view(hidden_shape)),
                self.k_norm(self.k_proj(hidden_states).view(hidden_shape)),
                self.v_proj(hidden_states).view(hidden_shape))


class TrimKVQwen3DecoderLayer(TrimKVDecoderLayer):
    attention_cls = TrimKVQwen3Attention
    mlp_cls = GatedMLP


class TrimKVQwen3Model(TrimKVModel):
    config_class = TrimKVQwen3Config
    layer_cls = TrimKVQwen3DecoderLayer
    compress_extra = ("alpha_threshold",)
    _no_split_modules = ["TrimKVQwen3DecoderLayer"]


class TrimKVQwen3ForCausalLM(TrimKVForCausalLM):
    config_class = TrimKVQwen3Config
    model_cls = TrimKVQwen3Model
    _no_split_modules = ["TrimKVQwen3DecoderLayer"]


__all__ = ["TrimKVQwen3Config", "TrimKVQwen3ForCausalLM", "TrimKVQwen3Model"]
