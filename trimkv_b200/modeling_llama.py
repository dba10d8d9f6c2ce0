"""Llama decoder with retention gates over the same cache path.

Mirrors the inference path of src/trimkv/models/llama/modeling_trimkv_llama.py: q/k/v projections without any
per-head norm (:303-305), optional ``attention_bias`` / ``mlp_bias`` (:165-177, 280-291), gates ``rg`` and ``rg2``
(:275-278), ``compress`` called without ``alpha_threshold`` (:680-688).
"""
from __future__ import annotations

from torch import nn
from transformers import LlamaConfig

from .modeling_trimkv import (GatedMLP, TrimKVAttention, TrimKVDecoderLayer, TrimKVForCausalLM, TrimKVModel,
                              set_trimkv_flags)


class TrimKVLlamaConfig(LlamaConfig):
    """Flag surface and defaults of ``TrimKVLlamaConfig`` (configuration_trimkv_llama.py:26-60)."""

    _flags = dict(retention_gate_bias_init=10.0, retention_weight=1.0, memory_size=2048, retention_gate="rg",
                  base_loss="fwkl", attn_impl="rg_attn_flex", compress_memory=True, compress_strategy="alpha",
                  floor_budget_ratio=0.0, buffer_size=1, trainable_params=None, max_seq_len=20480,
                  retention_gate_intermediate_size=512, rg_dropout=0.1, skip_layers=0)

    def __init__(self, **kwargs):
        rest = set_trimkv_flags(self, self._flags, kwargs)
        rest.setdefault("attn_implementation", "tkv_b200")
        super().__init__(**rest)


class TrimKVLlamaAttention(TrimKVAttention):
    gate_kinds = ("rg", "rg2")

    def __init__(self, config, layer_idx):
        super().__init__(config, layer_idx)
        h, d, bias = config.hidden_size, self.head_dim, config.attention_bias
        self.q_proj = nn.Linear(h, config.num_attention_heads * d, bias=bias)
        self.k_proj = nn.Linear(h, config.num_key_value_heads * d, bias=bias)
        self.v_proj = nn.Linear(h, config.num_key_value_heads * d, bias=bias)
        self.o_proj = nn.Linear(config.num_attention_heads * d, h, bias=bias)

    def project(self, hidden_states, hidden_shape):
        return (self.q_proj(hidden_states).view(hidden_shape), self.k_proj(hidden_states).view(hidden_shape),
                self.v_proj(hidden_states).view(hidden_shape))


class LlamaMLP(GatedMLP):
    def __init__(self, config):
        super().__init__(config, bias=getattr(config, "mlp_bias", False))


class TrimKVLlamaDecoderLayer(TrimKVDecoderLayer):
    attention_cls = TrimKVLlamaAttention
    mlp_cls = LlamaMLP


class TrimKVLlamaModel(TrimKVModel):
    config_class = TrimKVLlamaConfig
    layer_cls = TrimKVLlamaDecoderLayer
    _no_split_modules = ["TrimKVLlamaDecoderLayer"]


class TrimKVLlamaForCausalLM(TrimKVForCausalLM):
    config_class = TrimKVLlamaConfig
    model_cls = TrimKVLlamaModel
    _no_split_modules = ["TrimKVLlamaDecoderLayer"]


__all__ = ["TrimKVLlamaConfig", "TrimKVLlamaForCausalLM", "TrimKVLlamaModel"]
