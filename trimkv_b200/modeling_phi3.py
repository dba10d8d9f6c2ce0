"""Phi-3 decoder with retention gates over the same cache path.

Mirrors the inference path of src/trimkv/models/phi3/modeling_trimkv_phi3.py: one fused ``qkv_proj`` whose output
rows are ``[q | k | v]`` (:338, 353-357), one fused ``gate_up_proj`` whose output is chunked into gate and up
(:93-108), rotary embedding over the first ``rotary_dim`` dims of each head (:160-185), no per-head norm, gates
``rg`` and ``rg2`` (:331-334), ``compress`` called without ``alpha_threshold`` (:791-799).
"""
from __future__ import annotations

from torch import nn
from transformers.activations import ACT2FN
from transformers.models.phi3 import Phi3Config

from .modeling_trimkv import TrimKVAttention, TrimKVDecoderLayer, TrimKVForCausalLM, TrimKVModel, set_trimkv_flags


class TrimKVPhi3Config(Phi3Config):
    """Flag surface and defaults of ``TrimKVPhi3Config`` (configuration_trimkv_phi3.py:10-41)."""

    _flags = dict(retention_gate_bias_init=10.0, retention_weight=1.0, memory_size=1024, retention_gate="rg",
                  base_loss="fwkl", attn_impl="rg_attn_flex", compress_memory=False, compress_strategy="alpha",
                  floor_budget_ratio=0.0, buffer_size=1, trainable_params=None, max_seq_len=20480,
                  retention_gate_intermediate_size=1024)

    def __init__(self, **kwargs):
        rest = set_trimkv_flags(self, self._flags, kwargs)
        rest.setdefault("attn_implementation", "tkv_b200")
        super().__init__(**rest)


class TrimKVPhi3Attention(TrimKVAttention):
    gate_kinds = ("rg", "rg2")

    def __init__(self, config, layer_idx):
        super().__init__(config, layer_idx)
        d = self.head_dim
        self.q_width, self.kv_width = config.num_attention_heads * d, config.num_key_value_heads * d
        self.o_proj = nn.Linear(self.q_width, config.hidden_size, bias=False)
        self.qkv_proj = nn.Linear(config.hidden_size, self.q_width + 2 * self.kv_width, bias=False)

    def project(self, hidden_states, hidden_shape):
        qkv = self.qkv_proj(hidden_states)
        q, k, v = qkv.split([self.q_width, self.kv_width, self.kv_width], dim=-1)
        return q.reshape(hidden_shape), k.reshape(hidden_shape), v.reshape(hidden_shape)


class Phi3MLP(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.gate_up_proj = nn.Linear(config.hidden_size, 2 * config.intermediate_size, bias=False)
        self.down_proj = nn.Linear(config.intermediate_size, config.hidden_size, bias=False)
        self.activation_fn = ACT2FN[config.hidden_act]

    def forward(self, x):
        gate, up = self.gate_up_proj(x).chunk(2, dim=-1)
        return self.down_proj(up * self.activation_fn(gate))


class TrimKVPhi3DecoderLayer(TrimKVDecoderLayer):
    attention_cls = TrimKVPhi3Attention
    mlp_cls = Phi3MLP


class TrimKVPhi3Model(TrimKVModel):
    config_class = TrimKVPhi3Config
    layer_cls = TrimKVPhi3DecoderLayer
    _no_split_modules = ["TrimKVPhi3DecoderLayer"]


class TrimKVPhi3ForCausalLM(TrimKVForCausalLM):
    config_class = TrimKVPhi3Config
    model_cls = TrimKVPhi3Model
    _no_split_modules = ["TrimKVPhi3DecoderLayer"]


__all__ = ["TrimKVPhi3Config", "TrimKVPhi3ForCausalLM", "TrimKVPhi3Model"]
