"""Qwen3 decoder with retention gates: the caller of the cache hot path.

Mirrors the inference path of the reference model (src/trimkv/models/qwen3/modeling_trimkv_qwen3.py):
``RetentionGate`` (:140-179), attention forward with the order gate -> RoPE -> cache.update ->
attention (:315-388), decoder layer (:401-439), model forward with one ``cache.compress`` after the
layer stack (:612-769) and the LM head on the kept positions (:803-871).  Parameter names follow the
reference so its state dicts load.  Dense GEMMs, RMSNorm and RoPE are plain PyTorch; the cache path
(append, eviction, decode attention) is the CUDA library.  ``generate`` is a greedy loop with the
reference's calling convention (``past_key_values=TrimKVCache()``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn.functional as F
from torch import nn

from .attn import get_attention_interface
from .cache_utils import TrimKVCache


class TrimKVQwen3Config:
    """Flag surface of ``TrimKVQwen3Config`` (configuration_trimkv_qwen3.py:10-47) plus the Qwen3 shape fields."""

    def __init__(
        self,
        vocab_size=151936, hidden_size=2048, intermediate_size=6144, num_hidden_layers=28,
        num_attention_heads=16, num_key_value_heads=8, head_dim=128, hidden_act="silu",
        max_position_embeddings=40960, initializer_range=0.02, rms_norm_eps=1e-6, rope_theta=1000000.0,
        attention_bias=False, tie_word_embeddings=False,
        retention_gate_bias_init=10.0, retention_weight=1.0, memory_size=1024, retention_gate="rg",
        base_loss="fwkl", attn_impl="rg_attn_flex", compress_memory=True, compress_strategy="alpha",
        floor_budget_ratio=0.0, alpha_threshold=0.0, buffer_size=128, trainable_params=None,
        max_seq_len=131072, retention_gate_intermediate_size=512, logit_block_size=-1,
        attn_implementation="tkv_b200", torch_dtype=torch.bfloat16, **kwargs,
    ):
        self.vocab_size, self.hidden_size, self.intermediate_size = vocab_size, hidden_size, intermediate_size
        self.num_hidden_layers, self.num_attention_heads = num_hidden_layers, num_attention_heads
        self.num_key_value_heads, self.head_dim, self.hidden_act = num_key_value_heads, head_dim, hidden_act
        self.max_position_embeddings, self.initializer_range = max_position_embeddings, initializer_range
        self.rms_norm_eps, self.rope_theta, self.attention_bias = rms_norm_eps, rope_theta, attention_bias
        self.tie_word_embeddings = tie_word_embeddings
        self.retention_gate_bias_init, self.retention_weight = retention_gate_bias_init, retention_weight
        self.memory_size, self.retention_gate, self.base_loss = memory_size, retention_gate, base_loss
        self.attn_impl, self.compress_memory, self.compress_strategy = attn_impl, compress_memory, compress_strategy
        self.floor_budget_ratio, self.alpha_threshold, self.buffer_size = floor_budget_ratio, alpha_threshold, buffer_size
        self.trainable_params, self.max_seq_len = trainable_params, max_seq_len
        self.retention_gate_intermediate_size, self.logit_block_size = retention_gate_intermediate_size, logit_block_size
        self._attn_implementation = attn_implementation
        self.torch_dtype = torch_dtype
        self.use_cache = True
        for k, v in kwargs.items():
            setattr(self, k, v)


class Qwen3RMSNorm(nn.Module):
    def __init__(self, hidden_size, eps=1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size))
        self.variance_epsilon = eps

    def forward(self, x):
        dt = x.dtype
        x = x.to(torch.float32)
        x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.variance_epsilon)
        return self.weight * x.to(dt)


def rotate_half(x):
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


def apply_rotary_pos_emb(q, k, cos, sin):
    cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    return (q * cos) + (rotate_half(q) * sin), (k * cos) + (rotate_half(k) * sin)


class RetentionGate(nn.Module):
    """hidden -> intermediate -> Hkv, log-sigmoid output = log beta (modeling_trimkv_qwen3.py:140-179)."""

    def __init__(self, config):
        super().__init__()
        self.linear1 = nn.Linear(config.hidden_size, config.retention_gate_intermediate_size, bias=True)
        self.linear2 = nn.Linear(config.retention_gate_intermediate_size, config.num_key_value_heads, bias=False)
        self.bias = nn.Parameter(torch.zeros(config.num_key_value_heads))
        self._init_range, self._bias_init = config.initializer_range, config.retention_gate_bias_init
        self.reset_parameters()

    def reset_parameters(self):
        nn.init.normal_(self.linear1.weight, mean=0.0, std=self._init_range)
        nn.init.zeros_(self.linear1.bias)
        nn.init.normal_(self.linear2.weight, mean=0.0, std=self._init_range)
        with torch.no_grad():
            self.bias.fill_(self._bias_init)

    def forward(self, x):
        return F.logsigmoid(self.linear2(F.silu(self.linear1(x))) + self.bias)


class TrimKVQwen3Attention(nn.Module):
    def __init__(self, config, layer_idx):
        super().__init__()
        self.config, self.layer_idx = config, layer_idx
        self.head_dim = config.head_dim
        self.num_key_value_groups = config.num_attention_heads // config.num_key_value_heads
        self.scaling = self.head_dim ** -0.5
        h, d = config.hidden_size, self.head_dim
        self.q_proj = nn.Linear(h, config.num_attention_heads * d, bias=config.attention_bias)
        self.k_proj = nn.Linear(h, config.num_key_value_heads * d, bias=config.attention_bias)
        self.v_proj = nn.Linear(h, config.num_key_value_heads * d, bias=config.attention_bias)
        self.o_proj = nn.Linear(config.num_attention_heads * d, h, bias=config.attention_bias)
        if config.retention_gate != "rg":
            raise NotImplementedError(f"retention_gate={config.retention_gate!r} (only 'rg' is built)")
        self.retention_gate = RetentionGate(config)
        self.q_norm = Qwen3RMSNorm(d, eps=config.rms_norm_eps)
        self.k_norm = Qwen3RMSNorm(d, eps=config.rms_norm_eps)

    def forward(self, hidden_states, position_embeddings, past_key_values, cache_position):
        input_shape = hidden_states.shape[:-1]
        hidden_shape = (*input_shape, -1, self.head_dim)
        q = self.q_norm(self.q_proj(hidden_states).view(hidden_shape)).transpose(1, 2)
        k = self.k_norm(self.k_proj(hidden_states).view(hidden_shape)).transpose(1, 2)
        v = self.v_proj(hidden_states).view(hidden_shape).transpose(1, 2)
        retention_weights = self.retention_gate(hidden_states).transpose(1, 2)
        cos, sin = position_embeddings
        q, k = apply_rotary_pos_emb(q, k, cos, sin)
        offset = past_key_values.get_seq_length(self.layer_idx)
        k, v, retention_weights, kv_positions, flash_attn_kwargs = past_key_values.update(
            k, v, retention_weights, cache_position, self.layer_idx, None)
        attention_interface = get_attention_interface(self.config._attn_implementation)
        attn_output, _, _ = attention_interface(
            self, q, k, v, attention_mask=None, retention_weights=retention_weights, kv_positions=kv_positions,
            offset=offset, dropout=0.0, scaling=self.scaling, sliding_window=None, is_causal=True,
            flash_attn_kwargs=flash_attn_kwargs)
        return self.o_proj(attn_output.reshape(*input_shape, -1).contiguous())


class Qwen3MLP(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.gate_proj = nn.Linear(config.hidden_size, config.intermediate_size, bias=False)
        self.up_proj = nn.Linear(config.hidden_size, config.intermediate_size, bias=False)
        self.down_proj = nn.Linear(config.intermediate_size, config.hidden_size, bias=False)

    def forward(self, x):
        return self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x))


class TrimKVQwen3DecoderLayer(nn.Module):
    def __init__(self, config, layer_idx):
        super().__init__()
        self.self_attn = TrimKVQwen3Attention(config, layer_idx)
        self.mlp = Qwen3MLP(config)
        self.input_layernorm = Qwen3RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.post_attention_layernorm = Qwen3RMSNorm(config.hidden_size, eps=config.rms_norm_eps)

    def forward(self, hidden_states, position_embeddings, past_key_values, cache_position):
        hidden_states = hidden_states + self.self_attn(
            self.input_layernorm(hidden_states), position_embeddings, past_key_values, cache_position)
        return hidden_states + self.mlp(self.post_attention_layernorm(hidden_states))


class Qwen3RotaryEmbedding(nn.Module):
    """cos/sin of the rotary embedding.  The inverse frequencies stay in fp32 whatever dtype the model is cast
    to (they are not a registered buffer, so ``model.to(bfloat16)`` cannot round them), as they do when the
    reference model is loaded through ``from_pretrained(torch_dtype=bfloat16)``."""

    def __init__(self, config):
        super().__init__()
        d = config.head_dim
        self._inv_freq = 1.0 / (config.rope_theta ** (torch.arange(0, d, 2, dtype=torch.int64).float() / d))
        self._per_device = {}

    def inv_freq_on(self, device):
        t = self._per_device.get(device)
        if t is None:
            t = self._inv_freq.to(device=device, dtype=torch.float32)
            self._per_device[device] = t
        return t

    @torch.no_grad()
    def forward(self, x, position_ids):
        inv = self.inv_freq_on(x.device)
        freqs = position_ids[:, :, None].float() * inv[None, None, :]
        emb = torch.cat((freqs, freqs), dim=-1)
        return emb.cos().to(x.dtype), emb.sin().to(x.dtype)


@dataclass
class TrimKVModelOutput:
    last_hidden_state: torch.Tensor = None
    past_key_values: Optional[TrimKVCache] = None
    logits: Optional[torch.Tensor] = None


class TrimKVQwen3Model(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.config = config
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size)
        self.layers = nn.ModuleList([TrimKVQwen3DecoderLayer(config, i) for i in range(config.num_hidden_layers)])
        self.norm = Qwen3RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.rotary_emb = Qwen3RotaryEmbedding(config)

    def forward(self, input_ids=None, past_key_values=None, inputs_embeds=None, use_cache=True,
                cache_position=None, position_ids=None, **_unused):
        if (input_ids is None) == (inputs_embeds is None):
            raise ValueError("You must specify exactly one of input_ids or inputs_embeds")
        if inputs_embeds is None:
            inputs_embeds = self.embed_tokens(input_ids)
        if past_key_values is None:
            past_key_values = TrimKVCache(max_seq_len=self.config.max_seq_len, device=inputs_embeds.device)
        if cache_position is None:
            seen = past_key_values.get_seq_length()
            cache_position = torch.arange(seen, seen + inputs_embeds.shape[1], device=inputs_embeds.device)
        if position_ids is None:
            position_ids = cache_position.unsqueeze(0)
        hidden_states = inputs_embeds
        position_embeddings = self.rotary_emb(hidden_states, position_ids)
        for layer in self.layers[: self.config.num_hidden_layers]:
            hidden_states = layer(hidden_states, position_embeddings, past_key_values, cache_position)
        hidden_states = self.norm(hidden_states)
        if self.config.compress_memory:
            past_key_values.compress(
                strategy=self.config.compress_strategy, memory_size=self.config.memory_size,
                buffer_size=self.config.buffer_size, floor_budget_ratio=self.config.floor_budget_ratio,
                alpha_threshold=self.config.alpha_threshold, num_layers=self.config.num_hidden_layers,
                num_key_value_heads=self.config.num_key_value_heads)
        return TrimKVModelOutput(last_hidden_state=hidden_states, past_key_values=past_key_values)


class TrimKVQwen3ForCausalLM(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.config = config
        self.model = TrimKVQwen3Model(config)
        self.vocab_size = config.vocab_size
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)
        self.apply(self._init_weights)

    def _init_weights(self, module):
        std = self.config.initializer_range
        if isinstance(module, RetentionGate):
            module.reset_parameters()
        elif isinstance(module, nn.Linear):
            nn.init.normal_(module.weight, mean=0.0, std=std)
            if module.bias is not None:
                nn.init.zeros_(module.bias)
        elif isinstance(module, nn.Embedding):
            nn.init.normal_(module.weight, mean=0.0, std=std)

    @property
    def device(self):
        return self.lm_head.weight.device

    def forward(self, input_ids=None, past_key_values=None, inputs_embeds=None, use_cache=True,
                cache_position=None, logits_to_keep=0, **kwargs):
        out = self.model(input_ids=input_ids, past_key_values=past_key_values, inputs_embeds=inputs_embeds,
                         use_cache=use_cache, cache_position=cache_position, **kwargs)
        sl = slice(-logits_to_keep, None) if isinstance(logits_to_keep, int) else logits_to_keep
        out.logits = self.lm_head(out.last_hidden_state[:, sl, :])
        return out

    @torch.inference_mode()
    def generate(self, input_ids, max_new_tokens=16, past_key_values=None, eos_token_id=None,
                 prefill_chunk_size=None, **_unused):
        """Greedy decoding; returns ``[B, prompt + new]`` token ids like HF ``generate``.

        ``prefill_chunk_size``: feed the prompt in pieces of that many tokens, evicting after each piece (the model
        calls ``compress`` at the end of every forward), so that a prompt much longer than ``memory_size`` never has
        its whole K/V resident.  The eviction schedule, and with it the result, differs from the one-piece prompt pass
        exactly as it would in the reference if it were fed the same pieces."""
        if past_key_values is None:
            hints = dict(memory_size=self.config.memory_size, buffer_size=self.config.buffer_size,
                         num_layers=self.config.num_hidden_layers) \
                if (self.config.compress_memory and self.config.compress_strategy == "alpha") else {}
            past_key_values = TrimKVCache(max_seq_len=self.config.max_seq_len, device=input_ids.device, **hints)
        if prefill_chunk_size:
            for lo in range(0, input_ids.shape[1], prefill_chunk_size):
                out = self(input_ids=input_ids[:, lo:lo + prefill_chunk_size], past_key_values=past_key_values,
                           logits_to_keep=1)
        else:
            out = self(input_ids=input_ids, past_key_values=past_key_values, logits_to_keep=1)
        tokens = [input_ids]
        nxt = out.logits[:, -1].argmax(-1, keepdim=True)
        done = torch.zeros_like(nxt, dtype=torch.bool)
        for i in range(max_new_tokens):
            tokens.append(nxt)
            if eos_token_id is not None:
                done |= nxt == eos_token_id
                if bool(done.all()):
                    break
            if i + 1 == max_new_tokens:
                break
            out = self(input_ids=nxt, past_key_values=past_key_values, logits_to_keep=1)
            nxt = out.logits[:, -1].argmax(-1, keepdim=True)
        return torch.cat(tokens, dim=1)
