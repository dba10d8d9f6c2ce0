"""Family-independent parts of the TRIM-KV decoders: the callers of the cache hot path.

The reference ships one model file per family (src/trimkv/models/{qwen3,llama,phi3}/modeling_trimkv_*.py);
their inference paths differ only in how q/k/v and the MLP are projected (separate or fused weights, q/k
RMSNorm or none, full or partial rotary dims) and in which keywords they hand to ``cache.compress``.
Everything else is shared and lives here:

  * retention gates ``rg`` / ``rg2`` / ``rg3`` (modeling_trimkv_qwen3.py:140-267): ``rg`` reads the layer's
    hidden states, ``rg2``/``rg3`` read the rotated keys concatenated with the values;
  * the attention forward order gate -> RoPE -> ``cache.update`` -> attention -> o_proj (:315-388);
  * the model forward with ONE ``cache.compress`` after the layer stack (:612-769) and the LM head on the kept
    positions (:803-871);
  * ``from_pretrained(path, load_trimkv_weights=True)``: base checkpoint + ``trimkv_weights.pth`` (:510-571),
    local paths only (this library never downloads).

The classes derive from transformers' ``PreTrainedModel`` / ``GenerationMixin`` as the reference's do, so
``model.generate(..., past_key_values=TrimKVCache(...))`` is HF generation.  Dense GEMMs, norms and RoPE are
plain PyTorch here; the fused CUDA decode step is ``decoder.FusedDecodeStep``.
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.nn.functional as F
from torch import nn
from transformers import GenerationMixin, PreTrainedModel
from transformers.activations import ACT2FN
from transformers.modeling_outputs import BaseModelOutputWithPast, CausalLMOutputWithPast

from .attn import get_attention_interface, register_with_transformers
from .cache_utils import TrimKVCache

register_with_transformers()

# Flag surface shared by the three TrimKV*Config classes (configuration_trimkv_qwen3.py:10-47,
# configuration_trimkv_llama.py:26-60, configuration_trimkv_phi3.py:10-41); defaults differ per family.
TRIMKV_FLAGS = ("retention_gate_bias_init", "retention_weight", "memory_size", "retention_gate", "base_loss", "attn_impl",
                "compress_memory", "compress_strategy", "floor_budget_ratio", "alpha_threshold", "buffer_size",
                "trainable_params", "max_seq_len", "retention_gate_intermediate_size", "logit_block_size", "rg_dropout",
                "skip_layers")


def _constant(param, value):
    """``param.fill_(value)`` that leaves alone a parameter transformers has just loaded from a checkpoint (its
    loader re-runs ``_init_weights`` on every module and guards only its own / torch.nn.init's functions)."""
    try:
        from transformers import initialization as hf_init
        hf_init.constant_(param, value)
    except ImportError:
        nn.init.constant_(param, value)


def set_trimkv_flags(config, defaults: dict, given: dict) -> dict:
    """Moves the TRIM-KV flags out of ``given`` onto ``config`` (family defaults where absent); returns the rest."""
    rest = dict(given)
    for name, value in defaults.items():
        setattr(config, name, rest.pop(name, value))
    return rest


def rope_theta_of(config) -> float:
    rp = getattr(config, "rope_parameters", None) or {}
    return float(rp.get("rope_theta", getattr(config, "rope_theta", 10000.0)))


def head_dim_of(config) -> int:
    return getattr(config, "head_dim", None) or config.hidden_size // config.num_attention_heads


def rotary_dim_of(config) -> int:
    rp = getattr(config, "rope_parameters", None) or {}
    factor = rp.get("partial_rotary_factor", getattr(config, "partial_rotary_factor", 1.0)) or 1.0
    return int(head_dim_of(config) * factor)


class RMSNorm(nn.Module):
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
    """Rotates the first ``cos.shape[-1]`` dims of q and k (all of them unless the family uses partial rotary)."""
    cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    rd = cos.shape[-1]
    if rd == q.shape[-1]:
        return (q * cos) + (rotate_half(q) * sin), (k * cos) + (rotate_half(k) * sin)
    q_rot, q_pass, k_rot, k_pass = q[..., :rd], q[..., rd:], k[..., :rd], k[..., rd:]
    return (torch.cat([(q_rot * cos) + (rotate_half(q_rot) * sin), q_pass], dim=-1),
            torch.cat([(k_rot * cos) + (rotate_half(k_rot) * sin), k_pass], dim=-1))


class RetentionGate(nn.Module):
    """``rg``: hidden -> intermediate -> Hkv, log-sigmoid output = log beta (modeling_trimkv_qwen3.py:140-179)."""

    reads_hidden_states = True

    def __init__(self, config):
        super().__init__()
        self.config = config
        self.linear1 = nn.Linear(self._in_features(config), config.retention_gate_intermediate_size, bias=True)
        self.linear2 = nn.Linear(config.retention_gate_intermediate_size, config.num_key_value_heads, bias=False)
        self.bias = nn.Parameter(torch.zeros(config.num_key_value_heads))
        self.act_fn = ACT2FN[config.hidden_act]
        self.reset_parameters()

    @staticmethod
    def _in_features(config):
        return config.hidden_size

    def reset_parameters(self):
        std = getattr(self.config, "initializer_range", 0.02)
        for lin in (m for m in self.children() if isinstance(m, nn.Linear)):
            nn.init.normal_(lin.weight, mean=0.0, std=std)
            if lin.bias is not None:
                nn.init.zeros_(lin.bias)
        _constant(self.bias, self.config.retention_gate_bias_init)

    def forward(self, x):
        return F.logsigmoid(self.linear2(self.act_fn(self.linear1(x))) + self.bias)


class RetentionGate2(RetentionGate):
    """``rg2``: same MLP over ``cat(k_rotated, v)`` of all KV heads of a token (:182-224).  Input ``[B,Hkv,S,2D]``."""

    reads_hidden_states = False

    @staticmethod
    def _in_features(config):
        return head_dim_of(config) * config.num_key_value_heads * 2

    def forward(self, kv, transpose=True):
        x = kv.transpose(1, 2) if transpose else kv
        return super().forward(x.reshape(x.shape[0], x.shape[1], -1))


class RetentionGate3(nn.Module):
    """``rg3``: gated MLP (gate_proj, up_proj, down_proj) over the same input as ``rg2`` (:227-267)."""

    reads_hidden_states = False

    def __init__(self, config):
        super().__init__()
        self.config = config
        width, inter = head_dim_of(config) * config.num_key_value_heads * 2, config.retention_gate_intermediate_size
        self.gate_proj = nn.Linear(width, inter, bias=False)
        self.up_proj = nn.Linear(width, inter, bias=False)
        self.down_proj = nn.Linear(inter, config.num_key_value_heads, bias=False)
        self.bias = nn.Parameter(torch.zeros(config.num_key_value_heads))
        self.act_fn = ACT2FN[config.hidden_act]
        self.reset_parameters()

    reset_parameters = RetentionGate.reset_parameters

    def forward(self, kv, transpose=True):
        x = kv.transpose(1, 2) if transpose else kv
        x = x.reshape(x.shape[0], x.shape[1], -1)
        return F.logsigmoid(self.down_proj(self.act_fn(self.gate_proj(x)) * self.up_proj(x)) + self.bias)


GATES = {"rg": RetentionGate, "rg2": RetentionGate2, "rg3": RetentionGate3}


class TrimKVAttention(nn.Module):
    """Shared attention forward; a family supplies ``project`` (hidden states -> q, k, v as ``[B,S,H,D]``)."""

    gate_kinds = ("rg", "rg2", "rg3")

    def __init__(self, config, layer_idx):
        super().__init__()
        self.config, self.layer_idx = config, layer_idx
        self.head_dim = head_dim_of(config)
        self.num_key_value_groups = config.num_attention_heads // config.num_key_value_heads
        self.num_key_value_heads = config.num_key_value_heads
        self.scaling = self.head_dim ** -0.5
        self.is_causal = True
        kind = config.retention_gate
        if kind is not None and kind not in self.gate_kinds:
            raise ValueError(f"retention_gate={kind!r}: this family has {self.gate_kinds}")
        self.retention_gate = GATES[kind](config) if kind is not None else None

    def project(self, hidden_states, hidden_shape):
        raise NotImplementedError

    def forward(self, hidden_states, position_embeddings, past_key_values, cache_position):
        input_shape = hidden_states.shape[:-1]
        q, k, v = self.project(hidden_states, (*input_shape, -1, self.head_dim))
        gate = self.retention_gate
        retention_weights = None
        if gate is not None and gate.reads_hidden_states:
            retention_weights = gate(hidden_states).transpose(1, 2)
        q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
        cos, sin = position_embeddings
        q, k = apply_rotary_pos_emb(q, k, cos, sin)
        if gate is not None and not gate.reads_hidden_states:
            retention_weights = gate(torch.cat([k, v], dim=-1)).transpose(1, 2)
        offset = past_key_values.get_seq_length(self.layer_idx)
        k, v, retention_weights, kv_positions, flash_attn_kwargs = past_key_values.update(
            k, v, retention_weights, cache_position, self.layer_idx, {"sin": sin, "cos": cos})
        attention_interface = get_attention_interface(self.config._attn_implementation)
        attn_output, _, _ = attention_interface(
            self, q, k, v, attention_mask=None, retention_weights=retention_weights, kv_positions=kv_positions,
            offset=offset, dropout=0.0, scaling=self.scaling, sliding_window=None, is_causal=True,
            flash_attn_kwargs=flash_attn_kwargs)
        return self.o_proj(attn_output.reshape(*input_shape, -1).contiguous())


class GatedMLP(nn.Module):
    """SwiGLU with separate gate/up weights (Qwen3, Llama)."""

    def __init__(self, config, bias=False):
        super().__init__()
        self.gate_proj = nn.Linear(config.hidden_size, config.intermediate_size, bias=bias)
        self.up_proj = nn.Linear(config.hidden_size, config.intermediate_size, bias=bias)
        self.down_proj = nn.Linear(config.intermediate_size, config.hidden_size, bias=bias)
        self.act_fn = ACT2FN[config.hidden_act]

    def forward(self, x):
        return self.down_proj(self.act_fn(self.gate_proj(x)) * self.up_proj(x))


class TrimKVDecoderLayer(nn.Module):
    attention_cls = TrimKVAttention
    mlp_cls = GatedMLP

    def __init__(self, config, layer_idx):
        super().__init__()
        self.hidden_size = config.hidden_size
        self.self_attn = self.attention_cls(config, layer_idx)
        self.mlp = self.mlp_cls(config)
        self.input_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)

    def forward(self, hidden_states, position_embeddings, past_key_values, cache_position):
        hidden_states = hidden_states + self.self_attn(
            self.input_layernorm(hidden_states), position_embeddings, past_key_values, cache_position)
        return hidden_states + self.mlp(self.post_attention_layernorm(hidden_states))


class RotaryEmbedding(nn.Module):
    """cos/sin of the (default, unscaled) rotary embedding.  The inverse frequencies stay in fp32 whatever dtype the
    model is cast to (they are not a registered buffer, so ``model.to(bfloat16)`` cannot round them), as they do when
    the reference model is loaded through ``from_pretrained(torch_dtype=bfloat16)``."""

    def __init__(self, config):
        super().__init__()
        rp = getattr(config, "rope_parameters", None) or {}
        kind = rp.get("rope_type", "default")
        if kind != "default":
            raise NotImplementedError(f"rope_type={kind!r} (only the default rotary embedding is built)")
        d = rotary_dim_of(config)
        self._inv_freq = 1.0 / (rope_theta_of(config) ** (torch.arange(0, d, 2, dtype=torch.int64).float() / d))
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


class TrimKVPreTrainedModel(PreTrainedModel):
    base_model_prefix = "model"
    supports_gradient_checkpointing = False
    _skip_keys_device_placement = ["past_key_values"]
    _supports_sdpa = True
    _supports_flash_attn = True
    _supports_attention_backend = True
    # compress() keyword arguments the family's model forward passes besides the common ones
    compress_extra = ()

    def _init_weights(self, module):
        std = self.config.initializer_range
        if isinstance(module, (RetentionGate, RetentionGate3)):
            module.reset_parameters()
        elif isinstance(module, nn.Linear):
            nn.init.normal_(module.weight, mean=0.0, std=std)
            if module.bias is not None:
                nn.init.zeros_(module.bias)
        elif isinstance(module, nn.Embedding):
            nn.init.normal_(module.weight, mean=0.0, std=std)
        elif isinstance(module, RMSNorm):
            nn.init.ones_(module.weight)

    @classmethod
    def from_pretrained(cls, pretrained_model_name_or_path, load_trimkv_weights=True, download_from="local",
                        *model_args, **kwargs):
        """Base checkpoint named by ``config.base_model`` plus the retention-gate weights ``trimkv_weights.pth``
        stored beside ``config.json`` (modeling_trimkv_qwen3.py:510-571).  Only ``download_from="local"`` exists."""
        if not load_trimkv_weights:
            return super().from_pretrained(pretrained_model_name_or_path, *model_args, **kwargs)
        if download_from != "local":
            raise ValueError(f"download_from={download_from!r}: this library loads local paths only")
        path = pretrained_model_name_or_path
        if not os.path.isdir(path):
            raise ValueError(f"Path {path} does not exist.")
        config = cls.config_class.from_pretrained(path)
        base = getattr(config, "base_model", None) or path
        config.base_model = base
        for key in list(kwargs.keys()):
            if hasattr(config, key) and key not in ("torch_dtype", "dtype"):
                setattr(config, key, kwargs.pop(key))
        model = super().from_pretrained(base, *model_args, config=config, **kwargs)
        gate_weights = torch.load(os.path.join(path, "trimkv_weights.pth"), map_location="cpu")
        wanted = [p for p in (config.trainable_params or "retention_gate").split("|") if p]
        mine = {k for k in model.state_dict() if any(w in k for w in wanted)}
        if mine != set(gate_weights.keys()):
            raise ValueError(f"Mismatch between trainable gate state keys: {sorted(mine)} and loaded weights keys: "
                             f"{sorted(gate_weights.keys())}")
        model.load_state_dict(gate_weights, strict=False)
        return model


class TrimKVModel(TrimKVPreTrainedModel):
    layer_cls = TrimKVDecoderLayer

    def __init__(self, config):
        super().__init__(config)
        self.vocab_size = config.vocab_size
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size)
        self.layers = nn.ModuleList([self.layer_cls(config, i) for i in range(config.num_hidden_layers)])
        self.norm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.rotary_emb = RotaryEmbedding(config)
        self.post_init()

    def get_input_embeddings(self):
        return self.embed_tokens

    def set_input_embeddings(self, value):
        self.embed_tokens = value

    def forward(self, input_ids=None, attention_mask=None, position_ids=None, past_key_values=None, inputs_embeds=None,
                use_cache=None, cache_position=None, **_unused):
        # attention_mask is accepted for HF generate and not applied: like the reference's varlen attention
        # (attn/flash_attn.py:79-151) the cache path attends over every cached row of a segment.
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
        self.compress_after_forward(past_key_values)
        return BaseModelOutputWithPast(last_hidden_state=hidden_states, past_key_values=past_key_values)

    def compress_after_forward(self, past_key_values) -> None:
        """The eviction check that ends every forward pass (modeling_trimkv_qwen3.py:751-760)."""
        if self.config.compress_memory:
            extra = {name: getattr(self.config, name) for name in self.compress_extra}
            past_key_values.compress(
                strategy=self.config.compress_strategy, memory_size=self.config.memory_size,
                buffer_size=self.config.buffer_size, floor_budget_ratio=self.config.floor_budget_ratio,
                num_layers=self.config.num_hidden_layers, num_key_value_heads=self.config.num_key_value_heads, **extra)


class TrimKVForCausalLM(TrimKVPreTrainedModel, GenerationMixin):
    model_cls = TrimKVModel
    _tied_weights_keys = {"lm_head.weight": "model.embed_tokens.weight"}

    def __init__(self, config):
        super().__init__(config)
        self.model = self.model_cls(config)
        self.vocab_size = config.vocab_size
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)
        self.post_init()

    def get_input_embeddings(self):
        return self.model.embed_tokens

    def set_input_embeddings(self, value):
        self.model.embed_tokens = value

    def get_output_embeddings(self):
        return self.lm_head

    def set_output_embeddings(self, new_embeddings):
        self.lm_head = new_embeddings

    def get_decoder(self):
        return self.model

    def set_decoder(self, decoder):
        self.model = decoder

    def _fused_step_for(self, input_ids, past_key_values, inputs_embeds, kwargs):
        """The fused CUDA decode step for this call, or None.  Opt-in (``config.fused_decode_step = True``): a forward
        pass of one new token per request on a cache that holds the prompt then runs as ten fused launches per layer
        (``decoder.FusedDecodeStep``) instead of module by module, replayed from a CUDA graph from the third such call
        on (``"eager"`` instead of True: launched from Python every time), under HF ``generate`` as under a
        hand-written loop; same arithmetic up to the summation order of the kernels.  Anything the fused step does not cover (other
        shapes or dtypes, ``inputs_embeds``, hidden-state or attention outputs, CPU, a call with autograd enabled) takes
        the module path."""
        if not getattr(self.config, "fused_decode_step", False) or input_ids is None or inputs_embeds is not None:
            return None
        if (input_ids.dim() != 2 or input_ids.shape[1] != 1 or not input_ids.is_cuda or self.training
                or torch.is_grad_enabled()):      # the fused kernels record nothing for autograd
            return None
        if kwargs.get("output_attentions") or kwargs.get("output_hidden_states") or kwargs.get("labels") is not None:
            return None
        cache = past_key_values
        if (not isinstance(cache, TrimKVCache) or cache.get_seq_length() == 0
                or getattr(cache, "_batch", None) != input_ids.shape[0]):
            return None
        from .decoder import FusedDecodeStep, GraphedForwardStep
        if self.lm_head.weight.dtype not in (torch.bfloat16, torch.float16) or not FusedDecodeStep.supports(self):
            return None
        step = cache.__dict__.get("_fused_step")
        graph = self.config.fused_decode_step != "eager"
        if step is None or step.model is not self or step.use_graph != graph or step.ids.shape[0] != input_ids.shape[0]:
            if step is not None:
                step.release_graph()
            step = cache.__dict__["_fused_step"] = GraphedForwardStep(self, cache, use_graph=graph)
        return step

    def forward(self, input_ids=None, attention_mask=None, position_ids=None, past_key_values=None, inputs_embeds=None,
                use_cache=None, cache_position=None, logits_to_keep=0, **kwargs):
        step = self._fused_step_for(input_ids, past_key_values, inputs_embeds, kwargs)
        if step is not None:
            pos = cache_position[-1:] if cache_position is not None else torch.full(
                (1,), past_key_values.get_seq_length(), device=input_ids.device)
            logits = step(past_key_values, input_ids, pos.to(torch.int64))
            self.model.compress_after_forward(past_key_values)
            return CausalLMOutputWithPast(logits=logits[:, None, :], past_key_values=past_key_values)
        out = self.model(input_ids=input_ids, attention_mask=attention_mask, position_ids=position_ids,
                         past_key_values=past_key_values, inputs_embeds=inputs_embeds, use_cache=use_cache,
                         cache_position=cache_position)
        sl = slice(-logits_to_keep, None) if isinstance(logits_to_keep, int) else logits_to_keep
        logits = self.lm_head(out.last_hidden_state[:, sl, :])
        res = CausalLMOutputWithPast(logits=logits, past_key_values=out.past_key_values)
        res.last_hidden_state = out.last_hidden_state
        return res

    def new_cache(self, device=None) -> TrimKVCache:
        """A ``TrimKVCache`` with this model's eviction settings as sizing hints (the slabs are then allocated once,
        at ``memory_size + buffer_size`` rows per head, and each layer's prompt K/V is reduced inside ``update``)."""
        c = self.config
        hints = dict(memory_size=c.memory_size, buffer_size=c.buffer_size, num_layers=c.num_hidden_layers) \
            if (c.compress_memory and c.compress_strategy == "alpha") else {}
        return TrimKVCache(max_seq_len=c.max_seq_len, device=device or self.device, **hints)

    def generate(self, inputs=None, *args, prefill_chunk_size=None, fused_decode=False, **kwargs):
        """HF ``generate`` with a ``TrimKVCache`` (the reference's usage, examples/test_qwen3.py:51-55); a cache is
        created if none is passed.  ``prefill_chunk_size`` (chunked prompt pass) or ``fused_decode=True`` (the fused
        CUDA decode step replayed from a CUDA graph) select ``generate_greedy`` instead of the HF loop."""
        if prefill_chunk_size or fused_decode:
            ids = inputs if inputs is not None else kwargs.pop("input_ids")
            return self.generate_greedy(ids, prefill_chunk_size=prefill_chunk_size, fused_decode=fused_decode,
                                        **{k: v for k, v in kwargs.items()
                                           if k in ("max_new_tokens", "past_key_values", "eos_token_id")})
        if kwargs.get("past_key_values") is None:
            ids = inputs if inputs is not None else kwargs.get("input_ids")
            kwargs["past_key_values"] = self.new_cache(ids.device if ids is not None else None)
        return super().generate(inputs, *args, **kwargs)

    @torch.inference_mode()
    def generate_greedy(self, input_ids, max_new_tokens=16, past_key_values=None, eos_token_id=None,
                        prefill_chunk_size=None, fused_decode=False):
        """Greedy decoding without the HF machinery; returns ``[B, prompt + new]`` token ids.

        ``fused_decode``: decode through ``decoder.GreedyDecoder`` (ten fused launches per layer, one CUDA graph per
        step, the next token fed back on the device) instead of the module-by-module forward.  Same arithmetic up to
        the summation order of the kernels, several times faster; needs a CUDA model in bf16/f16 of a shape the fused
        step covers (``FusedDecodeStep.supports``) and raises otherwise.

        ``prefill_chunk_size``: feed the prompt in pieces of that many tokens, evicting after each piece (the model
        calls ``compress`` at the end of every forward), so that a prompt much longer than ``memory_size`` never has
        its whole K/V resident.  The eviction schedule, and with it the result, differs from the one-piece prompt pass
        exactly as it would in the reference if it were fed the same pieces."""
        if past_key_values is None:
            past_key_values = self.new_cache(input_ids.device)
        if prefill_chunk_size:
            for lo in range(0, input_ids.shape[1], prefill_chunk_size):
                out = self(input_ids=input_ids[:, lo:lo + prefill_chunk_size], past_key_values=past_key_values,
                           logits_to_keep=1)
        else:
            out = self(input_ids=input_ids, past_key_values=past_key_values, logits_to_keep=1)
        tokens = [input_ids]
        nxt = out.logits[:, -1].argmax(-1, keepdim=True)
        done = torch.zeros_like(nxt, dtype=torch.bool)
        if fused_decode:
            from .decoder import FusedDecodeStep, GreedyDecoder
            if not (input_ids.is_cuda and FusedDecodeStep.supports(self)
                    and self.lm_head.weight.dtype in (torch.bfloat16, torch.float16)):
                raise NotImplementedError("fused_decode needs a CUDA model in bf16/f16 with head_dim 128, the 'rg' gate and SiLU")
            dec = GreedyDecoder(self, past_key_values, use_graph=True, fused=True)
            dec.ids.copy_(nxt)
            try:
                for i in range(max_new_tokens):
                    tokens.append(nxt)
                    if eos_token_id is not None:
                        done |= nxt == eos_token_id
                        if bool(done.all()):
                            break
                    if i + 1 == max_new_tokens:
                        break
                    nxt = dec.step(eager=(i < 2)).clone()   # two plain steps size the workspaces before the capture
            finally:
                dec.release_graph()
                past_key_values.static_views = False
            return torch.cat(tokens, dim=1)
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
