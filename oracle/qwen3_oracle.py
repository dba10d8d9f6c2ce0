"""CPU restatement (eager PyTorch) of the reference's decode path.  TEST / BASELINE INFRASTRUCTURE ONLY.

Used as (1) the checker for the model-level parity test and (2) the host-core baseline the benchmark
times (``cpu_baseline`` and ``--impl reference``).  Nothing in the product package imports it.

The reference is eager PyTorch itself, so this restatement uses the same torch ops on CPU tensors:
  * ``EagerTrimKVCache``: ``TrimKVCache.update`` = torch.cat x4 (src/trimkv/cache_utils.py:104-108),
    ``compress``/``compress_layer`` = fp32 score, top-M, sort, 4 gathers (:140-198).  With
    ``canonical=True`` the top-M uses a stable descending sort (lower index wins ties) instead of
    ``torch.topk`` whose tie order is unspecified; the two agree whenever no tie straddles the boundary.
  * ``eager_attention``: src/trimkv/attn/eager_attn.py:48-73 with the causal mask the HF glue builds.
  * ``OracleDecoder`` (alias ``OracleQwen3``): attention forward order gate -> RoPE -> update -> attention
    (src/trimkv/models/qwen3/modeling_trimkv_qwen3.py:315-388), decoder layer (:401-439), model forward
    with compress after the layer stack (:612-769), LM head on the last position (:847-849); the Llama and
    Phi-3 projections and the ``rg2`` / ``rg3`` gates as their model files have them.
Pinning: the cache class is checked against the reference-generated golden vectors in tests/test_oracle.py;
the decoder against tests/golden/model_*.npz, which are outputs of the reference's own model classes run on
CPU (tests/test_model_golden.py: fp32 logits to 1e-5, cache lengths and kept positions exact at every step).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


class EagerTrimKVCache:
    def __init__(self, canonical: bool = True):
        self._seen_tokens = 0
        self.key_cache, self.value_cache = [], []
        self.retention_weights, self.kv_positions = [], []
        self.n_seen_tokens = []
        self.canonical = canonical

    def __len__(self):
        return len(self.key_cache)

    # What HF generation reads from any cache object; the reference's class inherits these from DynamicCache.
    is_compileable = False
    is_sliding = [False]

    def get_mask_sizes(self, cache_position, layer_idx=0):
        return self.get_cache_length(layer_idx) + cache_position.shape[0], 0

    def get_seq_length(self, layer_idx=None):
        if layer_idx is None:
            return self._seen_tokens
        return self.n_seen_tokens[layer_idx] if layer_idx < len(self.n_seen_tokens) else 0

    def get_cache_length(self, layer_idx=0):
        return self.key_cache[layer_idx].shape[-2] if layer_idx < len(self.key_cache) else 0

    def update(self, key_states, value_states, retention_weights, cache_positions, layer_idx, cache_kwargs=None):
        if layer_idx == 0:
            self._seen_tokens += key_states.shape[-2]
        if cache_positions.dim() == 1:
            cache_positions = cache_positions[None, None, :].expand_as(retention_weights)
        if len(self.key_cache) <= layer_idx:
            self.key_cache.append(key_states); self.value_cache.append(value_states)
            self.retention_weights.append(retention_weights); self.kv_positions.append(cache_positions)
            self.n_seen_tokens.append(key_states.shape[-2])
        else:
            self.key_cache[layer_idx] = torch.cat([self.key_cache[layer_idx], key_states], dim=-2)
            self.value_cache[layer_idx] = torch.cat([self.value_cache[layer_idx], value_states], dim=-2)
            self.retention_weights[layer_idx] = torch.cat([self.retention_weights[layer_idx], retention_weights], dim=-1)
            self.kv_positions[layer_idx] = torch.cat([self.kv_positions[layer_idx], cache_positions], dim=-1)
            self.n_seen_tokens[layer_idx] += key_states.shape[-2]
        return (self.key_cache[layer_idx], self.value_cache[layer_idx], self.retention_weights[layer_idx],
                self.kv_positions[layer_idx], {})

    def compress(self, strategy="alpha", memory_size=2048, buffer_size=512, **_ignored):
        for layer_idx in range(len(self.key_cache)):
            if memory_size + buffer_size <= self.get_cache_length(layer_idx):
                self.compress_layer(layer_idx, memory_size)

    def compress_layer(self, layer_idx, memory_size):
        k, v = self.key_cache[layer_idx], self.value_cache[layer_idx]
        pos, rw = self.kv_positions[layer_idx], self.retention_weights[layer_idx]
        q_idx = self.get_seq_length(layer_idx) + 1
        scores = rw.to(torch.float32) * (q_idx - pos)
        if self.canonical:
            idx = torch.sort(scores, dim=-1, descending=True, stable=True).indices[..., :memory_size]
        else:
            idx = torch.topk(scores, memory_size, dim=-1).indices
        idx, _ = torch.sort(idx, dim=-1)
        self.key_cache[layer_idx] = k.gather(-2, idx.unsqueeze(-1).expand(-1, -1, -1, k.shape[-1]))
        self.value_cache[layer_idx] = v.gather(-2, idx.unsqueeze(-1).expand(-1, -1, -1, v.shape[-1]))
        self.retention_weights[layer_idx] = rw.gather(-1, idx)
        self.kv_positions[layer_idx] = pos.gather(-1, idx)


def eager_attention(query, key, value, num_key_value_groups, scaling):
    """query [B,Hq,Q,D]; key/value [B,Hkv,n,D]; causal, bottom-right aligned; returns [B,Q,Hq,D]."""
    b, hkv, n, d = key.shape
    g = num_key_value_groups
    key = key[:, :, None].expand(b, hkv, g, n, d).reshape(b, hkv * g, n, d)
    value = value[:, :, None].expand(b, hkv, g, n, d).reshape(b, hkv * g, n, d)
    w = torch.matmul(query, key.transpose(2, 3)) * scaling
    ql = query.shape[2]
    if ql > 1:
        mask = torch.full((ql, n), float("-inf"), dtype=w.dtype).triu(n - ql + 1)
        w = w + mask
    w = F.softmax(w, dim=-1, dtype=torch.float32).to(query.dtype)
    return torch.matmul(w, value).transpose(1, 2).contiguous()


def _rms(x, weight, eps):
    dt = x.dtype
    x = x.to(torch.float32)
    x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return weight * x.to(dt)


def _rot(x):
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


class OracleDecoder:
    """Functional decoder over a state dict with the reference's parameter names.

    The family is read off the names: ``qkv_proj`` / ``gate_up_proj`` (Phi-3, modeling_trimkv_phi3.py:93-108,338-357),
    ``q_norm`` / ``k_norm`` (Qwen3, modeling_trimkv_qwen3.py:319-320), neither (Llama); biases are applied where the
    state dict has them.  Gates: ``rg`` on the hidden states, ``rg2`` / ``rg3`` on cat(rotated k, v) (:182-267)."""

    def __init__(self, state_dict, config, dtype=torch.float32):
        self.w = {k: v.detach().to("cpu", dtype) for k, v in state_dict.items()}
        self.c = config
        rp = getattr(config, "rope_parameters", None) or {}
        theta = float(rp.get("rope_theta", getattr(config, "rope_theta", 10000.0)))
        self.head_dim = getattr(config, "head_dim", None) or config.hidden_size // config.num_attention_heads
        d = int(self.head_dim * (rp.get("partial_rotary_factor", getattr(config, "partial_rotary_factor", 1.0)) or 1.0))
        self.inv_freq = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.int64).float() / d))
        self.gate_kind = getattr(config, "retention_gate", "rg")

    def _lin(self, name, x):
        return F.linear(x, self.w[name + ".weight"], self.w.get(name + ".bias"))

    def _gate(self, p, x):
        w, g = self.w, p + "self_attn.retention_gate."
        if self.gate_kind == "rg3":
            y = self._lin(g + "down_proj", F.silu(self._lin(g + "gate_proj", x)) * self._lin(g + "up_proj", x))
        else:
            y = self._lin(g + "linear2", F.silu(self._lin(g + "linear1", x)))
        return F.logsigmoid(y + w[g + "bias"])

    def _rope(self, x, cos, sin):
        rd = cos.shape[-1]
        if rd == x.shape[-1]:
            return x * cos + _rot(x) * sin
        return torch.cat([x[..., :rd] * cos + _rot(x[..., :rd]) * sin, x[..., rd:]], dim=-1)

    @torch.no_grad()
    def forward(self, input_ids, cache: EagerTrimKVCache):
        c, w, D = self.c, self.w, self.head_dim
        x = F.embedding(input_ids, w["model.embed_tokens.weight"])
        seen = cache.get_seq_length()
        s = x.shape[1]
        cache_position = torch.arange(seen, seen + s)
        freqs = cache_position[:, None].float() * self.inv_freq[None, :]
        emb = torch.cat((freqs, freqs), dim=-1)
        cos, sin = emb.cos().to(x.dtype)[None, None], emb.sin().to(x.dtype)[None, None]
        g = c.num_attention_heads // c.num_key_value_heads
        nq, nkv = c.num_attention_heads * D, c.num_key_value_heads * D
        for l in range(c.num_hidden_layers):
            p = f"model.layers.{l}."
            h = _rms(x, w[p + "input_layernorm.weight"], c.rms_norm_eps)
            shp = (*h.shape[:-1], -1, D)
            if p + "self_attn.qkv_proj.weight" in w:
                q, k, v = self._lin(p + "self_attn.qkv_proj", h).split([nq, nkv, nkv], dim=-1)
                q, k, v = q.reshape(shp), k.reshape(shp), v.reshape(shp)
            else:
                q, k = self._lin(p + "self_attn.q_proj", h).view(shp), self._lin(p + "self_attn.k_proj", h).view(shp)
                v = self._lin(p + "self_attn.v_proj", h).view(shp)
            if p + "self_attn.q_norm.weight" in w:
                q = _rms(q, w[p + "self_attn.q_norm.weight"], c.rms_norm_eps)
                k = _rms(k, w[p + "self_attn.k_norm.weight"], c.rms_norm_eps)
            rw = self._gate(p, h).transpose(1, 2) if self.gate_kind == "rg" else None
            q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
            q, k = self._rope(q, cos, sin), self._rope(k, cos, sin)
            if rw is None:
                kv = torch.cat([k, v], dim=-1).transpose(1, 2)
                rw = self._gate(p, kv.reshape(kv.shape[0], kv.shape[1], -1)).transpose(1, 2)
            kk, vv, _, _, _ = cache.update(k, v, rw, cache_position, l)
            a = eager_attention(q, kk, vv, g, D ** -0.5)
            x = x + self._lin(p + "self_attn.o_proj", a.reshape(*h.shape[:-1], -1))
            h = _rms(x, w[p + "post_attention_layernorm.weight"], c.rms_norm_eps)
            if p + "mlp.gate_up_proj.weight" in w:
                gate, up = self._lin(p + "mlp.gate_up_proj", h).chunk(2, dim=-1)
                x = x + self._lin(p + "mlp.down_proj", up * F.silu(gate))
            else:
                x = x + self._lin(p + "mlp.down_proj", F.silu(self._lin(p + "mlp.gate_proj", h)) * self._lin(p + "mlp.up_proj", h))
        x = _rms(x, w["model.norm.weight"], c.rms_norm_eps)
        if c.compress_memory:
            cache.compress(strategy=c.compress_strategy, memory_size=c.memory_size, buffer_size=c.buffer_size)
        return F.linear(x[:, -1:, :], w["lm_head.weight"])


OracleQwen3 = OracleDecoder
