"""Tiny decoder configurations and a deterministic weight filler shared by the golden generator and the tests.

The model-level golden vectors (``model_<family>.npz``) are outputs of the reference's own model classes
run on CPU with these configurations and weights (see make_golden.py).  The tests rebuild the same weights
for this library's models through ``fill_state_dict``, so no weight tensor has to be committed: every
parameter is drawn from a NumPy generator seeded by the parameter's name.
"""
import zlib

import numpy as np

# Shared shape of the three families: 3 layers, 4 query / 2 KV heads of 128 dims, hidden 128, vocabulary 256.
_COMMON = dict(vocab_size=256, hidden_size=128, intermediate_size=256, num_hidden_layers=3, num_attention_heads=4,
               num_key_value_heads=2, head_dim=128, retention_gate_intermediate_size=32, retention_gate_bias_init=3.0,
               memory_size=64, buffer_size=16, compress_memory=True, compress_strategy="alpha", rms_norm_eps=1e-6,
               max_position_embeddings=4096, tie_word_embeddings=False)

FAMILIES = {
    "qwen3": dict(_COMMON, rope_theta=1e6, attention_bias=False),
    "llama": dict(_COMMON, rope_theta=5e5, attention_bias=True, mlp_bias=True),
    "phi3": dict(_COMMON, rope_theta=1e4),
}

PROMPT_LEN, DECODE_STEPS, BATCH = 100, 56, 2

# golden file suffix -> (family, config overrides, decode steps)
CASES = {
    "qwen3": ("qwen3", {}, DECODE_STEPS),
    "llama": ("llama", {}, DECODE_STEPS),
    "phi3": ("phi3", {}, DECODE_STEPS),
    "qwen3_rg2": ("qwen3", {"retention_gate": "rg2"}, 24),
    "qwen3_rg3": ("qwen3", {"retention_gate": "rg3"}, 24),
    "llama_rg2": ("llama", {"retention_gate": "rg2"}, 24),
    "phi3_partial_rotary": ("phi3", {"partial_rotary_factor": 0.5}, 24),
}


def _rng(name: str, seed: int):
    return np.random.default_rng([seed, zlib.crc32(name.encode())])


def fill_state_dict(shapes, seed: int = 0):
    """``{name: shape}`` -> ``{name: float32 array}``.  Linear weights ~ N(0, 1/fan_in), embeddings ~ N(0, 1), norm
    weights ~ 1 + 0.1 N(0,1), the retention gate's output bias ~ 3 + 0.5 N(0,1) (beta spread around 0.95), other
    biases ~ 0.1 N(0,1), so that activations are O(1) and the kept sets are not trivial; the LM head is scaled down so that logits stay within
    about 0.1."""
    out = {}
    for name in sorted(shapes):
        shape = tuple(shapes[name])
        r = _rng(name, seed)
        x = r.standard_normal(shape).astype(np.float32)
        if name.endswith("retention_gate.bias"):
            x = 3.0 + 0.5 * x
        elif name.endswith("norm.weight") or name.endswith("layernorm.weight"):
            x = 1.0 + 0.1 * x
        elif name.endswith(".bias"):
            x = 0.1 * x
        elif "embed_tokens" in name:
            pass
        elif name == "lm_head.weight":
            x = x * (0.03 / np.sqrt(shape[-1]))     # logits around 0.1: bf16 noise stays well below the 2e-2 tolerance
        elif "retention_gate.linear2" in name or "retention_gate.down_proj" in name or "retention_gate.up_proj" in name:
            x = x * (2.0 / np.sqrt(shape[-1]))      # a wider spread of gate logits
        else:
            x = x / np.sqrt(shape[-1])
        out[name] = x.astype(np.float32)
    return out


def prompt_ids(family: str, vocab: int):
    r = _rng("prompt:" + family, 0)
    return r.integers(0, vocab, size=(BATCH, PROMPT_LEN), dtype=np.int64)
