"""trimkv_b200 — the TRIM-KV memory-bounded KV-cache hot path on B200 (sm_100a).

Host code in Python/PyTorch (device memory, streams), arithmetic in hand-written CUDA behind
the C ABI of include/trimkv_b200.h.  Importing the package does not need a GPU; using it does.
"""
from .cache_utils import BatchedDynamicBudgetTrimKVCache, DynamicBudgetTrimKVCache, TrimKVCache
from .ops import update_flatten_view, update_flatten_view_triton
from .attn import TRIMKV_ATTENTION_IMPLEMENTATIONS, get_attention_interface
from .modeling_qwen3 import TrimKVQwen3Config, TrimKVQwen3ForCausalLM, TrimKVQwen3Model
from .modeling_llama import TrimKVLlamaConfig, TrimKVLlamaForCausalLM, TrimKVLlamaModel
from .modeling_phi3 import TrimKVPhi3Config, TrimKVPhi3ForCausalLM, TrimKVPhi3Model

__all__ = [
    "TrimKVCache", "DynamicBudgetTrimKVCache", "BatchedDynamicBudgetTrimKVCache", "update_flatten_view",
    "update_flatten_view_triton", "TRIMKV_ATTENTION_IMPLEMENTATIONS", "get_attention_interface",
    "TrimKVQwen3Config", "TrimKVQwen3ForCausalLM", "TrimKVQwen3Model",
    "TrimKVLlamaConfig", "TrimKVLlamaForCausalLM", "TrimKVLlamaModel",
    "TrimKVPhi3Config", "TrimKVPhi3ForCausalLM", "TrimKVPhi3Model",
]
