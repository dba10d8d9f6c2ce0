"""Attention registry with the reference's string-keyed interface.

Mirrors src/trimkv/attn/__init__.py:8-37 (``TRIMKV_ATTENTION_IMPLEMENTATIONS``,
``get_attention_interface``) and the call signature of
``batched_dynamic_kv_budget_attention_forward`` (src/trimkv/attn/flash_attn.py:79-89):

    fn(module, query[B,Hq,Q,D], key, value, attention_mask, scaling=None, dropout_p=0.0,
       flash_attn_kwargs={}, **kwargs) -> (attn_output[B,Q,Hq,D], None, None)

Decode (one query token, a cache that carries ``head_lens``) runs the split-KV CUDA kernel; the
prompt pass (dense K/V, Q > 1) is ordinary causal attention and stays in PyTorch.
"""
from __future__ import annotations

from typing import Callable, Dict

import torch
import torch.nn.functional as F

from . import ops

_workspaces: Dict[torch.device, torch.Tensor] = {}
_retired = []   # outgrown workspaces: kept alive because a captured CUDA graph may still hold their address

# Optional profiling hook: when set to a list, the decode path appends (start_event, end_event, batch, hkv)
# around each native attention call.  The benchmark uses it to time the kernel on the launching stream.
event_log = None


def _workspace(device, nbytes: int) -> torch.Tensor:
    """Scratch for the split-KV partials, one growing buffer per device.  A buffer that is outgrown is retired, not
    freed: a decode step captured in a CUDA graph has its address baked in and keeps writing there on replay.  Calls
    on one device are expected on one stream (they share the buffer)."""
    ws = _workspaces.get(device)
    if ws is None or ws.numel() < nbytes:
        if ws is not None:
            _retired.append(ws)
        ws = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[device] = ws
    return ws


# Several query tokens against a materialised cache (a piece of a chunked prefill, a follow-up prompt, multi-token
# decoding).  Timings on B200, batch 32, 16/8 heads, about 4100 cached tokens per head, ms per layer, by query rows per
# segment (new tokens x query heads per KV head):
#   rows   split-KV kernels (16 / 32 rows per CTA)   query-resident kernel   library causal   library with a length mask
#    16        0.19                                     0.16                    0.35             0.47
#    64        0.46                                     0.13                    0.37             0.78
#   128        0.90                                     0.13                    0.37             1.20
#   256        1.79                                     0.23                    0.64             2.29
#  1024        7.58                                     0.79                    0.90             7.91
# The split-KV kernels re-read the K/V chunk once per 16 / 32 rows but spread a segment over many CTAs; the
# query-resident kernel reads K/V once per 128 rows with one CTA per (segment, block of 128 rows).  So: the
# query-resident kernel whenever it gets enough CTAs to fill the GPU, up to 1024 rows where all heads have one length
# (the library's causal kernel catches up around there and is ahead on whole prompts) and without limit where the
# lengths differ between heads (the library would need a materialised mask); with few segments the split-KV kernels up
# to the limits below, then the library.  A dense prompt pass (no cache yet) stays with the library, which is about twice
# as fast there (1.44 PFLOP/s against 0.77 for the query-resident kernel at 8192 tokens).
MULTI_TOKEN_MAX_ROWS_UNIFORM = 32
MULTI_TOKEN_MAX_ROWS_RAGGED = 256
RESIDENT_MIN_CTAS = 96
RESIDENT_MAX_ROWS_UNIFORM = 1024


def _dense_causal(query, key, value, scaling):
    """Causal attention with bottom-right alignment over dense ``[B,Hkv,n,D]`` keys (prompt pass)."""
    ql, n = query.shape[2], key.shape[2]
    if ql == n:
        out = F.scaled_dot_product_attention(query, key, value, is_causal=True, scale=scaling, enable_gqa=True)
    else:
        mask = torch.ones(ql, n, dtype=torch.bool, device=query.device).tril(n - ql)
        out = F.scaled_dot_product_attention(query, key, value, attn_mask=mask, scale=scaling, enable_gqa=True)
    return out.transpose(1, 2)


def _ragged_causal(query, key, value, head_lens, scaling):
    """Multi-token queries over strided ``[B,Hkv,n_max,D]`` views whose segments differ in length (a second prompt
    appended to a budget-sharing cache).  Query row i of segment (b, h) sees keys ``j <= len[b,h] - Q + i``, the
    bottom-right alignment flash-attn's ``causal=True`` gives the reference (src/trimkv/attn/flash_attn.py:135-145).
    Not a decode-path kernel: the library attention is called with an explicit mask built from the lengths."""
    bsz, hq, ql, _ = query.shape
    hkv, n_max = key.shape[1], key.shape[2]
    lens = head_lens.view(bsz, hkv, 1, 1).to(torch.int64)
    j = torch.arange(n_max, device=query.device).view(1, 1, 1, n_max)
    i = torch.arange(ql, device=query.device).view(1, 1, ql, 1)
    mask = j <= lens - ql + i                                            # [B, Hkv, Q, n_max]
    mask = mask[:, :, None].expand(bsz, hkv, hq // hkv, ql, n_max).reshape(bsz, hq, ql, n_max)
    out = F.scaled_dot_product_attention(query, key, value, attn_mask=mask, scale=scaling, enable_gqa=True)
    # rows of an empty segment see nothing: zeros, as the decode kernel writes
    out = torch.where(mask.any(-1, keepdim=True), out, torch.zeros_like(out))
    return out.transpose(1, 2)


def tkv_attention_forward(
    module,
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    attention_mask=None,
    scaling: float = None,
    dropout_p: float = 0.0,
    flash_attn_kwargs: dict = {},
    **kwargs,  # retention_weights, kv_positions, offset, dropout, sliding_window, is_causal: accepted, unused
):
    bsz, hq, ql, dim = query.shape
    if scaling is None:
        scaling = dim ** -0.5  # the reference's varlen wrappers always use flash-attn's default (flash_attn.py:85)
    head_lens = flash_attn_kwargs.get("head_lens") if flash_attn_kwargs else None
    if head_lens is None or ql != 1:
        if key.dim() != 4:
            raise NotImplementedError("multi-token queries over a packed flat cache")
        hkv = key.shape[1]
        uniform = head_lens is not None and flash_attn_kwargs.get("uniform_lengths", False)
        limit = MULTI_TOKEN_MAX_ROWS_UNIFORM if uniform else MULTI_TOKEN_MAX_ROWS_RAGGED
        rows = ql * (hq // hkv)
        if (head_lens is not None and dim == 128
                and query.dtype in (torch.bfloat16, torch.float16) and key.stride(3) == 1 and key.stride(2) == dim
                and key.stride(0) == hkv * key.stride(1) and key.shape[0] * key.stride(0) // dim >= 128):
            # New tokens against the materialised cache: the tensor-core kernels (see the table above).
            resident = rows > 8 and (not uniform or rows <= RESIDENT_MAX_ROWS_UNIFORM) and (
                bsz * hkv * -(-rows // 128) >= RESIDENT_MIN_CTAS or (not uniform and rows > limit))
            if resident or rows <= limit:
                out = torch.empty(bsz, ql, hq, dim, dtype=query.dtype, device=query.device)
                run = ops.prefill_attn if resident else ops.decode_attn_multi
                run(query.transpose(1, 2), key, value, head_lens, key.stride(1) // dim, out, hkv, scaling,
                    key.shape[2], status=flash_attn_kwargs.get("status"))
                return out, None, None
        if head_lens is not None and not flash_attn_kwargs.get("uniform_lengths", False):
            return _ragged_causal(query, key, value, head_lens, scaling), None, None
        return _dense_causal(query, key, value, scaling), None, None

    q3 = query[:, :, 0, :]
    out = torch.empty(bsz, 1, hq, dim, dtype=query.dtype, device=query.device)
    if key.dim() == 4:
        # Strided views of the capacity-strided cache: the segment stride is the capacity.
        hkv, max_len = key.shape[1], key.shape[2]
        if key.stride(3) != 1 or key.stride(2) != dim or key.stride(0) != hkv * key.stride(1):
            raise ValueError("key is not a view of a capacity-strided cache")
        cap, seg_start = key.stride(1) // dim, None
    else:
        # Packed [sum n, D] layout of the reference's flat caches: segment starts are cu_seqlens_k.
        hkv = flash_attn_kwargs.get("num_kv_heads") or head_lens.shape[0] // bsz
        seg_start = flash_attn_kwargs["cu_seqlens_k"]
        max_len = flash_attn_kwargs.get("max_seqlen_k") or int(head_lens.max().item())
        cap = 0
    bound = flash_attn_kwargs.get("total_len_bound") if seg_start is None else None
    ws = _workspace(query.device, ops.decode_attn_workspace_bytes(bsz, hq, hkv, dim, max_len) if bound is None else
                    ops.decode_attn_workspace_bytes_ragged(bsz, hq, hkv, dim, max_len, bound))
    if event_log is not None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    ops.decode_attn(q3, key, value, head_lens, seg_start, cap, out, ws, hkv, scaling, max_len,
                    flash_attn_kwargs.get("status"), total_len_bound=bound)
    if event_log is not None:
        e1.record()
        event_log.append((e0, e1))
    return out, None, None


def dense_attention_forward(module, query, key, value, attention_mask=None, scaling=None, **kwargs):
    """Stand-in for the reference's wrapper around HF attention functions (attn/__init__.py:15-26)."""
    if scaling is None:
        scaling = query.shape[-1] ** -0.5
    return _dense_causal(query, key, value, scaling), None, None


TRIMKV_ATTENTION_IMPLEMENTATIONS: Dict[str, Callable] = {
    "tkv_b200": tkv_attention_forward,
    "db_attn_flash": tkv_attention_forward,
    "db_attn_flash_batched": tkv_attention_forward,
}


def register_with_transformers() -> None:
    """Makes the registry's names known to transformers' own table of attention functions, so that a config whose
    ``_attn_implementation`` is one of them passes ``PreTrainedModel``'s check at construction.  The models here
    resolve the name through ``get_attention_interface``; transformers never calls these entries itself."""
    try:
        from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS
    except ImportError:
        return
    for name, fn in TRIMKV_ATTENTION_IMPLEMENTATIONS.items():
        if name not in ALL_ATTENTION_FUNCTIONS:
            ALL_ATTENTION_FUNCTIONS.register(name, lambda *a, _fn=fn, **k: _fn(*a, **k)[:2])


def get_attention_interface(attn_impl: str, compile: bool = False) -> Callable:
    if compile:
        raise NotImplementedError("torch.compile is not used on this path")
    if attn_impl in TRIMKV_ATTENTION_IMPLEMENTATIONS:
        return TRIMKV_ATTENTION_IMPLEMENTATIONS[attn_impl]
    if attn_impl in ("sdpa", "eager", "attn_eager", "flash_attention_2"):
        return dense_attention_forward
    raise KeyError(f"unknown attention implementation {attn_impl!r}")
