"""Tensor-level wrappers over the C ABI: validate, pass raw pointers, launch on torch's current stream.

PyTorch is used for device memory and streams only; all arithmetic of the cache path runs in the
CUDA kernels of libtrimkv_b200.so.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib
from ._lib import TKV_BF16, TKV_F16, TKV_F32, check, lib

_DTYPE = {torch.bfloat16: TKV_BF16, torch.float16: TKV_F16, torch.float32: TKV_F32}


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPE[dt]
    except KeyError:
        raise TypeError(f"unsupported dtype {dt}") from None


def _stream(t: torch.Tensor) -> int:
    if not t.is_cuda:
        raise _lib.TrimKVNativeError("trimkv_b200 runs on CUDA tensors only (no CPU path)")
    return torch.cuda.current_stream(t.device).cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


# Kernels launched through this module since import (the benchmark reports the delta of a timed region).
launch_count = 0


def _count(n: int) -> None:
    global launch_count
    launch_count += n


def new_status(device) -> torch.Tensor:
    return torch.zeros(1, dtype=torch.int32, device=device)


def read_status(status: torch.Tensor) -> int:
    """Synchronises the current stream and returns (then clears) the device status word."""
    return lib().tkv_read_status(status.data_ptr(), _stream(status))


def append(k_cache, v_cache, beta_cache, pos_cache, seg_len, cu_seqlens,
           k_new, v_new, beta_new, pos_new, cap: int, status=None) -> None:
    """In-place append of ``k_new/v_new [B,H,S,D]``, ``beta_new [B,H,S]``, ``pos_new`` int64 ``[S]`` or ``[B,H,S]``."""
    b, h, s, d = k_new.shape
    if v_new.shape != k_new.shape or v_new.stride() != k_new.stride():
        v_new = v_new.contiguous(); k_new = k_new.contiguous()
    if k_new.stride(3) != 1:
        k_new = k_new.contiguous(); v_new = v_new.contiguous()
    if pos_new.dtype != torch.int64:
        pos_new = pos_new.to(torch.int64)
    if pos_new.dim() == 1:
        ps = (0, 0, pos_new.stride(0))
    else:
        pos_new = pos_new.expand(b, h, s)
        ps = pos_new.stride()
    if beta_new.shape != (b, h, s):
        raise ValueError(f"retention weights {tuple(beta_new.shape)} do not match keys {tuple(k_new.shape)}")
    rc = lib().tkv_append(
        k_cache.data_ptr(), v_cache.data_ptr(), beta_cache.data_ptr(), pos_cache.data_ptr(),
        seg_len.data_ptr(), _ptr(cu_seqlens),
        k_new.data_ptr(), v_new.data_ptr(), k_new.stride(0), k_new.stride(1), k_new.stride(2),
        beta_new.data_ptr(), dtype_code(beta_new.dtype), beta_new.stride(0), beta_new.stride(1), beta_new.stride(2),
        pos_new.data_ptr(), ps[0], ps[1], ps[2],
        b, h, s, d, cap, dtype_code(k_cache.dtype), _ptr(status), _stream(k_cache))
    check(rc, "tkv_append")
    _count(1 if s <= 8 else 2)


def evict(k_cache, v_cache, beta_cache, pos_cache, seg_len, cu_seqlens, group: int, nseg: int, cap: int,
          q_idx: int, memory_size: int, trigger_len: int, max_len: int, kept_idx_out=None, status=None) -> None:
    d = k_cache.shape[-1]
    rc = lib().tkv_evict(
        k_cache.data_ptr(), v_cache.data_ptr(), beta_cache.data_ptr(), pos_cache.data_ptr(),
        seg_len.data_ptr(), _ptr(cu_seqlens), group, nseg, cap, d, dtype_code(k_cache.dtype), q_idx,
        memory_size, trigger_len, max_len, _ptr(kept_idx_out), _ptr(status), _stream(k_cache))
    check(rc, "tkv_evict")
    _count(1 if cu_seqlens is None else 2)


def evict_select(beta, pos, seg_len, n_uniform: int, nseg: int, q_idx: int, memory_size: int,
                 trigger_len: int, max_len: int, kept_idx, kept_cnt, status=None) -> None:
    """beta f32 ``[nseg, n]`` (row stride taken from the tensor); pos i32 ``[nseg, n]`` or ``[n]`` (shared)."""
    if beta.dtype != torch.float32 or pos.dtype != torch.int32:
        raise TypeError("evict_select wants f32 log beta and i32 positions")
    pos_stride = 0 if pos.dim() == 1 else pos.stride(0)
    rc = lib().tkv_evict_select(
        beta.data_ptr(), beta.stride(0), pos.data_ptr(), pos_stride, _ptr(seg_len), n_uniform, nseg, q_idx,
        memory_size, trigger_len, max_len, kept_idx.data_ptr(), kept_cnt.data_ptr(), _ptr(status), _stream(beta))
    check(rc, "tkv_evict_select")
    _count(1)


def compact(k_dst, v_dst, beta_dst, pos_dst, cap: int, k_src, v_src, beta_src, pos_src, kept_idx, kept_cnt,
            seg_len, cu_seqlens, group: int, status=None) -> None:
    """Gather rows of dense ``k_src/v_src [B,H,n,D]`` listed in ``kept_idx [B*H, M]`` into a strided cache."""
    b, h, n, d = k_src.shape
    if v_src.stride() != k_src.stride() or k_src.stride(3) != 1:
        k_src = k_src.contiguous(); v_src = v_src.contiguous()
    pos_stride = 0 if pos_src.dim() == 1 else pos_src.stride(0)
    rc = lib().tkv_compact(
        k_dst.data_ptr(), v_dst.data_ptr(), beta_dst.data_ptr(), pos_dst.data_ptr(), cap,
        k_src.data_ptr(), v_src.data_ptr(), k_src.stride(0), k_src.stride(1), k_src.stride(2),
        beta_src.data_ptr(), beta_src.stride(0), pos_src.data_ptr(), pos_stride,
        _ptr(kept_idx), 0 if kept_idx is None else kept_idx.stride(0), _ptr(kept_cnt),
        seg_len.data_ptr(), _ptr(cu_seqlens), group, b, h, n, d, dtype_code(k_dst.dtype),
        _ptr(status), _stream(k_dst))
    check(rc, "tkv_compact")
    _count(1 if cu_seqlens is None else 2)


def rebuild_cu_seqlens(seg_len, cu_seqlens, nseg: int, group: int) -> None:
    check(lib().tkv_rebuild_cu_seqlens(seg_len.data_ptr(), cu_seqlens.data_ptr(), nseg, group, _stream(seg_len)),
          "tkv_rebuild_cu_seqlens")


def decode_attn_workspace_bytes(batch: int, hq: int, hkv: int, head_dim: int, max_len: int) -> int:
    return int(lib().tkv_decode_attn_workspace_bytes(batch, hq, hkv, head_dim, max_len))


def decode_attn_workspace_bytes_ragged(batch: int, hq: int, hkv: int, head_dim: int, max_len: int,
                                       total_len_bound: int) -> int:
    return int(lib().tkv_decode_attn_ragged_workspace_bytes(batch, hq, hkv, head_dim, max_len, total_len_bound))


def decode_attn(q, k_cache, v_cache, seg_len, seg_start, cap: int, out, workspace, hkv: int, scale: float,
                max_len: int, status=None, total_len_bound=None, packed_rows=None) -> None:
    """q ``[B,Hq,D]`` (any batch/head strides), out ``[B,Hq,D]`` contiguous, workspace uint8.
    ``total_len_bound``: host-known bound on ``seg_len.sum()`` for ragged lengths (sizes the grid by tokens instead of
    by ``max_len``); the workspace must then have ``decode_attn_workspace_bytes_ragged`` bytes.
    With ``seg_start`` (packed ``[sum n, D]`` K/V) the C entry point takes the packed row count in place of ``cap``:
    ``packed_rows`` (default: the K tensor's first dimension; 0 = not stated, which selects the CUDA-core kernel)."""
    b, hq, d = q.shape
    if q.stride(2) != 1:
        q = q.contiguous()
    if seg_start is not None:
        cap = int(packed_rows) if packed_rows is not None else (k_cache.shape[0] if k_cache.dim() == 2 else 0)
    if total_len_bound is not None:
        rc = lib().tkv_decode_attn_ragged(
            q.data_ptr(), q.stride(0), q.stride(1), k_cache.data_ptr(), v_cache.data_ptr(),
            seg_len.data_ptr(), _ptr(seg_start), cap, out.data_ptr(), workspace.data_ptr(), workspace.numel(),
            b, hq, hkv, d, dtype_code(k_cache.dtype), float(scale), max_len, int(total_len_bound), _ptr(status), _stream(q))
        check(rc, "tkv_decode_attn_ragged")
        _count(3)
        return
    rc = lib().tkv_decode_attn(
        q.data_ptr(), q.stride(0), q.stride(1), k_cache.data_ptr(), v_cache.data_ptr(),
        seg_len.data_ptr(), _ptr(seg_start), cap, out.data_ptr(), workspace.data_ptr(), workspace.numel(),
        b, hq, hkv, d, dtype_code(k_cache.dtype), float(scale), max_len, _ptr(status), _stream(q))
    check(rc, "tkv_decode_attn")
    _count(2)


def decode_attn_multi(q, k_cache, v_cache, seg_len, cap: int, out, hkv: int, scale: float, max_len: int,
                      workspace=None, status=None):
    """q ``[B,Q,Hq,D]`` (any batch/token/head strides) against caches that already hold the Q new tokens; out
    ``[B,Q,Hq,D]`` contiguous; bottom-right aligned causal mask per segment."""
    b, ql, hq, d = q.shape
    if q.stride(3) != 1:
        q = q.contiguous()
    if workspace is None:
        workspace = torch.empty(lib().tkv_decode_attn_multi_workspace_bytes(b, hq, hkv, d, max_len, ql), dtype=torch.uint8,
                                device=q.device)
    rc = lib().tkv_decode_attn_multi(
        q.data_ptr(), q.stride(0), q.stride(1), q.stride(2), k_cache.data_ptr(), v_cache.data_ptr(), seg_len.data_ptr(), cap,
        out.data_ptr(), workspace.data_ptr(), workspace.numel(), b, hq, hkv, d, dtype_code(k_cache.dtype), float(scale),
        max_len, ql, _ptr(status), _stream(q))
    check(rc, "tkv_decode_attn_multi")
    _count(2)


def prefill_attn(q, k_cache, v_cache, seg_len, cap: int, out, hkv: int, scale: float, max_len: int, status=None):
    """q ``[B,Q,Hq,D]`` (any batch/token/head strides) against capacity-strided caches that already hold the Q new
    tokens (``seg_len`` None: every segment holds ``max_len`` tokens, e.g. a dense prompt with ``cap`` = S); out
    ``[B,Q,Hq,D]`` contiguous; bottom-right aligned causal mask per segment.  Query-resident kernel, no workspace."""
    b, ql, hq, d = q.shape
    if q.stride(3) != 1:
        q = q.contiguous()
    rc = lib().tkv_prefill_attn(
        q.data_ptr(), q.stride(0), q.stride(1), q.stride(2), k_cache.data_ptr(), v_cache.data_ptr(), _ptr(seg_len), cap,
        out.data_ptr(), b, hq, hkv, d, dtype_code(k_cache.dtype), float(scale), max_len, ql, _ptr(status), _stream(q))
    check(rc, "tkv_prefill_attn")
    _count(1)


def decode_attn_push(q, k_cache, v_cache, seg_len, cap: int, out, workspace, hkv: int, scale: float, max_len: int,
                     peer_out, peer_flags, world: int, rank: int, row_stride: int, col_offset: int, sync_state,
                     status=None) -> None:
    """:func:`decode_attn` whose merge step stores into every rank's gathered buffer and raises this rank's flag on
    the peers.  ``peer_out`` / ``peer_flags``: ``ctypes`` arrays of ``world`` device pointers."""
    b, hq, d = q.shape
    if q.stride(2) != 1:
        q = q.contiguous()
    rc = lib().tkv_decode_attn_push(
        q.data_ptr(), q.stride(0), q.stride(1), k_cache.data_ptr(), v_cache.data_ptr(),
        seg_len.data_ptr(), None, cap, out.data_ptr(), workspace.data_ptr(), workspace.numel(),
        b, hq, hkv, d, dtype_code(k_cache.dtype), float(scale), max_len,
        peer_out, peer_flags, world, rank, row_stride, col_offset, sync_state.data_ptr(), _ptr(status), _stream(q))
    check(rc, "tkv_decode_attn_push")
    _count(2)


def enable_peer_access(peer_device: int) -> None:
    check(lib().tkv_enable_peer_access(int(peer_device)), "tkv_enable_peer_access")


def ipc_export(t: torch.Tensor):
    """``(handle bytes, offset)`` under which other rank processes of this box can map ``t``'s allocation."""
    import ctypes
    handle, off = ctypes.create_string_buffer(64), ctypes.c_int64(0)
    check(lib().tkv_ipc_export(t.data_ptr(), handle, ctypes.byref(off)), "tkv_ipc_export")
    return handle.raw, int(off.value)


_ipc_bases = {}   # (device, handle) -> [base address, users]: an allocation is mapped once per process and device


def ipc_import(handle: bytes) -> int:
    """Maps an exported allocation with the current device; returns its base address in this process.  A handle that
    is already mapped is not opened again (one mapping per handle and process); ``ipc_release`` undoes one import."""
    import ctypes
    key = (torch.cuda.current_device(), handle)
    if key not in _ipc_bases:
        base = ctypes.c_void_p(0)
        check(lib().tkv_ipc_import(ctypes.create_string_buffer(handle, 64), ctypes.byref(base)), "tkv_ipc_import")
        _ipc_bases[key] = [int(base.value), 0]
    _ipc_bases[key][1] += 1
    return _ipc_bases[key][0]


def ipc_release(handle: bytes) -> None:
    """Drops one user of an imported allocation; the mapping is closed when the last one is gone."""
    import ctypes
    key = (torch.cuda.current_device(), handle)
    entry = _ipc_bases.get(key)
    if entry is None:
        return
    entry[1] -= 1
    if entry[1] <= 0:
        del _ipc_bases[key]
        check(lib().tkv_ipc_close(ctypes.c_void_p(entry[0])), "tkv_ipc_close")


def peer_wait(flags, sync_state, world: int, rank: int, status=None, max_polls: int = 0) -> None:
    """Holds the stream until every peer has raised its flag for this rank's next exchange.  Bounded: after
    ``max_polls`` polls (default about four seconds) the status word reports a timeout and the stream carries on."""
    rc = lib().tkv_peer_wait(flags.data_ptr(), sync_state.data_ptr(), world, rank, max_polls, _ptr(status), _stream(flags))
    check(rc, "tkv_peer_wait")
    _count(1)


def decode_prep(qkvg, q_norm_w, k_norm_w, eps: float, cos, sin, gate_w2, gate_bias, pos, q_out,
                k_cache, v_cache, beta_cache, pos_cache, seg_len, cu_seqlens, cap: int, hq: int, hkv: int,
                status=None, in_splits: int = 0, in_bias=None) -> None:
    """Fused q/k-norm + RoPE + retention-gate tail + append for one new token per request (head_dim 128).
    ``q_norm_w`` / ``k_norm_w`` are both None for families without a per-head norm (Llama, Phi-3).
    ``qkvg`` is ``[B, cols]`` in the model dtype, or (``in_splits`` > 0) the fp32 ``[splits, B, cols]`` of skinny_gemm."""
    b, cols = qkvg.shape[-2], qkvg.shape[-1]
    rc = lib().tkv_decode_prep(
        qkvg.data_ptr(), cols if in_splits else qkvg.stride(0), _ptr(q_norm_w), _ptr(k_norm_w), float(eps),
        cos.data_ptr(), sin.data_ptr(), gate_w2.data_ptr(), gate_bias.data_ptr(), gate_w2.shape[1],
        pos.data_ptr(), q_out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), beta_cache.data_ptr(),
        pos_cache.data_ptr(), seg_len.data_ptr(), _ptr(cu_seqlens), cap, b, hq, hkv, 128,
        dtype_code(q_out.dtype), in_splits, _ptr(in_bias), _ptr(status), _stream(qkvg))
    check(rc, "tkv_decode_prep")
    _count(1)


def add_rmsnorm(residual, delta, weight, out, eps: float, in_splits: int = 0, in_bias=None) -> None:
    rows, cols = residual.shape
    rc = lib().tkv_add_rmsnorm(residual.data_ptr(), _ptr(delta), weight.data_ptr(), out.data_ptr(), rows, cols,
                               float(eps), dtype_code(residual.dtype), in_splits, _ptr(in_bias), _stream(residual))
    check(rc, "tkv_add_rmsnorm")
    _count(1)


def silu_mul(gate_up, out, in_splits: int = 0, in_bias=None) -> None:
    rows, two_inter = gate_up.shape[-2], gate_up.shape[-1]
    rc = lib().tkv_silu_mul(gate_up.data_ptr(), out.data_ptr(), rows, two_inter // 2, dtype_code(out.dtype),
                            in_splits, _ptr(in_bias), _stream(gate_up))
    check(rc, "tkv_silu_mul")
    _count(1)


def skinny_gemm_splits(m: int, n: int, k: int) -> int:
    """Number of fp32 partial sums tkv_skinny_gemm produces for this shape; 0 = shape not supported."""
    return int(lib().tkv_skinny_gemm_splits(m, n, k))


def skinny_gemm(x, w, partial, status=None) -> int:
    """``partial [splits, M, N]`` fp32 with ``sum(partial, 0) == x [M, K] @ w [N, K].T``; returns ``splits``."""
    m, k = x.shape
    n = w.shape[0]
    if not (x.is_contiguous() and w.is_contiguous() and partial.is_contiguous() and partial.dtype == torch.float32):
        raise ValueError("skinny_gemm wants contiguous x, w and an fp32 contiguous partial buffer")
    rc = lib().tkv_skinny_gemm(x.data_ptr(), w.data_ptr(), partial.data_ptr(), m, n, k, dtype_code(x.dtype),
                               _ptr(status), _stream(x))
    check(rc, "tkv_skinny_gemm")
    _count(1)
    return skinny_gemm_splits(m, n, k)


def skinny_gemm_swiglu(gate_up, w, partial, status=None) -> int:
    """:func:`skinny_gemm` over ``x = SiLU(gate_up[:, :K]) * gate_up[:, K:]`` computed inside the kernel
    (``gate_up [M, 2K]``, ``w [N, K]``): the MLP's activation and down projection in one launch."""
    m, two_k = gate_up.shape
    n, k = w.shape
    if two_k != 2 * k:
        raise ValueError(f"gate_up has {two_k} columns, the weight wants 2 x {k}")
    if not (gate_up.is_contiguous() and w.is_contiguous() and partial.is_contiguous() and partial.dtype == torch.float32):
        raise ValueError("skinny_gemm_swiglu wants contiguous gate_up, w and an fp32 contiguous partial buffer")
    rc = lib().tkv_skinny_gemm_swiglu(gate_up.data_ptr(), w.data_ptr(), partial.data_ptr(), m, n, k,
                                      dtype_code(gate_up.dtype), _ptr(status), _stream(gate_up))
    check(rc, "tkv_skinny_gemm_swiglu")
    _count(1)
    return skinny_gemm_splits(m, n, k)


def evict_ex(k_cache, v_cache, beta_cache, pos_cache, seg_len, cu_seqlens, group: int, nseg: int, cap: int,
             q_idx: int, max_len: int, keep_cnt, protect_last: int = 0, memory_size: int = 1, trigger_len: int = 0,
             kept_idx_out=None, kept_stride: int = 0, status=None, knorm: bool = False, score_dtype: int = 0,
             scores=None) -> None:
    """In-place eviction with a keep count per segment (``keep_cnt`` int32 ``[nseg]``) and/or a protected tail.
    ``score_dtype``: 0 fp32, 1 bf16, 2 f16 (the dtype the retention score is computed in)."""
    d = k_cache.shape[-1]
    rc = lib().tkv_evict_ex(
        k_cache.data_ptr(), v_cache.data_ptr(), beta_cache.data_ptr(), pos_cache.data_ptr(),
        seg_len.data_ptr(), _ptr(cu_seqlens), group, nseg, cap, d, dtype_code(k_cache.dtype), q_idx,
        memory_size, trigger_len, max_len, _ptr(keep_cnt), protect_last, kept_stride,
        (1 if knorm else 0) | (score_dtype << 8), _ptr(scores), _ptr(kept_idx_out),
        _ptr(status), _stream(k_cache))
    check(rc, "tkv_evict_ex")
    _count(1 if cu_seqlens is None else 2)


def evict_multi_workspace(nseg: int, memory_size: int, ctas_per_segment: int, device) -> torch.Tensor:
    """Scratch for :func:`evict_multi` (contents irrelevant between calls; one stream at a time)."""
    nbytes = lib().tkv_evict_multi_workspace_bytes(nseg, memory_size, ctas_per_segment)
    return torch.empty(max(nbytes, 4) // 4, dtype=torch.int32, device=device)


def evict_multi(k_cache, v_cache, beta_cache, pos_cache, seg_len, cu_seqlens, group: int, nseg: int, cap: int,
                q_idx: int, memory_size: int, trigger_len: int, max_len: int, ctas_per_segment: int, workspace,
                protect_last: int = 0, knorm: bool = False, kept_idx_out=None, status=None) -> None:
    """:func:`evict` with ``ctas_per_segment`` CTAs sharing each evicting segment (identical result)."""
    d = k_cache.shape[-1]
    rc = lib().tkv_evict_multi(
        k_cache.data_ptr(), v_cache.data_ptr(), beta_cache.data_ptr(), pos_cache.data_ptr(),
        seg_len.data_ptr(), _ptr(cu_seqlens), group, nseg, cap, d, dtype_code(k_cache.dtype), q_idx,
        memory_size, trigger_len, max_len, protect_last, 1 if knorm else 0, ctas_per_segment,
        _ptr(workspace), 0 if workspace is None else workspace.numel() * workspace.element_size(),
        _ptr(kept_idx_out), _ptr(status), _stream(k_cache))
    check(rc, "tkv_evict_multi")
    n = 1 if ctas_per_segment <= 1 else 2
    _count(n if cu_seqlens is None else n + 1)


def flat_scores(k_cache, beta_cache, pos_cache, seg_len, nseg: int, cap: int, q_idx: int, max_len: int, scores_out,
                knorm: bool = True, score_dtype: int = 0) -> None:
    """Scores of every live row (fp32 array of ``nseg*cap``) for the strategies that read K ("knorm_alpha" on the
    flat caches: the norm is clamped at 1e-12 as the reference does there)."""
    rc = lib().tkv_flat_scores(k_cache.data_ptr(), beta_cache.data_ptr(), pos_cache.data_ptr(), seg_len.data_ptr(),
                               nseg, cap, k_cache.shape[-1], dtype_code(k_cache.dtype), q_idx,
                               (2 if knorm else 0) | (score_dtype << 8), max_len, scores_out.data_ptr(),
                               _stream(k_cache))
    check(rc, "tkv_flat_scores")
    _count(1)


def group_budget(beta_cache, pos_cache, seg_len, cap: int, groups: int, inner: int, n_outer: int, outer_stride: int,
                 q_idx: int, k_total: int, keep_cnt, threshold=None, floor_mode: int = 0, floor_cnt: int = 0,
                 status=None, score_dtype: int = 0, scores=None) -> None:
    """Per-segment keep counts when ``k_total`` rows (or all rows scoring >= ``threshold``) are kept per group."""
    rc = lib().tkv_group_budget(
        beta_cache.data_ptr(), pos_cache.data_ptr(), seg_len.data_ptr(), cap, groups, inner, n_outer, outer_stride,
        q_idx, k_total, 0 if threshold is None else 1, 0.0 if threshold is None else float(threshold),
        floor_mode, floor_cnt, score_dtype, _ptr(scores), keep_cnt.data_ptr(), _ptr(status), _stream(beta_cache))
    check(rc, "tkv_group_budget")
    _count(1)


def update_flatten_view(cache: torch.Tensor, state: torch.Tensor, headlens: torch.Tensor,
                        cu_headlens: torch.Tensor) -> torch.Tensor:
    """Functional packed append with the contract of the reference's ``update_flatten_view_triton``
    (src/trimkv/triton/db_cache_utils.py:86-186): ``cache [origin_len, D]`` + ``state [1, H, S, D]`` ->
    ``out [origin_len + H*S, D]``; same argument checks, no host synchronisation."""
    assert cache.is_cuda and state.is_cuda, "Tensors must be on CUDA device"
    assert headlens.is_cuda and cu_headlens.is_cuda, "Index tensors must be on CUDA"
    assert headlens.dtype == torch.int32, "headlens must be int32"
    assert cu_headlens.dtype == torch.int32, "cu_headlens must be int32"
    assert cache.dtype == state.dtype, "cache/state dtypes must match"
    assert cache.is_contiguous(), "cache must be contiguous [origin_len, D]"
    assert headlens.is_contiguous() and cu_headlens.is_contiguous(), "index tensors must be contiguous"
    assert state.ndim == 4, "state must be [B, H, state_len, D]"
    b, h, s, d_state = state.shape
    assert b == 1, "This kernel currently assumes B == 1"
    origin_len, d = cache.shape
    assert d == d_state, "cache and state last dim (D) must match"
    assert headlens.shape[0] == h, "headlens must be length H"
    assert cu_headlens.numel() == h + 1, "cu_headlens must be length H+1"
    assert state.is_contiguous(), "state must be contiguous [B, H, state_len, D]"
    out = torch.empty((origin_len + h * s, d), dtype=cache.dtype, device=cache.device)
    rc = lib().tkv_flat_append_packed(cache.data_ptr(), state.data_ptr(), cu_headlens.data_ptr(), out.data_ptr(),
                                      h, s, origin_len, d * cache.element_size(), _stream(cache))
    check(rc, "tkv_flat_append_packed")
    _count(1)
    return out


update_flatten_view_triton = update_flatten_view  # the reference's name for the same operation
