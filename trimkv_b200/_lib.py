"""ctypes binding of the C ABI declared in include/trimkv_b200.h.

The shared library is the product: there is no Python or CPU fallback.  If it has not
been built, ``lib()`` raises with the build command instead of degrading silently.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtrimkv_b200.so")

TKV_BF16, TKV_F16, TKV_F32 = 0, 1, 2

P, I, L, F = c_void_p, c_int, c_int64, c_float

# name -> (restype, argtypes); must list every symbol of include/trimkv_b200.h
SIGNATURES = {
    "tkv_version": (I, []),
    "tkv_last_error": (c_char_p, []),
    "tkv_append": (I, [P, P, P, P, P, P, P, P, L, L, L, P, I, L, L, L, P, L, L, L, I, I, I, I, L, I, P, P]),
    "tkv_evict_select": (I, [P, L, P, L, P, I, I, L, I, I, I, P, P, P, P]),
    "tkv_compact": (I, [P, P, P, P, L, P, P, L, L, L, P, L, P, L, P, L, P, P, P, I, I, I, I, I, I, P, P]),
    "tkv_evict": (I, [P, P, P, P, P, P, I, I, L, I, I, L, I, I, I, P, P, P]),
    "tkv_evict_ex": (I, [P, P, P, P, P, P, I, I, L, I, I, L, I, I, I, P, I, I, I, P, P, P, P]),
    "tkv_flat_scores": (I, [P, P, P, P, I, L, I, I, L, I, I, P, P]),
    "tkv_evict_multi_workspace_bytes": (L, [I, I, I]),
    "tkv_evict_multi": (I, [P, P, P, P, P, P, I, I, L, I, I, L, I, I, I, I, I, I, P, L, P, P, P]),
    "tkv_group_budget": (I, [P, P, P, L, I, I, I, L, L, L, I, F, I, I, I, P, P, P, P]),
    "tkv_flat_append_packed": (I, [P, P, P, P, I, I, L, L, P]),
    "tkv_rebuild_cu_seqlens": (I, [P, P, I, I, P]),
    "tkv_decode_attn_workspace_bytes": (c_size_t, [I, I, I, I, I]),
    "tkv_decode_attn": (I, [P, L, L, P, P, P, P, L, P, P, c_size_t, I, I, I, I, I, F, I, P, P]),
    "tkv_decode_attn_ragged_workspace_bytes": (c_size_t, [I, I, I, I, I, L]),
    "tkv_decode_attn_ragged": (I, [P, L, L, P, P, P, P, L, P, P, c_size_t, I, I, I, I, I, F, I, L, P, P]),
    "tkv_decode_attn_push": (I, [P, L, L, P, P, P, P, L, P, P, c_size_t, I, I, I, I, I, F, I, P, P, I, I, L, L, P, P, P]),
    "tkv_peer_wait": (I, [P, P, I, I, I, P, P]),
    "tkv_enable_peer_access": (I, [I]),
    "tkv_ipc_export": (I, [P, P, P]),
    "tkv_ipc_import": (I, [P, P]),
    "tkv_ipc_close": (I, [P]),
    "tkv_decode_attn_multi_workspace_bytes": (c_size_t, [I, I, I, I, I, I]),
    "tkv_decode_attn_multi": (I, [P, L, L, L, P, P, P, L, P, P, c_size_t, I, I, I, I, I, F, I, I, P, P]),
    "tkv_prefill_attn": (I, [P, L, L, L, P, P, P, L, P, I, I, I, I, I, F, I, I, P, P]),
    "tkv_decode_attn_static": (I, [P, L, L, P, P, P, P, L, P, I, I, I, I, I, F, I, P, P]),
    "tkv_decode_prep": (I, [P, L, P, P, F, P, P, P, P, I, P, P, P, P, P, P, P, P, L, I, I, I, I, I, I, P, P, P]),
    "tkv_add_rmsnorm": (I, [P, P, P, P, I, I, F, I, I, P, P]),
    "tkv_silu_mul": (I, [P, P, I, I, I, I, P, P]),
    "tkv_skinny_gemm_splits": (I, [I, I, I]),
    "tkv_skinny_gemm": (I, [P, P, P, I, I, I, I, P, P]),
    "tkv_skinny_gemm_swiglu": (I, [P, P, P, I, I, I, I, P, P]),
    "tkv_read_status": (I, [P, P]),
}

_lib = None


class TrimKVNativeError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise TrimKVNativeError(
                f"{LIB_PATH} is missing: build it with `python -m trimkv_b200.build` "
                "(needs nvcc; there is no fallback path)")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError if the library lacks a declared symbol
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = lib().tkv_last_error().decode("utf-8", "replace")
        raise TrimKVNativeError(f"{what} failed with code {rc}: {msg}")
