"""The C-ABI library loads and exports every symbol the header declares, with matching ctypes signatures."""
import ctypes
import os
import re

import pytest

from trimkv_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "trimkv_b200.h")

_KIND = {"int": "i", "int64_t": "l", "float": "f", "size_t": "z"}
_CT = {ctypes.c_int: "i", ctypes.c_int64: "l", ctypes.c_float: "f", ctypes.c_size_t: "z", ctypes.c_void_p: "p",
       ctypes.c_char_p: "p"}


def _declared():
    text = re.sub(r"/\*.*?\*/", "", open(HEADER).read(), flags=re.S)
    out = {}
    for m in re.finditer(r"([\w\s\*]+?)\b(tkv_\w+)\s*\(([^;{]*?)\)\s*;", text):
        args = m.group(3).strip()
        kinds = []
        if args != "void":
            for a in args.split(","):
                a = a.strip()
                if "*" in a or "tkv_stream_t" in a:
                    kinds.append("p")
                else:
                    kinds.append(_KIND[a.replace("const ", "").split()[0]])
        out[m.group(2)] = kinds
    return out


@pytest.fixture(scope="module")
def built():
    return build.build()


def test_header_and_binding_agree():
    decl = _declared()
    assert set(decl) == set(_lib.SIGNATURES)
    for name, kinds in decl.items():
        assert [_CT[a] for a in _lib.SIGNATURES[name][1]] == kinds, name


def test_library_exports_every_symbol(built):
    handle = ctypes.CDLL(built)
    for name in _declared():
        assert hasattr(handle, name), name
    assert _lib.lib().tkv_version() >= 100
    assert _lib.lib().tkv_last_error() == b""


def test_argument_errors_are_reported_without_a_gpu(built):
    lib = _lib.lib()
    # NULL pointers and bad sizes are rejected on the host before any launch.
    rc = lib.tkv_evict(None, None, None, None, None, None, 1, 1, 8, 128, 0, 1, 4, 8, 8, None, None, None)
    assert rc == -1 and b"NULL" in lib.tkv_last_error()
    rc = lib.tkv_rebuild_cu_seqlens(None, None, 4, 2, None)
    assert rc == -1
    assert lib.tkv_decode_attn_workspace_bytes(0, 16, 8, 128, 100) == 0
    assert lib.tkv_decode_attn_workspace_bytes(2, 16, 8, 128, 4224) > 0
    # entry points added around the core path: same contract
    dummy = ctypes.create_string_buffer(4096)
    ptr = ctypes.cast(dummy, ctypes.c_void_p)
    rc = lib.tkv_evict_multi(ptr, ptr, ptr, ptr, ptr, None, 1, 1, 4224, 128, 0, 1, 4096, 4224, 4224, 0, 0, 64, ptr, 1 << 20,
                             None, None, None)
    assert rc == -2 and b"ctas_per_segment" in lib.tkv_last_error()          # more CTAs per segment than supported
    rc = lib.tkv_evict_multi(ptr, ptr, ptr, ptr, ptr, None, 1, 1, 4224, 128, 0, 1, 4096, 4224, 4224, 0, 0, 4, None, 0,
                             None, None, None)
    assert rc == -1 and b"workspace" in lib.tkv_last_error()
    assert lib.tkv_evict_multi_workspace_bytes(8, 4096, 16) == (2 * 8 * 16 + 3 * 8 + 1 + 8 * 4096) * 4
    # the ragged entry point's workspace holds the dense workspace plus one 8-byte item per possible chunk
    dense = lib.tkv_decode_attn_workspace_bytes(64, 32, 8, 128, 8192)
    ragged = lib.tkv_decode_attn_ragged_workspace_bytes(64, 32, 8, 128, 8192, 1_000_000)
    assert ragged >= dense + (1_000_000 // 256 + 512) * 8
    assert lib.tkv_decode_attn_multi_workspace_bytes(2, 16, 8, 128, 700, 1) == lib.tkv_decode_attn_workspace_bytes(2, 16, 8, 128, 700)
    assert lib.tkv_decode_attn_multi_workspace_bytes(2, 16, 8, 128, 700, 5) > lib.tkv_decode_attn_multi_workspace_bytes(2, 16, 8, 128, 700, 2)
    rc = lib.tkv_decode_attn_push(ptr, 0, 0, ptr, ptr, ptr, None, 4224, ptr, ptr, 1 << 20, 1, 2, 1, 128, 0, 0.1, 4224,
                                  None, None, 2, 0, 512, 0, None, None, None)
    assert rc == -1 and b"NULL" in lib.tkv_last_error()
    rc = lib.tkv_peer_wait(ptr, ptr, 9, 0, 0, None, None)
    assert rc == -1 and b"world" in lib.tkv_last_error()
    rc = lib.tkv_flat_scores(ptr, ptr, ptr, ptr, 4, 100, 128, 7, 1, 0, 100, ptr, None)
    assert rc == -1                                                            # unknown K/V dtype
    rc = lib.tkv_group_budget(ptr, ptr, ptr, 100, 1, 4000, 1, 0, 1, 10, 0, 0.0, 0, 0, 0, None, ptr, None, None)
    assert rc == -2 and b"segments per group" in lib.tkv_last_error()
    # the query-resident attention: head_dim 128 and 16-bit only, positive scale, capacity at least the stated length
    ok = (ptr, 4096, 2048, 128, ptr, ptr, None)
    assert lib.tkv_prefill_attn(*ok, 300, ptr, 1, 16, 8, 64, 0, 0.1, 300, 8, None, None) == -2      # head_dim 64
    assert lib.tkv_prefill_attn(*ok, 300, ptr, 1, 16, 8, 128, 2, 0.1, 300, 8, None, None) == -2     # fp32
    assert lib.tkv_prefill_attn(*ok, 300, ptr, 1, 16, 8, 128, 0, 0.0, 300, 8, None, None) == -1     # scale
    assert lib.tkv_prefill_attn(*ok, 200, ptr, 1, 16, 8, 128, 0, 0.1, 300, 8, None, None) == -1     # cap < max_len
    assert lib.tkv_prefill_attn(None, 4096, 2048, 128, ptr, ptr, None, 300, ptr, 1, 16, 8, 128, 0, 0.1, 300, 8, None, None) == -1
    assert lib.tkv_prefill_attn(*ok, 300, ptr, 0, 16, 8, 128, 0, 0.1, 300, 8, None, None) == 0      # empty batch: nothing to do
    # the GEMM with the SwiGLU prologue shares the envelope of tkv_skinny_gemm
    assert lib.tkv_skinny_gemm_swiglu(ptr, ptr, ptr, 33, 2048, 6144, 0, None, None) == -2            # more than 32 rows
    assert lib.tkv_skinny_gemm_swiglu(ptr, ptr, ptr, 8, 2048, 100, 0, None, None) == -2              # k not a multiple of 64
    assert lib.tkv_skinny_gemm_swiglu(None, ptr, ptr, 8, 2048, 128, 0, None, None) == -1
    # the allocation-free attention refuses what does not fit its built-in scratch before touching the device
    rc = lib.tkv_decode_attn_static(ptr, 8192, 128, ptr, ptr, ptr, None, 8192, ptr, 256, 64, 8, 128, 0, 1.0, 8192, None, None)
    assert rc == -2 and b"built-in array" in lib.tkv_last_error()


def test_cpu_tensors_are_refused():
    import torch
    from trimkv_b200 import TrimKVCache
    c = TrimKVCache(device="cpu")
    with pytest.raises(_lib.TrimKVNativeError):
        c.update(torch.zeros(1, 2, 3, 16), torch.zeros(1, 2, 3, 16), torch.zeros(1, 2, 3), torch.arange(3), 0)
