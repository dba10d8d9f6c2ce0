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


def test_cpu_tensors_are_refused():
    import torch
    from trimkv_b200 import TrimKVCache
    c = TrimKVCache(device="cpu")
    with pytest.raises(_lib.TrimKVNativeError):
        c.update(torch.zeros(1, 2, 3, 16), torch.zeros(1, 2, 3, 16), torch.zeros(1, 2, 3), torch.arange(3), 0)
