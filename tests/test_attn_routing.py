"""Which kernel serves a multi-token query: the host-side routing of `tkv_attention_forward`, checked on CPU with the
native calls replaced by recorders (no arithmetic happens here; the kernels themselves are compared with the oracle
in the GPU tests)."""
import pytest
import torch

from trimkv_b200 import attn as attn_mod


@pytest.fixture
def routes(monkeypatch):
    calls = []

    def recorder(name):
        def fn(*args, **kwargs):
            calls.append(name)
            if name in ("library_causal", "library_masked"):
                q = args[0]
                return torch.zeros(q.shape[0], q.shape[2], q.shape[1], q.shape[3], dtype=q.dtype)
        return fn
    monkeypatch.setattr(attn_mod.ops, "prefill_attn", recorder("query_resident"))
    monkeypatch.setattr(attn_mod.ops, "decode_attn_multi", recorder("split_kv"))
    monkeypatch.setattr(attn_mod, "_dense_causal", recorder("library_causal"))
    monkeypatch.setattr(attn_mod, "_ragged_causal", recorder("library_masked"))
    return calls


def _call(bsz, hq, hkv, ql, n, cap, uniform, dense=False):
    d = 128
    q = torch.zeros(bsz, hq, ql, d, dtype=torch.bfloat16)
    slab = torch.zeros(bsz, hkv, cap, d, dtype=torch.bfloat16)
    k = slab[:, :, :n]
    kw = {} if dense else {"head_lens": torch.full((bsz * hkv,), n, dtype=torch.int32), "uniform_lengths": uniform}
    out, _, _ = attn_mod.tkv_attention_forward(None, q, k, k, None, flash_attn_kwargs=kw)
    assert out.shape == (bsz, ql, hq, d)


@pytest.mark.parametrize("bsz,hq,hkv,ql,uniform,want", [
    (32, 16, 8, 3, True, "split_kv"),            # 6 rows: the decode kernel's multi-token form
    (32, 16, 8, 8, True, "query_resident"),      # 16 rows, 256 CTAs
    (32, 16, 8, 32, True, "query_resident"),     # 64 rows, 256 CTAs
    (32, 16, 8, 128, True, "query_resident"),    # 256 rows, 512 CTAs
    (32, 16, 8, 1024, True, "library_causal"),   # 2048 rows on a uniform cache: the library's causal kernel is ahead
    (32, 16, 8, 1024, False, "query_resident"),  # ... but not where the lengths differ (it would need a mask)
    (2, 4, 2, 12, True, "split_kv"),             # 24 rows, 4 segments: too few CTAs for the query-resident kernel
    (2, 4, 2, 40, True, "library_causal"),       # 80 rows, few segments, uniform
    (2, 4, 2, 40, False, "split_kv"),            # 80 rows, few segments, ragged: 32-row kernel up to 256 rows
    (2, 4, 2, 150, False, "query_resident"),     # 300 rows, ragged: never a materialised mask
])
def test_multi_token_routing(routes, bsz, hq, hkv, ql, uniform, want):
    _call(bsz, hq, hkv, ql, n=max(600, ql), cap=max(640, ql), uniform=uniform)
    assert routes == [want]


def test_dense_prompt_pass_stays_with_the_library(routes):
    _call(4, 16, 8, 300, n=300, cap=300, uniform=True, dense=True)
    assert routes == ["library_causal"]


def test_registry_names_and_unknown_implementation():
    for name in ("tkv_b200", "db_attn_flash", "db_attn_flash_batched"):
        assert attn_mod.get_attention_interface(name) is attn_mod.tkv_attention_forward
    assert attn_mod.get_attention_interface("sdpa") is attn_mod.dense_attention_forward
    with pytest.raises(KeyError):
        attn_mod.get_attention_interface("no_such_attention")
    with pytest.raises(NotImplementedError):
        attn_mod.get_attention_interface("tkv_b200", compile=True)
