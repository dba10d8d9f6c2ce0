"""The host side of `TrimKVCache` on CPU: the Python class with its native calls replaced by the stand-ins of
tests/host_emulation.py, against the golden vectors made by the reference's own class.  Covers what the class decides by
itself (slab sizing, the two forms of the prompt hand-off, counters, the compress trigger, launch-form choice, views,
batch operations); the kernels are compared with the oracle on a GPU."""
import os

import numpy as np
import pytest
import torch

from tests import host_emulation as emu


@pytest.fixture
def host_cache(monkeypatch):
    from trimkv_b200 import cache_utils
    monkeypatch.setattr(cache_utils, "ops", emu)
    monkeypatch.setattr(torch.cuda, "is_current_stream_capturing", lambda: False)   # asked before the slabs grow
    emu.multi_calls.clear()
    return cache_utils.TrimKVCache


@pytest.fixture
def host_flat_caches(host_cache):
    from trimkv_b200 import cache_utils
    return cache_utils.BatchedDynamicBudgetTrimKVCache, cache_utils.DynamicBudgetTrimKVCache


@pytest.mark.parametrize("eager_handoff", [False, True])
def test_config1_lockstep_host_logic(host_cache, golden_dir, eager_handoff):
    """benchmark-spec configs[0] (batch 1, 8 KV heads, fp32, M 512, B 128, 4096-token prefill + 256 steps) through the
    real class: kept positions at every eviction and the length after every step equal the reference's own run, with
    the prompt reduced at compress() time or, with the constructor hints, inside update()."""
    g = np.load(os.path.join(golden_dir, "config1_lockstep.npz"))
    M, B, S, T = int(g["M"]), int(g["B"]), int(g["S"]), int(g["T"])
    logb = torch.from_numpy(g["log_beta"])[None]
    H, D = logb.shape[1], 16
    cache = host_cache(device="cpu", **(dict(memory_size=M, buffer_size=B, num_layers=1) if eager_handoff else {}))
    payload = torch.randn(S + T, D, generator=torch.Generator().manual_seed(0))
    lens, ev = [], 0
    for t in range(T + 1):
        lo, hi = (0, S) if t == 0 else (S + t - 1, S + t)
        k = emu.on_device(payload[lo:hi][None, None].expand(1, H, hi - lo, D).contiguous())
        kk, vv, bb, pp, kw = cache.update(k, (k * 2).contiguous(), logb[:, :, lo:hi].contiguous(), torch.arange(lo, hi), 0)
        before = cache.get_cache_length(0)
        cache.compress(memory_size=M, buffer_size=B)
        lens.append(cache.get_cache_length(0))
        if (t == 0 and eager_handoff) or lens[-1] != before:
            pos = cache.kv_positions[0][0]
            assert np.array_equal(pos.numpy(), g["kept_positions"][ev]), t
            assert torch.equal(cache.key_cache[0][0], payload[pos.long()])
            assert torch.equal(cache.value_cache[0][0], payload[pos.long()] * 2)
            assert cache.head_lens[0].tolist() == [M] * H
            assert cache.cu_seqlens_k[0].tolist() == list(range(0, H * M + 1, M))
            ev += 1
    assert np.array_equal(np.asarray(lens, np.int32), g["lens"])
    assert ev == g["kept_positions"].shape[0]
    assert cache._cap == M + B                        # the slab is sized once, at M + B rows per head
    assert cache.get_seq_length() == S + T and cache.get_total_cached_tokens() == lens[-1] * H
    assert emu.multi_calls and all(n == H for n, _ in emu.multi_calls)   # 8 segments: several CTAs per segment
    cache.check_status()


def test_growth_without_eviction_and_trigger_semantics(host_cache):
    """No compress(): the slabs double when a segment would overflow.  With compress(): nothing happens below M + B,
    and the layer falls back to exactly M at M + B (src/trimkv/cache_utils.py:157)."""
    H, D = 2, 8
    gen = torch.Generator().manual_seed(1)
    cache = host_cache(device="cpu")
    for t in range(700):
        n = 5 if t == 0 else 1
        k = emu.on_device(torch.randn(2, H, n, D, generator=gen))
        cache.update(k, k.clone(), torch.zeros(2, H, n) - 0.1, torch.arange(cache.get_seq_length(), cache.get_seq_length() + n), 0)
    assert cache.get_cache_length(0) == 704 and cache._cap >= 704
    assert cache.kv_positions[0][1, 1].tolist() == list(range(704))
    cache.check_status()
    cache = host_cache(device="cpu")
    lens = []
    for t in range(60):
        k = emu.on_device(torch.randn(1, H, 1, D, generator=gen))
        cache.update(k, k.clone(), -torch.rand(1, H, 1, generator=gen), torch.arange(t, t + 1), 0)
        cache.compress(memory_size=16, buffer_size=4)
        lens.append(cache.get_cache_length(0))
    assert lens[:19] == list(range(1, 20)) and lens[19] == 16 and lens[20:24] == [17, 18, 19, 16]


def test_batch_split_and_select_keep_rows_and_counters(host_cache):
    gen = torch.Generator().manual_seed(2)
    Bt, H, D, S = 4, 2, 8, 12
    cache = host_cache(device="cpu")
    k = emu.on_device(torch.randn(Bt, H, S, D, generator=gen))
    cache.update(k, (k + 1).contiguous(), -torch.rand(Bt, H, S, generator=gen), torch.arange(S), 0)
    parts = cache.batch_split(Bt, 2)
    assert len(parts) == 2 and all(p.get_cache_length(0) == S for p in parts)
    assert torch.equal(parts[1].key_cache[0], torch.Tensor(k[2:4]))
    cache.batch_select_indices(torch.tensor([3, 0]))
    assert torch.equal(cache.key_cache[0], torch.Tensor(k[[3, 0]]))
    assert torch.equal(cache.value_cache[0], torch.Tensor(k[[3, 0]]) + 1)
    assert cache.get_seq_length() == S and len(cache) == 1
    with pytest.raises(KeyError):
        cache[1]
    logs = cache.log()
    assert logs[0]["seen_tokens"] == S and logs[0]["kv_positions"].dtype == torch.int64


def test_one_piece_prompt_beyond_the_selection_limit_is_refused_with_advice(host_cache):
    from trimkv_b200.cache_utils import MAX_ONE_PIECE_PROMPT
    n = MAX_ONE_PIECE_PROMPT + 1
    cache = host_cache(device="cpu")
    k = emu.on_device(torch.zeros(1, 1, n, 2))
    cache.update(k, k, torch.zeros(1, 1, n), torch.arange(n), 0)
    with pytest.raises(ValueError, match="prefill_chunk_size"):
        cache.compress(memory_size=64, buffer_size=8)


@pytest.mark.parametrize("ci", range(7))
def test_flat_budget_classes_host_logic(host_flat_caches, golden_dir, ci):
    """The budget-sharing classes' own decisions (when a layer or a request fires, the group shapes and budgets they ask
    for, the floor arithmetic they pass on, the read-back after an eviction) against the reference's classes: head
    lengths after every step and kept positions at three steps, for `alpha`, `layer_wise_alpha` (with and without a
    floor), `alpha_threshold` and the batch-1 class."""
    batched_cls, single_cls = host_flat_caches
    g = np.load(os.path.join(golden_dir, "flat_budget.npz"))
    L, B, H, D, S, T, M, Bf = [int(x) for x in g["meta"]]
    kind, strategy, floor, thr = str(g["cases"][ci]).split("|")
    floor, thr = float(floor), float(thr)
    logb = torch.from_numpy(g[f"c{ci}_logb"])
    bsz = logb.shape[1]
    cache = (batched_cls if kind == "batched" else single_cls)(device="cpu")
    for t in range(T + 1):
        lo, hi = (0, S) if t == 0 else (S + t - 1, S + t)
        for l in range(L):
            k = emu.on_device((torch.arange(lo, hi, dtype=torch.float32)[None, None, :, None] + 1000 * l)
                              .expand(bsz, H, hi - lo, D).contiguous())
            cache.update(k, (-k).contiguous(), logb[l, :, :, lo:hi].contiguous(), torch.arange(lo, hi), l)
        cache.compress(strategy=strategy, memory_size=M, buffer_size=Bf, floor_budget_ratio=floor, alpha_threshold=thr,
                       num_layers=L, num_key_value_heads=H)
        got = torch.stack([cache.head_lens[l] for l in range(L)]).numpy()
        assert np.array_equal(got, g[f"c{ci}_lens"][t]), (ci, t)
        assert cache.get_total_cached_tokens() == int(g[f"c{ci}_lens"][t].sum())
        if t in (0, T // 2, T):
            for l in range(L):
                kp, vp, bp, pp = cache.packed(l)
                assert np.array_equal(pp[:, 0].numpy(), g[f"c{ci}_pos_t{t}_l{l}"]), (ci, t, l)
                assert torch.equal(torch.Tensor(kp[:, 0]), pp[:, 0].float() + 1000.0 * l)
    cache.check_status()


def test_caches_are_freed_by_their_last_reference(host_flat_caches, host_cache):
    """No reference cycle inside a cache: gigabytes of slabs must not wait for the cycle collector."""
    import gc
    import weakref
    gc.collect()
    gc.disable()
    try:
        for cls in (host_cache,) + tuple(host_flat_caches):
            c = cls(device="cpu")
            k = emu.on_device(torch.randn(1, 2, 10, 16))
            c.update(k, k.clone(), emu.on_device(torch.zeros(1, 2, 10)), torch.arange(10), 0)
            c.compress(strategy="alpha", memory_size=4, buffer_size=2, num_layers=1, num_key_value_heads=2)
            views = c.key_cache
            assert views[0].shape[-1] == 16
            alive = weakref.ref(c)
            del c
            assert alive() is None, cls.__name__
            with pytest.raises(ReferenceError):
                views[0]
    finally:
        gc.enable()


def test_counter_snapshot_covers_the_row_totals_of_the_flat_classes(host_flat_caches):
    """A CUDA graph capture runs the host side of a decode step without its kernels and then puts the counters back;
    for the budget-sharing classes that includes the per-layer row totals compress() triggers on."""
    for cls in host_flat_caches:
        c = cls(device="cpu")
        k = emu.on_device(torch.randn(1, 2, 10, 16))
        for l in range(2):
            c.update(k, k.clone(), emu.on_device(torch.zeros(1, 2, 10)), torch.arange(10), l)
        snap = c.snapshot_counters()
        before = (c.get_seq_length(), list(c._rows), c.get_total_cached_tokens())
        c.advance(1)
        assert c.get_total_cached_tokens() == before[2] + 2 * 2
        c.restore_counters(snap)
        assert (c.get_seq_length(), list(c._rows), c.get_total_cached_tokens()) == before


def test_constructor_hints_refuse_knorm_alpha(host_cache):
    """The hints make update() reduce the prompt by the "alpha" score; compressing by key norms afterwards is refused
    instead of silently mixing the two."""
    c = host_cache(device="cpu", memory_size=4, buffer_size=2, num_layers=1)
    k = emu.on_device(torch.randn(1, 2, 10, 16))
    c.update(k, k.clone(), emu.on_device(torch.zeros(1, 2, 10)), torch.arange(10), 0)
    with pytest.raises(ValueError, match="knorm_alpha"):
        c.compress(strategy="knorm_alpha", memory_size=4, buffer_size=2)
    c.compress(strategy="alpha", memory_size=4, buffer_size=2)
    assert c.get_cache_length(0) == 4
