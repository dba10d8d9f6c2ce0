"""The oracle against the golden vectors produced by the reference's own Python (CPU)."""
import os

import numpy as np
import pytest

from oracle import trimkv_oracle as orc


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


def test_config1_lockstep_positions_and_lengths(golden_dir):
    g = _load(golden_dir, "config1_lockstep.npz")
    M, B, S, T = int(g["M"]), int(g["B"]), int(g["S"]), int(g["T"])
    logb = g["log_beta"][None]  # [1,H,S+T]
    H = logb.shape[1]
    cache = orc.OracleTrimKVCache()
    lens, kept = [], []
    for t in range(T + 1):
        lo, hi = (0, S) if t == 0 else (S + t - 1, S + t)
        k = np.broadcast_to(np.arange(lo, hi, dtype=np.float32)[None, None, :, None], (1, H, hi - lo, 4)).copy()
        cache.update(k, k.copy(), logb[:, :, lo:hi], np.arange(lo, hi), 0)
        before = cache.get_cache_length(0)
        cache.compress(memory_size=M, buffer_size=B)
        lens.append(cache.get_cache_length(0))
        if lens[-1] != before:
            kept.append(cache.kv_positions[0][0].astype(np.int32))
            # moved rows carry their payload: K row value == its position
            assert np.array_equal(cache.key_cache[0][0, :, :, 0], cache.kv_positions[0][0].astype(np.float32))
    assert np.array_equal(np.asarray(lens, np.int32), g["lens"])
    assert np.array_equal(np.stack(kept), g["kept_positions"])


def test_ties_bf16_kept_score_multiset(golden_dir):
    g = _load(golden_dir, "ties_bf16.npz")
    M, B, S, T = int(g["M"]), int(g["B"]), int(g["S"]), int(g["T"])
    bits = g["log_beta_bits"].astype(np.uint16).astype(np.uint32) << 16
    logb = bits.view(np.float32)  # bf16 -> fp32, exact
    Bt, H, _ = logb.shape
    cache = orc.OracleTrimKVCache()
    ev = 0
    for t in range(T + 1):
        lo, hi = (0, S) if t == 0 else (S + t - 1, S + t)
        k = np.zeros((Bt, H, hi - lo, 2), np.float32)
        cache.update(k, k, logb[:, :, lo:hi], np.arange(lo, hi), 0)
        before = cache.get_cache_length(0)
        q_idx = cache.get_seq_length(0) + 1
        cache.compress(memory_size=M, buffer_size=B)
        if cache.get_cache_length(0) != before:
            assert t == int(g["evict_steps"][ev])
            sc = orc.retention_scores(cache.retention_weights[0], cache.kv_positions[0], q_idx)
            got = np.sort(sc.reshape(Bt * H, M), axis=-1)
            # The kept-score multiset is independent of how boundary ties are broken.
            assert np.array_equal(got, g["kept_scores_sorted"][ev])
            # No boundary tie occurs in this run, so the canonical rule and the reference agree.
            assert np.array_equal(cache.kv_positions[0].reshape(Bt * H, M), g["kept_positions_reference"][ev])
            ev += 1
    assert ev == len(g["evict_steps"])


def test_ties_single_shot_boundary_classes(golden_dir):
    g = _load(golden_dir, "ties_single_shot.npz")
    M = int(g["M"])
    logb = g["log_beta"]
    R, n = logb.shape
    pos = np.broadcast_to(np.arange(n), (R, n))
    sc = orc.retention_scores(logb, pos, n + 1)
    keep = orc.canonical_topm(sc, M)
    kept_sc = np.take_along_axis(sc, keep, -1)
    # Same multiset of kept scores as the reference's topk, whatever its tie order.
    assert np.array_equal(np.sort(kept_sc, -1), g["kept_scores_sorted"])
    differing = 0
    for r in range(R):
        ref = g["kept_positions_reference"][r]
        thr = kept_sc[r].min()
        only_mine, only_ref = np.setdiff1d(keep[r], ref), np.setdiff1d(ref, keep[r])
        differing += only_mine.size
        # Differences are confined to the class of scores equal to the threshold ...
        assert np.all(sc[r, only_mine] == thr) and np.all(sc[r, only_ref] == thr)
        # ... and inside that class the canonical rule keeps the lowest positions.
        tie_idx = np.nonzero(sc[r] == thr)[0]
        kept_ties = np.intersect1d(tie_idx, keep[r])
        assert np.array_equal(kept_ties, tie_idx[:kept_ties.size])
    assert differing > 0  # the fixture does exercise the tie rule


def test_flat_layout(golden_dir):
    g = _load(golden_dir, "flat_layout.npz")
    S = int(g["S"])
    k, b = g["k"], g["log_beta"]
    cache = orc.OracleBatchedFlatCache()
    cache.update(k[:, :, :S], k[:, :, :S] * 2, b[:, :, :S], np.arange(S), 0)
    for lo, hi in ((S, S + 1), (S + 1, S + 2), (S + 2, S + 4)):
        _, _, _, _, kw = cache.update(k[:, :, lo:hi], k[:, :, lo:hi] * 2, b[:, :, lo:hi], np.arange(lo, hi), 0)
    assert np.array_equal(cache.key_cache[0], g["key_flat"])
    assert np.array_equal(cache.value_cache[0], g["value_flat"])
    assert np.array_equal(cache.retention_weights[0], g["rw_flat"])
    assert np.array_equal(cache.kv_positions[0], g["pos_flat"])
    assert np.array_equal(kw["head_lens"], g["head_lens"])
    assert np.array_equal(kw["cu_seqlens_k"], g["cu_seqlens_k"])


@pytest.mark.parametrize("ql", [1, 3])
def test_attention_vs_reference_eager(golden_dir, ql):
    g = _load(golden_dir, "eager_attention.npz")
    o = orc.dense_gqa_attention(g[f"q{ql}"], g[f"k{ql}"], g[f"v{ql}"])
    assert np.allclose(o, g[f"o{ql}"], atol=2e-5, rtol=1e-5)


def test_canonical_topm_tie_rule():
    s = np.array([[-1.0, -2.0, -1.0, -0.0, 0.0, -2.0, np.nan, -1.0]], np.float32)
    assert orc.canonical_topm(s, 1).tolist() == [[6]]          # NaN is the largest
    assert orc.canonical_topm(s, 2).tolist() == [[3, 6]]       # -0.0 == +0.0, lower index first
    assert orc.canonical_topm(s, 3).tolist() == [[3, 4, 6]]
    assert orc.canonical_topm(s, 5).tolist() == [[0, 2, 3, 4, 6]]
    assert orc.canonical_topm(s, 7).tolist() == [[0, 1, 2, 3, 4, 6, 7]]
    assert orc.canonical_topm(s, 8).tolist() == [list(range(8))]


def test_score_is_single_fp32_multiply():
    lb = np.array([-0.3, -1e-3, -7.25], np.float32)
    pos = np.array([0, 16777217, 5], np.int64)
    got = orc.retention_scores(lb, pos, 16777300)
    want = lb * (16777300 - pos).astype(np.float32)
    assert got.dtype == np.float32 and np.array_equal(got, want)


def _replay_flat_budget(g, ci, make_cache, step_hook=None):
    L, B, H, D, S, T, M, Bf = [int(x) for x in g["meta"]]
    kind, strategy, floor, thr = str(g["cases"][ci]).split("|")
    floor, thr = float(floor), float(thr)
    logb = g[f"c{ci}_logb"]
    bsz = logb.shape[1]
    cache = make_cache(kind == "batched")
    for t in range(T + 1):
        lo, hi = (0, S) if t == 0 else (S + t - 1, S + t)
        for l in range(L):
            k = np.broadcast_to(np.arange(lo, hi, dtype=np.float32)[None, None, :, None], (bsz, H, hi - lo, D)) + 1000 * l
            cache.update(k.copy(), -k.copy(), logb[l, :, :, lo:hi], np.arange(lo, hi), l)
        cache.compress(strategy=strategy, memory_size=M, buffer_size=Bf, floor_budget_ratio=floor, alpha_threshold=thr)
        yield t, cache, (L, B, H, D, S, T, M, Bf)


@pytest.mark.parametrize("ci", range(7))
def test_flat_budget_compress_matches_reference(golden_dir, ci):
    """Head lengths after every step and kept positions at three steps, for every strategy of both flat classes."""
    g = _load(golden_dir, "flat_budget.npz")
    for t, cache, (L, B, H, D, S, T, M, Bf) in _replay_flat_budget(g, ci, lambda batched: orc.OracleFlatBudgetCache(batched)):
        got = np.stack([cache.head_lens[l] for l in range(L)])
        assert np.array_equal(got, g[f"c{ci}_lens"][t]), (ci, t)
        if t in (0, T // 2, T):
            for l in range(L):
                assert np.array_equal(cache.kv_positions[l][:, 0].astype(np.int32), g[f"c{ci}_pos_t{t}_l{l}"]), (ci, t, l)
                # payload moves with its row: K row value == position + 1000*layer
                assert np.array_equal(cache.key_cache[l][:, 0], cache.kv_positions[l][:, 0] + 1000.0 * l)


def test_sliding_window_protects_newest_rows(golden_dir):
    g = _load(golden_dir, "sliding_window.npz")
    M, B, S, T, W = (int(g[k]) for k in "MBSTW")
    logb = g["log_beta"]
    cache = orc.OracleTrimKVCache()
    cache.sliding_window_size = W
    ev = 0
    for t in range(T + 1):
        lo, hi = (0, S) if t == 0 else (S + t - 1, S + t)
        k = np.zeros(logb.shape[:2] + (hi - lo, 2), np.float32)
        cache.update(k, k, logb[:, :, lo:hi], np.arange(lo, hi), 0)
        before = cache.get_cache_length(0)
        cache.compress(memory_size=M, buffer_size=B)
        if cache.get_cache_length(0) != before:
            assert np.array_equal(cache.kv_positions[0].astype(np.int32), g["kept_positions"][ev])
            ev += 1
    assert ev == g["kept_positions"].shape[0] and ev >= 2


def test_knorm_alpha_strategy(golden_dir):
    g = _load(golden_dir, "knorm_alpha.npz")
    M, B, S, T = (int(g[k]) for k in "MBST")
    logb, keys = g["log_beta"], g["keys"]
    cache = orc.OracleTrimKVCache()
    ev = 0
    for t in range(T + 1):
        lo, hi = (0, S) if t == 0 else (S + t - 1, S + t)
        cache.update(keys[:, :, lo:hi], keys[:, :, lo:hi] * 0.5, logb[:, :, lo:hi], np.arange(lo, hi), 0)
        before = cache.get_cache_length(0)
        cache.compress(strategy="knorm_alpha", memory_size=M, buffer_size=B)
        if cache.get_cache_length(0) != before:
            assert np.array_equal(cache.kv_positions[0].astype(np.int32), g["kept_positions"][ev])
            ev += 1
    assert ev == g["kept_positions"].shape[0] and ev >= 2


def _bf16_bits_to_f32(bits):
    return (bits.astype(np.uint16).astype(np.uint32) << 16).view(np.float32)


def flat_bf16_groups(kind, strategy, L, bsz, H):
    """Groups of (layer, segment) pairs that share one budget, in the concatenated order the reference uses."""
    if "layer_wise" in strategy:
        return [[(l, b * H + h) for h in range(H)] for l in range(L) for b in range(bsz)]
    return [[(l, b * H + h) for l in range(L) for h in range(H)] for b in range(bsz)]


def check_flat_bf16_case(g, ci, lens, pos_of, score_of):
    """Shared by the oracle test (CPU) and the CUDA test: compares a compressed cache with what the reference kept.
    ``lens [L, nseg]``; ``pos_of(l)`` kept positions of layer l in packed order; ``score_of(l)`` their bf16 scores."""
    L, B, H, D, S, M, Bf = [int(x) for x in g["meta"]]
    kind, strategy, thr = str(g["cases"][ci]).split("|")
    bsz = B if kind == "batched" else 1
    ref_lens = g[f"c{ci}_lens"]
    cu_ref = [np.concatenate([[0], np.cumsum(ref_lens[l])]) for l in range(L)]
    cu_got = [np.concatenate([[0], np.cumsum(lens[l])]) for l in range(L)]
    exact = 0
    for grp in flat_bf16_groups(kind, strategy, L, bsz, H):
        ref_sc = np.concatenate([g[f"c{ci}_scores_l{l}"][cu_ref[l][s]:cu_ref[l][s + 1]] for l, s in grp])
        got_sc = np.concatenate([score_of(l)[cu_got[l][s]:cu_got[l][s + 1]] for l, s in grp])
        # Whatever the tie order of torch.topk: the same multiset of kept scores.
        assert np.array_equal(np.sort(ref_sc), np.sort(got_sc)), (ci, grp[0])
        ref_pos = [g[f"c{ci}_pos_l{l}"][cu_ref[l][s]:cu_ref[l][s + 1]] for l, s in grp]
        got_pos = [pos_of(l)[cu_got[l][s]:cu_got[l][s + 1]] for l, s in grp]
        thr_sc = ref_sc.min()
        same = all(np.array_equal(a, b) for a, b in zip(ref_pos, got_pos))
        exact += same
        if not same:
            # Differences are confined to rows whose score equals the group's threshold score.
            for (l, s), a, b in zip(grp, ref_pos, got_pos):
                full = orc.retention_scores(_bf16_bits_to_f32(g[f"c{ci}_logb_bits"])[l].reshape(-1, S)[s], np.arange(S), S + 1, "bfloat16")
                for p in np.setxor1d(a, b):
                    assert full[p] == thr_sc, (ci, l, s, p)
    return exact


@pytest.mark.parametrize("ci", range(5))
def test_flat_budget_bf16_scores_match_reference(golden_dir, ci):
    """The flat classes score in the dtype of their tensors; on bf16 inputs the restatement keeps the same multiset
    of scores as the reference, the same rows wherever no tie straddles a budget, and for the threshold strategy
    (no top-k, hence no tie order) exactly the same rows."""
    g = _load(golden_dir, "flat_budget_bf16.npz")
    L, B, H, D, S, M, Bf = [int(x) for x in g["meta"]]
    kind, strategy, thr = str(g["cases"][ci]).split("|")
    bsz = B if kind == "batched" else 1
    logb = _bf16_bits_to_f32(g[f"c{ci}_logb_bits"])
    cache = orc.OracleFlatBudgetCache(kind == "batched", "bfloat16")
    for l in range(L):
        k = np.broadcast_to(np.arange(S, dtype=np.float32)[None, None, :, None], (bsz, H, S, D)) + 1000 * l
        cache.update(k, -k, logb[l], np.arange(S), l)
    cache.compress(strategy=strategy, memory_size=M, buffer_size=Bf, alpha_threshold=float(thr))
    lens = np.stack([cache.head_lens[l] for l in range(L)])
    score_of = lambda l: orc.retention_scores(cache.retention_weights[l][:, 0], cache.kv_positions[l][:, 0], S + 1, "bfloat16")
    exact = check_flat_bf16_case(g, ci, lens, lambda l: cache.kv_positions[l][:, 0].astype(np.int32), score_of)
    if "threshold" in strategy:
        assert np.array_equal(lens, g[f"c{ci}_lens"])
        assert exact == len(flat_bf16_groups(kind, strategy, L, bsz, H))


def test_flat_budget_bf16_fixture_tells_score_dtypes_apart(golden_dir):
    """Scoring the same inputs in fp32 keeps other rows in at least one case: the fixture pins the dtype."""
    g = _load(golden_dir, "flat_budget_bf16.npz")
    L, B, H, D, S, M, Bf = [int(x) for x in g["meta"]]
    differing = 0
    for ci in range(len(g["cases"])):
        kind, strategy, thr = str(g["cases"][ci]).split("|")
        bsz = B if kind == "batched" else 1
        logb = _bf16_bits_to_f32(g[f"c{ci}_logb_bits"])
        caches = [orc.OracleFlatBudgetCache(kind == "batched", dt) for dt in ("bfloat16", "float32")]
        for c in caches:
            for l in range(L):
                k = np.broadcast_to(np.arange(S, dtype=np.float32)[None, None, :, None], (bsz, H, S, D)) + 1000 * l
                c.update(k, -k, logb[l], np.arange(S), l)
            c.compress(strategy=strategy, memory_size=M, buffer_size=Bf, alpha_threshold=float(thr))
        differing += any(not np.array_equal(caches[0].kv_positions[l], caches[1].kv_positions[l]) for l in range(L))
    assert differing >= 1


def load_knorm_case(g, ci):
    """Inputs of one case of flat_budget_knorm.npz as fp32 arrays holding the values of the case's dtype."""
    kind, strategy, thr, dt = str(g["cases"][ci]).split("|")
    logb, keys = g[f"c{ci}_logb"], g[f"c{ci}_keys"]
    if dt == "bfloat16":
        logb, keys = _bf16_bits_to_f32(logb), _bf16_bits_to_f32(keys)
    return kind, strategy, float(thr), dt, logb.astype(np.float32), keys.astype(np.float32)


def check_knorm_case(g, ci, lens, pos_of, score_of):
    """fp32 cases and threshold cases: exactly the reference's rows.  bf16 top-k cases: the same multiset of kept
    scores per budget group (equal scores are frequent in bf16 and torch.topk's tie order is unspecified)."""
    L, B, H, D, S, M, Bf = [int(x) for x in g["meta"]]
    kind, strategy, thr, dt = str(g["cases"][ci]).split("|")
    bsz = B if kind == "batched" else 1
    ref_lens = g[f"c{ci}_lens"]
    if dt == "float32" or "threshold" in strategy:
        assert np.array_equal(lens, ref_lens), ci
        for l in range(L):
            assert np.array_equal(pos_of(l), g[f"c{ci}_pos_l{l}"]), (ci, l)
        return
    cu_ref = [np.concatenate([[0], np.cumsum(ref_lens[l])]) for l in range(L)]
    cu_got = [np.concatenate([[0], np.cumsum(lens[l])]) for l in range(L)]
    for grp in flat_bf16_groups(kind, strategy, L, bsz, H):
        ref_sc = np.concatenate([g[f"c{ci}_scores_l{l}"][cu_ref[l][s]:cu_ref[l][s + 1]] for l, s in grp])
        got_sc = np.concatenate([score_of(l)[cu_got[l][s]:cu_got[l][s + 1]] for l, s in grp])
        assert np.array_equal(np.sort(ref_sc), np.sort(got_sc)), (ci, grp[0])


@pytest.mark.parametrize("ci", range(12))
def test_flat_budget_knorm_strategies_match_reference(golden_dir, ci):
    g = _load(golden_dir, "flat_budget_knorm.npz")
    L, B, H, D, S, M, Bf = [int(x) for x in g["meta"]]
    kind, strategy, thr, dt, logb, keys = load_knorm_case(g, ci)
    cache = orc.OracleFlatBudgetCache(kind == "batched", dt, dt)
    for l in range(L):
        cache.update(keys[l], keys[l] * 0.5, logb[l], np.arange(S), l)
    cache.compress(strategy=strategy, memory_size=M, buffer_size=Bf, alpha_threshold=thr)
    lens = np.stack([cache.head_lens[l] for l in range(L)])

    def score_of(l):   # scores of the kept rows, the way the cache computed them (q_idx = S + 1)
        cache._knorm = True
        return np.concatenate([cache._scores(l, s) for s in range(lens.shape[1])])
    check_knorm_case(g, ci, lens, lambda l: cache.kv_positions[l][:, 0].astype(np.int32), score_of)
