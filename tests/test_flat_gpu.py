"""Budget-sharing flat caches, the packed functional append and the sliding window on a B200, against the golden
vectors produced by the reference's own classes (and the oracle for the parts the goldens do not hold)."""
import os

import numpy as np
import pytest
import torch

from oracle import trimkv_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _g(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


@pytest.mark.parametrize("ci", range(7))
def test_flat_budget_classes_match_reference(golden_dir, ci):
    from trimkv_b200 import BatchedDynamicBudgetTrimKVCache, DynamicBudgetTrimKVCache
    g = _g(golden_dir, "flat_budget.npz")
    L, B, H, D, S, T, M, Bf = [int(x) for x in g["meta"]]
    D = 8  # rows must be multiples of 16 bytes on the CUDA path; the payload check below adapts
    kind, strategy, floor, thr = str(g["cases"][ci]).split("|")
    floor, thr = float(floor), float(thr)
    logb = torch.from_numpy(g[f"c{ci}_logb"]).to(DEV)
    bsz = logb.shape[1]
    cache = (BatchedDynamicBudgetTrimKVCache if kind == "batched" else DynamicBudgetTrimKVCache)(device=DEV)
    for t in range(T + 1):
        lo, hi = (0, S) if t == 0 else (S + t - 1, S + t)
        for l in range(L):
            k = (torch.arange(lo, hi, dtype=torch.float32, device=DEV)[None, None, :, None] + 1000 * l).expand(bsz, H, hi - lo, D)
            _, _, _, _, kw = cache.update(k.contiguous(), (-k).contiguous(), logb[l, :, :, lo:hi].contiguous(),
                                          torch.arange(lo, hi, device=DEV), l)
        cache.compress(strategy=strategy, memory_size=M, buffer_size=Bf, floor_budget_ratio=floor, alpha_threshold=thr,
                       num_layers=L, num_key_value_heads=H)
        got = torch.stack([cache.head_lens[l] for l in range(L)]).cpu().numpy()
        assert np.array_equal(got, g[f"c{ci}_lens"][t]), (ci, t)
        assert cache.get_total_cached_tokens() == int(g[f"c{ci}_lens"][t].sum())
        if t in (0, T // 2, T):
            for l in range(L):
                kp, vp, bp, pp = cache.packed(l)
                assert np.array_equal(pp[:, 0].cpu().numpy(), g[f"c{ci}_pos_t{t}_l{l}"]), (ci, t, l)
                assert torch.equal(kp[:, 0], pp[:, 0].float() + 1000.0 * l) and torch.equal(vp, -kp)
                cu = cache.cu_seqlens_k[l].cpu().numpy()
                assert np.array_equal(cu, np.concatenate([[0], np.cumsum(got[l])]))
    cache.check_status()
    assert cache.get_cache_length(0, *((0, 1) if kind == "batched" else (1,))) == int(g[f"c{ci}_lens"][T][0, 1])


def test_update_flatten_view_matches_reference_layout(golden_dir):
    """The functional packed append reproduces the reference's flat tensors (K rows, 1-column log beta / positions)."""
    from trimkv_b200 import update_flatten_view
    g = _g(golden_dir, "flat_layout.npz")
    S = int(g["S"])
    k, b = torch.from_numpy(g["k"]).to(DEV), torch.from_numpy(g["log_beta"]).to(DEV)
    Bt, H, _, D = k.shape
    nseq = Bt * H
    key = k[:, :, :S].reshape(-1, D).contiguous()
    rw = b[:, :, :S].reshape(-1, 1).contiguous()
    pos = torch.arange(S, device=DEV).expand(Bt, H, S).reshape(-1, 1).contiguous()
    hl = torch.full((nseq,), S, dtype=torch.int32, device=DEV)
    cu = torch.arange(0, nseq * S + 1, S, dtype=torch.int32, device=DEV)
    for lo, hi in ((S, S + 1), (S + 1, S + 2), (S + 2, S + 4)):
        s = hi - lo
        key = update_flatten_view(key, k[:, :, lo:hi].reshape(1, nseq, s, D).contiguous(), hl, cu)
        rw = update_flatten_view(rw, b[:, :, lo:hi].reshape(1, nseq, s, 1).contiguous(), hl, cu)
        pos = update_flatten_view(pos, torch.arange(lo, hi, device=DEV).expand(Bt, H, s).reshape(1, nseq, s, 1).contiguous(), hl, cu)
        hl = hl + s
        cu = cu + torch.arange(0, nseq * s + 1, s, dtype=torch.int32, device=DEV)
    assert np.array_equal(key.cpu().numpy(), g["key_flat"])
    assert np.array_equal(rw.cpu().numpy(), g["rw_flat"])
    assert np.array_equal(pos.cpu().numpy(), g["pos_flat"])
    with pytest.raises(AssertionError):
        update_flatten_view(key, k[:, :, :1].contiguous(), hl, cu)  # B must be 1, as in the reference


def test_sliding_window_matches_reference(golden_dir):
    from trimkv_b200 import TrimKVCache
    g = _g(golden_dir, "sliding_window.npz")
    M, B, S, T, W = (int(g[k]) for k in "MBSTW")
    logb = torch.from_numpy(g["log_beta"]).to(DEV)
    cache = TrimKVCache(device=DEV)
    cache.sliding_window_size = W
    ev = 0
    for t in range(T + 1):
        lo, hi = (0, S) if t == 0 else (S + t - 1, S + t)
        k = torch.zeros(logb.shape[0], logb.shape[1], hi - lo, 8, device=DEV)
        cache.update(k, k.clone(), logb[:, :, lo:hi].contiguous(), torch.arange(lo, hi, device=DEV), 0)
        before = cache.get_cache_length(0)
        cache.compress(memory_size=M, buffer_size=B)
        if cache.get_cache_length(0) != before:
            assert np.array_equal(cache.kv_positions[0].cpu().numpy(), g["kept_positions"][ev])
            ev += 1
    cache.check_status()
    assert ev == g["kept_positions"].shape[0]


def test_group_budget_large_group_vs_oracle():
    """One request, 28 layers x 8 heads sharing a budget: counts against the oracle's concatenated top-k."""
    from trimkv_b200 import ops
    gen = torch.Generator().manual_seed(3)
    L, H, cap = 28, 8, 300
    nseg = H
    lens = torch.randint(100, cap + 1, (L, nseg), generator=gen).to(torch.int32)
    beta = torch.nn.functional.logsigmoid(torch.randn(L, nseg, cap, generator=gen) * 1.5 + 3).bfloat16().float()
    pos = torch.sort(torch.rand(L, nseg, 2000, generator=gen).argsort(-1)[..., :cap], -1)[0].to(torch.int32)
    keep = torch.empty(L, nseg, dtype=torch.int32, device=DEV)
    k_total = L * H * 128
    ops.group_budget(beta.to(DEV).view(L, -1), pos.to(DEV).view(L, -1), lens.to(DEV), cap, 1, H, L, nseg, 2001, k_total, keep)
    sc = [orc.retention_scores(beta[l, h, :lens[l, h]].numpy(), pos[l, h, :lens[l, h]].numpy(), 2001)
          for l in range(L) for h in range(H)]
    want = orc._group_keep_counts(sc, k_total=k_total)
    assert keep.cpu().view(-1).tolist() == want
    assert sum(want) == k_total


def test_knorm_alpha_matches_reference(golden_dir):
    """strategy="knorm_alpha" on fp32 keys: kept positions equal the reference's at every eviction."""
    from trimkv_b200 import TrimKVCache
    g = _g(golden_dir, "knorm_alpha.npz")
    M, B, S, T = (int(g[k]) for k in "MBST")
    logb, keys = torch.from_numpy(g["log_beta"]).to(DEV), torch.from_numpy(g["keys"]).to(DEV)
    cache = TrimKVCache(device=DEV)
    ev = 0
    for t in range(T + 1):
        lo, hi = (0, S) if t == 0 else (S + t - 1, S + t)
        cache.update(keys[:, :, lo:hi].contiguous(), (keys[:, :, lo:hi] * 0.5).contiguous(), logb[:, :, lo:hi].contiguous(),
                     torch.arange(lo, hi, device=DEV), 0)
        before = cache.get_cache_length(0)
        cache.compress(strategy="knorm_alpha", memory_size=M, buffer_size=B)
        if cache.get_cache_length(0) != before:
            pos = cache.kv_positions[0]
            assert np.array_equal(pos.cpu().numpy(), g["kept_positions"][ev]), t
            assert torch.equal(cache.key_cache[0], torch.gather(keys, 2, pos.long().unsqueeze(-1).expand(-1, -1, -1, keys.shape[-1])))
            ev += 1
    cache.check_status()
    assert ev == g["kept_positions"].shape[0]


def test_decode_attention_over_a_budget_sharing_cache():
    """Decode attention through the registry entry over head lengths that differ widely (one head holds most of the
    shared budget): the cache hands its host-side token total to the kernel, which sizes its grid by it."""
    from trimkv_b200 import BatchedDynamicBudgetTrimKVCache
    from trimkv_b200.attn import TRIMKV_ATTENTION_IMPLEMENTATIONS
    attn = TRIMKV_ATTENTION_IMPLEMENTATIONS["db_attn_flash_batched"]
    gen = torch.Generator().manual_seed(5)
    L, B, H, G, D, S, M, Bf = 2, 2, 8, 2, 128, 3000, 512, 32
    dt = torch.bfloat16
    # retention close to 1 for head 0 (it keeps nearly everything), fast decay for the others
    mean = torch.tensor([9.0, 2.0, 1.0, 0.5, 0.0, 0.0, -0.5, -1.0]).view(1, H, 1)
    cache = BatchedDynamicBudgetTrimKVCache(device=DEV)
    for t in range(4):
        lo, hi = (0, S) if t == 0 else (S + t - 1, S + t)
        for l in range(L):
            k = torch.randn(B, H, hi - lo, D, generator=gen).to(dt).to(DEV)
            v = torch.randn(B, H, hi - lo, D, generator=gen).to(dt).to(DEV)
            logb = torch.nn.functional.logsigmoid(torch.randn(B, H, hi - lo, generator=gen) + mean).to(dt).to(DEV)
            kk, vv, _, _, kw = cache.update(k, v, logb, torch.arange(lo, hi, device=DEV), l)
            if t == 0:
                continue
            assert kw["total_len_bound"] == int(cache.head_lens[l].sum())
            q = torch.randn(B, H * G, 1, D, generator=gen).to(dt).to(DEV)
            out, _, _ = attn(None, q, kk, vv, None, flash_attn_kwargs=kw)
            kp, vp, _, _ = cache.packed(l)
            lens = cache.head_lens[l].cpu().numpy()
            want = orc.varlen_gqa_attention(q.float().cpu().numpy(), kp.float().cpu().numpy(), vp.float().cpu().numpy(),
                                            np.concatenate([[0], np.cumsum(lens)]), B, H)
            assert np.max(np.abs(out.float().cpu().numpy() - want)) <= 2e-2
        cache.compress(strategy="alpha", memory_size=M, buffer_size=Bf, num_layers=L, num_key_value_heads=H)
        if t == 0:
            lens = cache.head_lens[0].cpu().numpy()
            assert lens.max() > 4 * lens.min()          # the case is ragged
    cache.check_status()


@pytest.mark.parametrize("ci", range(5))
def test_flat_budget_bf16_scores(golden_dir, ci):
    """bf16 log beta: the flat classes score in bf16 like the reference.  Same rows as the CPU restatement, and
    against the reference's own result the same kept-score multisets (rows differ only inside tie classes)."""
    from test_oracle import _bf16_bits_to_f32, check_flat_bf16_case
    from trimkv_b200 import BatchedDynamicBudgetTrimKVCache, DynamicBudgetTrimKVCache
    g = _g(golden_dir, "flat_budget_bf16.npz")
    L, B, H, D, S, M, Bf = [int(x) for x in g["meta"]]
    D = 8
    kind, strategy, thr = str(g["cases"][ci]).split("|")
    bsz = B if kind == "batched" else 1
    logb = _bf16_bits_to_f32(g[f"c{ci}_logb_bits"])
    cache = (BatchedDynamicBudgetTrimKVCache if kind == "batched" else DynamicBudgetTrimKVCache)(device=DEV)
    want = orc.OracleFlatBudgetCache(kind == "batched", "bfloat16")
    for l in range(L):
        k = np.broadcast_to(np.arange(S, dtype=np.float32)[None, None, :, None], (bsz, H, S, D)) + 1000 * l
        want.update(k, -k, logb[l], np.arange(S), l)
        kt = torch.from_numpy(np.ascontiguousarray(k)).to(DEV)
        cache.update(kt, -kt, torch.from_numpy(logb[l]).to(torch.bfloat16).to(DEV), torch.arange(S, device=DEV), l)
    cache.compress(strategy=strategy, memory_size=M, buffer_size=Bf, alpha_threshold=float(thr), num_layers=L,
                   num_key_value_heads=H)
    want.compress(strategy=strategy, memory_size=M, buffer_size=Bf, alpha_threshold=float(thr))
    cache.check_status()
    lens = torch.stack([cache.head_lens[l] for l in range(L)]).cpu().numpy()
    assert np.array_equal(lens, np.stack([want.head_lens[l] for l in range(L)]))
    packed = [cache.packed(l) for l in range(L)]
    for l in range(L):
        assert np.array_equal(packed[l][3][:, 0].cpu().numpy(), want.kv_positions[l][:, 0])
        assert torch.equal(packed[l][0][:, 0], packed[l][3][:, 0].float() + 1000.0 * l)
    score_of = lambda l: orc.retention_scores(packed[l][2][:, 0].float().cpu().numpy(), packed[l][3][:, 0].cpu().numpy(),
                                              S + 1, "bfloat16")
    check_flat_bf16_case(g, ci, lens, lambda l: packed[l][3][:, 0].cpu().numpy().astype(np.int32), score_of)


@pytest.mark.parametrize("Q,resident_min_ctas", [(5, 96), (24, 96), (150, 96), (24, 1), (150, 1)])
def test_multi_token_query_over_ragged_cache(Q, resident_min_ctas, monkeypatch):
    """A second prompt (Q > 1) appended to a budget-sharing cache whose heads differ in length: bottom-right aligned
    causal attention per segment, against the per-segment restatement.  With the default routing (8 segments, too few
    CTAs for the query-resident kernel to be preferred) Q = 5 (10 query rows per segment) runs on the decode kernel,
    Q = 24 (48 rows) on the 32-rows-per-CTA kernel for the ragged cache and through the library's causal attention for
    the uniform one, Q = 150 (300 rows) on the query-resident kernel for the ragged cache (the library would need a
    materialised mask) and through the library for the uniform one; with the CTA threshold lowered to 1 the
    query-resident kernel serves both caches for Q = 24 and Q = 150."""
    from trimkv_b200 import BatchedDynamicBudgetTrimKVCache, TrimKVCache, attn as attn_mod
    from trimkv_b200.attn import TRIMKV_ATTENTION_IMPLEMENTATIONS
    monkeypatch.setattr(attn_mod, "RESIDENT_MIN_CTAS", resident_min_ctas)
    attn = TRIMKV_ATTENTION_IMPLEMENTATIONS["db_attn_flash_batched"]
    gen = torch.Generator().manual_seed(9)
    B, H, G, D, S, M, Bf = 2, 4, 2, 128, 400, 64, 8
    dt = torch.bfloat16
    mean = torch.tensor([8.0, 1.0, 0.0, -1.0]).view(1, H, 1)
    for cls in (BatchedDynamicBudgetTrimKVCache, TrimKVCache):
        cache = cls(device=DEV)
        k = torch.randn(B, H, S, D, generator=gen).to(dt).to(DEV)
        logb = torch.nn.functional.logsigmoid(torch.randn(B, H, S, generator=gen) + mean).to(dt).to(DEV)
        cache.update(k, -k, logb, torch.arange(S, device=DEV), 0)
        cache.compress(strategy="alpha", memory_size=M, buffer_size=Bf, num_layers=1, num_key_value_heads=H)
        k2 = torch.randn(B, H, Q, D, generator=gen).to(dt).to(DEV)
        kk, vv, _, _, kw = cache.update(k2, -k2, logb[:, :, :Q].contiguous(), torch.arange(S, S + Q, device=DEV), 0)
        q = torch.randn(B, H * G, Q, D, generator=gen).to(dt).to(DEV)
        out, _, _ = attn(None, q, kk, vv, None, flash_attn_kwargs=kw)
        lens = cache.head_lens[0].cpu().numpy()
        if cls is BatchedDynamicBudgetTrimKVCache:
            assert lens.max() > 2 * lens.min()
            kp, vp, _, _ = cache.packed(0)
        else:
            kp = torch.cat([kk[b, h, :lens[b * H + h]] for b in range(B) for h in range(H)])
            vp = torch.cat([vv[b, h, :lens[b * H + h]] for b in range(B) for h in range(H)])
        want = orc.varlen_gqa_attention(q.float().cpu().numpy(), kp.float().cpu().numpy(), vp.float().cpu().numpy(),
                                        np.concatenate([[0], np.cumsum(lens)]), B, H)
        assert out.shape == (B, Q, H * G, D)
        assert np.max(np.abs(out.float().cpu().numpy() - want)) <= 2e-2
        cache.check_status()


@pytest.mark.parametrize("ci", range(12))
def test_flat_budget_knorm_strategies(golden_dir, ci):
    """"knorm_alpha" / "knorm_alpha_threshold" (+ layer-wise) on both flat classes, fp32 and bf16 tensors, against the
    reference's result and the CPU restatement."""
    from test_oracle import check_knorm_case, load_knorm_case
    from trimkv_b200 import BatchedDynamicBudgetTrimKVCache, DynamicBudgetTrimKVCache
    g = _g(golden_dir, "flat_budget_knorm.npz")
    L, B, H, D, S, M, Bf = [int(x) for x in g["meta"]]
    kind, strategy, thr, dt, logb, keys = load_knorm_case(g, ci)
    tdt = getattr(torch, dt)
    cache = (BatchedDynamicBudgetTrimKVCache if kind == "batched" else DynamicBudgetTrimKVCache)(device=DEV)
    want = orc.OracleFlatBudgetCache(kind == "batched", dt, dt)
    for l in range(L):
        want.update(keys[l], keys[l] * 0.5, logb[l], np.arange(S), l)
        kt = torch.from_numpy(keys[l]).to(tdt).to(DEV)
        cache.update(kt, (kt.float() * 0.5).to(tdt), torch.from_numpy(logb[l]).to(tdt).to(DEV), torch.arange(S, device=DEV), l)
    cache.compress(strategy=strategy, memory_size=M, buffer_size=Bf, alpha_threshold=thr, num_layers=L, num_key_value_heads=H)
    want.compress(strategy=strategy, memory_size=M, buffer_size=Bf, alpha_threshold=thr)
    cache.check_status()
    lens = torch.stack([cache.head_lens[l] for l in range(L)]).cpu().numpy()
    packed = [cache.packed(l) for l in range(L)]
    assert np.array_equal(lens, np.stack([want.head_lens[l] for l in range(L)]))
    for l in range(L):
        assert np.array_equal(packed[l][3][:, 0].cpu().numpy(), want.kv_positions[l][:, 0])
        assert np.array_equal(packed[l][0].float().cpu().numpy(), want.key_cache[l])       # payload moved with its row

    def score_of(l):
        want._knorm = True
        return np.concatenate([want._scores(l, s) for s in range(lens.shape[1])])
    check_knorm_case(g, ci, lens, lambda l: packed[l][3][:, 0].cpu().numpy().astype(np.int32), score_of)
