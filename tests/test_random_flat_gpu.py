"""Seeded random walks of the budget-sharing flat caches (update -> compress every step, both classes, every strategy the
goldens hold, the key-norm forms included) against the oracle's restatement, at shapes the reference-generated fixtures do not cover: one to four
layers, one to five KV heads, budgets from 3 to 70, prompts below and far above the budget.  Needs a B200."""
import numpy as np
import pytest
import torch

from oracle import trimkv_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

COMBOS = [("batched", "alpha", False, False), ("batched", "layer_wise_alpha", False, False),
          ("batched", "layer_wise_alpha", True, False), ("batched", "alpha_threshold", False, True),
          ("single", "alpha", False, False), ("single", "alpha", True, False), ("single", "layer_wise_alpha", False, False),
          ("batched", "knorm_alpha", False, False), ("batched", "layer_wise_knorm_alpha", False, False),
          ("batched", "knorm_alpha_threshold", False, True), ("single", "knorm_alpha", False, False),
          ("single", "layer_wise_knorm_alpha", False, False)]


def _draw(seed):
    rng = np.random.default_rng(7000 + seed)
    kind, strategy, with_floor, with_thr = COMBOS[seed % len(COMBOS)]
    L, H = int(rng.integers(1, 5)), int(rng.integers(1, 6))
    bsz = int(rng.integers(1, 4)) if kind == "batched" else 1
    m = int(rng.choice([3, 8, 20, 33, 70]))
    buf = int(rng.choice([1, 2, 4, 9]))
    prompt = int(rng.choice([max(1, m // 2), m + buf, 2 * m + 1, 6 * m + 5]))
    steps = int(rng.integers(2 * buf + 2, 3 * buf + 12))
    floor = float(rng.choice([0.25, 0.5])) if with_floor else 0.0
    thr = float(rng.choice([0.2, 0.5])) if with_thr else 0.0
    return rng, kind, strategy, floor, thr, L, H, bsz, m, buf, prompt, steps


@pytest.mark.parametrize("seed", range(36))
def test_random_flat_budget_walk_matches_oracle(seed):
    from trimkv_b200 import BatchedDynamicBudgetTrimKVCache, DynamicBudgetTrimKVCache
    rng, kind, strategy, floor, thr, L, H, bsz, m, buf, prompt, steps = _draw(seed)
    d = 8
    torch.manual_seed(seed)
    logb = torch.nn.functional.logsigmoid(torch.randn(L, bsz, H, prompt + steps) * 1.5 + 3.0)
    if seed % 2:
        logb = (logb * 16).round() / 16     # coarse values: equal scores inside and across segments
    cache = (BatchedDynamicBudgetTrimKVCache if kind == "batched" else DynamicBudgetTrimKVCache)(device=DEV)
    ref = orc.OracleFlatBudgetCache(kind == "batched")
    tag = (seed, kind, strategy, floor, thr, L, H, bsz, m, buf, prompt)
    # keys of varied length (the knorm strategies add log ||k|| to the score); the values are their negatives
    keys = (torch.randn(L, bsz, H, prompt + steps, d) * (0.2 + 3 * torch.rand(L, bsz, H, prompt + steps, 1))).numpy()
    for t in range(steps + 1):
        lo, hi = (0, prompt) if t == 0 else (prompt + t - 1, prompt + t)
        for l in range(L):
            k = np.ascontiguousarray(keys[l, :, :, lo:hi])
            ref.update(k.copy(), -k.copy(), logb[l, :, :, lo:hi].numpy(), np.arange(lo, hi), l)
            kt = torch.from_numpy(k.copy()).to(DEV)
            cache.update(kt, -kt, logb[l, :, :, lo:hi].contiguous().to(DEV), torch.arange(lo, hi, device=DEV), l)
        ref.compress(strategy=strategy, memory_size=m, buffer_size=buf, floor_budget_ratio=floor, alpha_threshold=thr)
        cache.compress(strategy=strategy, memory_size=m, buffer_size=buf, floor_budget_ratio=floor, alpha_threshold=thr,
                       num_layers=L, num_key_value_heads=H)
        got = torch.stack([cache.head_lens[l] for l in range(L)]).cpu().numpy()
        want = np.stack([ref.head_lens[l] for l in range(L)])
        assert np.array_equal(got, want), (tag, t)
        if t in (0, steps // 2, steps):
            for l in range(L):
                kp, vp, bp, pp = cache.packed(l)
                assert np.array_equal(pp[:, 0].cpu().numpy(), ref.kv_positions[l][:, 0]), (tag, t, l)
                assert np.array_equal(kp.cpu().numpy(), ref.key_cache[l]) and torch.equal(vp, -kp)
                assert np.array_equal(bp[:, 0].float().cpu().numpy(), ref.retention_weights[l][:, 0])
                assert np.array_equal(cache.cu_seqlens_k[l].cpu().numpy(), np.concatenate([[0], np.cumsum(got[l])]))
    cache.check_status()
