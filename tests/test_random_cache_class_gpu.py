"""Seeded random walks of the `TrimKVCache` class itself (update -> compress after every token, one to three layers, with
and without a sliding window, strategies "alpha" and "knorm_alpha", constructor hints on and off) against the oracle's
restatement of the reference class: lengths after every step, kept positions and payload after every eviction.  fp32
keys, so that the knorm scores are exact.  Needs a B200."""
import numpy as np
import pytest
import torch

from oracle import trimkv_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _draw(seed):
    rng = np.random.default_rng(9000 + seed)
    layers, bsz, hkv = int(rng.integers(1, 4)), int(rng.integers(1, 4)), int(rng.choice([1, 2, 3, 8]))
    m = int(rng.choice([4, 9, 32, 65, 130]))
    buf = int(rng.choice([1, 3, 8, 20]))
    window = int(rng.choice([0, 0, 1, 3, m - 1]))
    strategy = str(rng.choice(["alpha", "knorm_alpha"]))
    prompt = int(rng.choice([1, m, m + buf, 3 * m + 7, 700]))
    hints = bool(rng.integers(0, 2)) and strategy == "alpha"   # the hints reduce the prompt by the "alpha" score inside update()
    return rng, layers, bsz, hkv, m, buf, window, strategy, prompt, hints


@pytest.mark.parametrize("seed", range(24))
def test_random_cache_class_walk_matches_oracle(seed):
    from trimkv_b200 import TrimKVCache
    rng, layers, bsz, hkv, m, buf, window, strategy, prompt, hints = _draw(seed)
    d, steps = 8, 2 * buf + 4
    tag = (seed, layers, bsz, hkv, m, buf, window, strategy, prompt, hints)
    gen = torch.Generator().manual_seed(seed)
    total = prompt + steps
    keys = torch.randn(layers, bsz, hkv, total, d, generator=gen) * torch.rand(layers, bsz, hkv, total, 1, generator=gen) * 3
    logb = torch.nn.functional.logsigmoid(torch.randn(layers, bsz, hkv, total, generator=gen) * 1.5 + 3.0)
    if seed % 2:
        logb = (logb * 16).round() / 16              # coarse: equal scores occur
    cache = TrimKVCache(device=DEV, **(dict(memory_size=m, buffer_size=buf, num_layers=layers) if hints else {}))
    ref = orc.OracleTrimKVCache()
    cache.sliding_window_size = ref.sliding_window_size = window
    for t in range(steps + 1):
        lo, hi = (0, prompt) if t == 0 else (prompt + t - 1, prompt + t)
        for l in range(layers):
            k = keys[l, :, :, lo:hi].contiguous()
            ref.update(k.numpy(), (k * 0.5).numpy(), logb[l, :, :, lo:hi].numpy(), np.arange(lo, hi), l)
            cache.update(k.to(DEV), (k * 0.5).to(DEV), logb[l, :, :, lo:hi].contiguous().to(DEV),
                         torch.arange(lo, hi, device=DEV), l)
        ref.compress(strategy=strategy, memory_size=m, buffer_size=buf)
        cache.compress(strategy=strategy, memory_size=m, buffer_size=buf, num_layers=layers, num_key_value_heads=hkv)
        for l in range(layers):
            n = ref.get_cache_length(l)
            assert cache.get_cache_length(l) == n, (tag, t, l)
            if t in (0, steps // 2, steps) or n == m:
                pos = cache.kv_positions[l][:, :, :n]
                assert np.array_equal(pos.cpu().numpy(), ref.kv_positions[l]), (tag, t, l)
                assert np.array_equal(cache.key_cache[l][:, :, :n].cpu().numpy(), ref.key_cache[l]), (tag, t, l)
                assert np.array_equal(cache.value_cache[l][:, :, :n].cpu().numpy(), ref.value_cache[l]), (tag, t, l)
                assert np.array_equal(cache.retention_weights[l][:, :, :n].cpu().numpy(), ref.retention_weights[l]), (tag, t, l)
        assert cache.get_seq_length() == ref.get_seq_length()
    cache.check_status()
