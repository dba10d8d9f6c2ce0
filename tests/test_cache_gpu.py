"""`TrimKVCache` on a B200 in lock-step with the reference-generated golden vectors and the oracle."""
import os

import numpy as np
import pytest
import torch

from oracle import trimkv_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("eager_handoff", [False, True])
def test_config1_lockstep(golden_dir, eager_handoff):
    """benchmark-spec configs[0]: batch 1, 8 KV heads, D 128, fp32, M 512, B 128, 4096-token prefill + 256 steps.
    Kept positions at every eviction and the length after every step equal the reference's own run; K/V rows and
    log beta follow their positions."""
    from trimkv_b200 import TrimKVCache
    g = np.load(os.path.join(golden_dir, "config1_lockstep.npz"))
    M, B, S, T = int(g["M"]), int(g["B"]), int(g["S"]), int(g["T"])
    logb = torch.from_numpy(g["log_beta"])[None].to(DEV)
    H, D = logb.shape[1], 128
    hints = dict(memory_size=M, buffer_size=B, num_layers=1) if eager_handoff else {}
    cache = TrimKVCache(device=DEV, **hints)
    cache.record_kept = True
    lens, ev = [], 0
    gen = torch.Generator(device=DEV).manual_seed(0)
    payload = torch.randn(S + T, D, generator=gen, device=DEV)  # row t of every head carries payload[t]
    for t in range(T + 1):
        lo, hi = (0, S) if t == 0 else (S + t - 1, S + t)
        k = payload[lo:hi][None, None].expand(1, H, hi - lo, D).contiguous()
        kk, vv, bb, pp, kw = cache.update(k, (k * 2).contiguous(), logb[:, :, lo:hi].contiguous(),
                                          torch.arange(lo, hi, device=DEV), 0)
        assert kk.shape[-2] == hi - lo if t == 0 else kk.shape[-2] == lens[-1] + 1
        before = cache.get_cache_length(0)
        cache.compress(memory_size=M, buffer_size=B)
        lens.append(cache.get_cache_length(0))
        fired = (t == 0 and eager_handoff and S >= M + B) or lens[-1] != before
        if fired:
            pos = cache.kv_positions[0][0]
            assert np.array_equal(pos.cpu().numpy(), g["kept_positions"][ev]), t
            assert torch.equal(cache.key_cache[0][0], payload[pos.long()])
            assert torch.equal(cache.value_cache[0][0], payload[pos.long()] * 2)
            assert torch.equal(cache.retention_weights[0][0], logb[0].gather(-1, pos.long()))
            assert cache.head_lens[0].cpu().tolist() == [M] * H
            assert cache.cu_seqlens_k[0].cpu().tolist() == list(range(0, H * M + 1, M))
            ev += 1
    assert np.array_equal(np.asarray(lens, np.int32), g["lens"])
    assert ev == g["kept_positions"].shape[0]
    assert cache.get_seq_length() == S + T and cache.get_seq_length(0) == S + T
    assert cache.get_total_cached_tokens() == lens[-1] * H
    cache.check_status()


def test_bookkeeping_and_batch_ops():
    from trimkv_b200 import TrimKVCache
    torch.manual_seed(0)
    Bt, H, D, S = 4, 2, 128, 40
    cache = TrimKVCache(device=DEV)
    for l in range(2):
        k = torch.randn(Bt, H, S, D, device=DEV, dtype=torch.bfloat16)
        b = torch.nn.functional.logsigmoid(torch.randn(Bt, H, S, device=DEV)).bfloat16()
        cache.update(k, k + 1, b, torch.arange(S, device=DEV), l)
    cache.compress(memory_size=16, buffer_size=8)
    for l in range(2):
        k = torch.randn(Bt, H, 1, D, device=DEV, dtype=torch.bfloat16)
        cache.update(k, k + 1, torch.zeros(Bt, H, 1, device=DEV, dtype=torch.bfloat16), torch.arange(S, S + 1, device=DEV), l)
    assert len(cache) == 2 and cache.get_cache_length(1) == 17 and cache.get_cache_length(5) == 0
    assert cache.get_seq_length() == S + 1
    k0, v0, b0, p0 = cache[1]
    assert k0.shape == (Bt, H, 17, D) and p0.shape == (Bt, H, 17) and len(list(iter(cache))) == 2
    with pytest.raises(KeyError):
        cache[2]
    log = cache.log()
    assert log[0]["seen_tokens"] == S + 1 and log[0]["kv_positions"].dtype == torch.int64
    assert torch.equal(cache.log(1)["kv_positions"], p0.cpu().long())
    parts = cache.batch_split(Bt, 2)
    assert len(parts) == 2 and torch.equal(parts[1].key_cache[0], cache.key_cache[0][2:4])
    # a split cache keeps working: append one more token and evict
    kk = torch.randn(2, H, 1, D, device=DEV, dtype=torch.bfloat16)
    parts[1].update(kk, kk, torch.zeros(2, H, 1, device=DEV, dtype=torch.bfloat16), torch.arange(S + 1, S + 2, device=DEV), 0)
    assert parts[1].get_cache_length(0) == 18
    moved = cache.copy_to_device(DEV)
    assert torch.equal(moved.value_cache[1], cache.value_cache[1]) and moved.n_seen_tokens == cache.n_seen_tokens
    cache.batch_select_indices(torch.tensor([3, 0], device=DEV))
    assert cache.key_cache[0].shape[0] == 2 and torch.equal(cache.key_cache[1][0], k0[3])
    with pytest.raises(ValueError):
        cache.compress(strategy="nope")
    with pytest.raises(NotImplementedError):
        TrimKVCache(_distributed_cache_data=[1])
