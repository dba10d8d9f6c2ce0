"""Seeded random walks through the whole cache path (append -> attention -> triggered eviction, through the C ABI) against the
numpy oracle: shapes the hand-picked cases do not hold (odd budgets and buffers, one KV head, eight query heads per KV
head, head_dim 64, f16, prompts shorter and much longer than the budget).  Needs a B200."""
import numpy as np
import pytest
import torch

from oracle import trimkv_oracle as orc

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _draw(seed):
    rng = np.random.default_rng(1000 + seed)
    d = int(rng.choice([64, 128, 128]))
    dtype = [torch.bfloat16, torch.float16][int(rng.integers(0, 2))]
    bsz, hkv, group = int(rng.integers(1, 5)), int(rng.choice([1, 2, 3, 8])), int(rng.choice([1, 2, 4, 8]))
    m = int(rng.choice([1, 2, 7, 33, 64, 100, 257, 300, 515]))
    buf = int(rng.choice([1, 2, 5, 16, 40]))
    prompt = int(rng.choice([1, max(1, m // 2), m, m + buf - 1, m + buf, 2 * m + 3, 5 * m + 11]))
    return rng, d, dtype, bsz, hkv, group, m, buf, prompt


@pytest.mark.parametrize("seed", range(24))
def test_random_walk_matches_oracle(seed):
    from trimkv_b200 import ops
    rng, d, dtype, bsz, hkv, group, m, buf, prompt = _draw(seed)
    gen = torch.Generator().manual_seed(seed)
    nseg, hq = bsz * hkv, hkv * group
    steps = 2 * buf + 3
    cap = max(prompt, m + buf) + 1
    k = torch.zeros(nseg * cap, d, dtype=dtype, device=DEV)
    v = torch.zeros_like(k)
    beta = torch.zeros(nseg * cap, dtype=torch.float32, device=DEV)
    pos = torch.zeros(nseg * cap, dtype=torch.int32, device=DEV)
    ln = torch.zeros(nseg, dtype=torch.int32, device=DEV)
    cu = torch.zeros(nseg + 1, dtype=torch.int32, device=DEV)
    status = ops.new_status(DEV)
    ws = torch.empty(ops.decode_attn_workspace_bytes(bsz, hq, hkv, d, cap), dtype=torch.uint8, device=DEV)
    # the oracle's state: one list of rows per segment
    rk = [np.zeros((0, d), np.float32) for _ in range(nseg)]
    rv = [np.zeros((0, d), np.float32) for _ in range(nseg)]
    rb = [np.zeros((0,), np.float32) for _ in range(nseg)]
    rp = [np.zeros((0,), np.int64) for _ in range(nseg)]
    tol = 2e-2 if dtype == torch.bfloat16 else 5e-3
    seen = 0

    def feed(s):
        nonlocal seen
        kn = torch.randn(bsz, s, hkv, d, generator=gen).to(dtype).to(DEV).transpose(1, 2)
        vn = torch.randn(bsz, s, hkv, d, generator=gen).to(dtype).to(DEV).transpose(1, 2)
        # log beta rounded to the model dtype, coarse enough that equal scores occur
        bn = (torch.nn.functional.logsigmoid(torch.randn(bsz, s, hkv, generator=gen) * 1.5 + 3.0) * 8).round() / 8
        bn = bn.to(dtype).to(DEV).transpose(1, 2)
        ops.append(k, v, beta, pos, ln, cu, kn, vn, bn, torch.arange(seen, seen + s, device=DEV), cap, status)
        for sg in range(nseg):
            b_, h_ = divmod(sg, hkv)
            rk[sg] = np.concatenate([rk[sg], kn[b_, h_].float().cpu().numpy()])
            rv[sg] = np.concatenate([rv[sg], vn[b_, h_].float().cpu().numpy()])
            rb[sg] = np.concatenate([rb[sg], bn[b_, h_].float().cpu().numpy()])
            rp[sg] = np.concatenate([rp[sg], np.arange(seen, seen + s)])
        seen += s

    def evict():
        q_idx = seen + 1                     # src/trimkv/cache_utils.py:173
        ops.evict(k, v, beta, pos, ln, cu, nseg, nseg, cap, q_idx, m, m + buf, cap, None, status)
        for sg in range(nseg):
            n = len(rb[sg])
            if n >= m + buf and n > m:
                keep = orc.canonical_topm(orc.retention_scores(rb[sg], rp[sg], q_idx)[None], m)[0]
                rk[sg], rv[sg], rb[sg], rp[sg] = rk[sg][keep], rv[sg][keep], rb[sg][keep], rp[sg][keep]

    def check_state():
        assert ops.read_status(status) == 0
        lens = [len(x) for x in rb]
        assert ln.cpu().tolist() == lens
        assert cu.cpu().tolist() == np.concatenate([[0], np.cumsum(lens)]).tolist()
        kk, vv = k.view(nseg, cap, d).float().cpu().numpy(), v.view(nseg, cap, d).float().cpu().numpy()
        bb, pp = beta.view(nseg, cap).cpu().numpy(), pos.view(nseg, cap).cpu().numpy()
        for sg in range(nseg):
            n = lens[sg]
            assert np.array_equal(pp[sg, :n], rp[sg]), (seed, sg)
            assert np.array_equal(bb[sg, :n], rb[sg])
            assert np.array_equal(kk[sg, :n], rk[sg])
            assert np.array_equal(vv[sg, :n], rv[sg])

    def attend():
        q = torch.randn(bsz, hq, d, generator=gen).to(dtype).to(DEV)
        out = torch.full_like(q, float("nan"))
        ops.decode_attn(q, k, v, ln, None, cap, out, ws, hkv, d ** -0.5, cap, status)
        lens = [len(x) for x in rb]
        want = orc.varlen_gqa_attention(q[:, :, None].float().cpu().numpy(), np.concatenate(rk), np.concatenate(rv),
                                        np.concatenate([[0], np.cumsum(lens)]), bsz, hkv)[:, 0]
        assert np.max(np.abs(out.float().cpu().numpy() - want)) <= tol, (seed, d, dtype, bsz, hkv, group, m, buf, prompt)

    feed(prompt)
    evict()
    check_state()
    for _ in range(steps):
        feed(1)
        attend()
        evict()
    check_state()
    assert max(len(x) for x in rb) < m + buf
