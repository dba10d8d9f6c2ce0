"""Seeded random shapes for the multi-token attention kernels (query-resident `tkv_prefill_attn` and split-KV
`tkv_decode_attn_multi`) against the numpy oracle: query-token counts from 2 to 300, one to eight query heads per KV head,
ragged lengths that include segments holding nothing but the new tokens, rows beyond a length filled with NaN/Inf, query
tensors with the model's head-major strides.  Needs a B200."""
import numpy as np
import pytest
import torch

from oracle import trimkv_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _draw(seed):
    rng = np.random.default_rng(5000 + seed)
    bsz, hkv, group = int(rng.integers(1, 4)), int(rng.choice([1, 2, 4])), int(rng.choice([1, 2, 4, 8]))
    ql = int(rng.choice([2, 3, 5, 9, 16, 17, 31, 64, 100, 129, 300]))
    cap = ql + int(rng.choice([0, 1, 60, 127, 128, 129, 700, 2100]))
    cap = max(cap, -(-128 // (bsz * hkv)))         # the tensor maps want at least one 128-row tile behind K and V
    dtype = [torch.bfloat16, torch.float16][int(rng.integers(0, 2))]
    return rng, bsz, hkv, group, ql, cap, dtype


@pytest.mark.parametrize("seed", range(20))
def test_random_multi_token_shapes_match_oracle(seed):
    from trimkv_b200 import ops
    rng, bsz, hkv, group, ql, cap, dtype = _draw(seed)
    d, hq, nseg = 128, hkv * group, bsz * hkv
    gen = torch.Generator().manual_seed(seed)
    lens = [int(x) for x in rng.integers(ql, cap + 1, nseg)]
    lens[0] = ql                                   # nothing cached before the new tokens
    lens[-1] = cap
    q = (torch.randn(bsz, hq, ql, d, generator=gen) * 1.5).to(dtype).to(DEV).transpose(1, 2)   # [B,Q,Hq,D] view, head-major storage
    k = torch.randn(nseg, cap, d, generator=gen).to(dtype).to(DEV)
    v = torch.randn(nseg, cap, d, generator=gen).to(dtype).to(DEV)
    for s, n in enumerate(lens):
        k[s, n:] = float("nan")
        v[s, n:] = float("inf")
    ln = torch.tensor(lens, dtype=torch.int32, device=DEV)
    status = ops.new_status(DEV)
    kp = torch.cat([k[s, :n] for s, n in enumerate(lens)]).float().cpu().numpy()
    vp = torch.cat([v[s, :n] for s, n in enumerate(lens)]).float().cpu().numpy()
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    want = orc.varlen_gqa_attention(q.float().cpu().numpy().transpose(0, 2, 1, 3), kp, vp, cu, bsz, hkv)
    tol = 2e-2 if dtype == torch.bfloat16 else 5e-3
    tag = (seed, bsz, hkv, group, ql, cap, dtype)
    out = torch.full((bsz, ql, hq, d), float("nan"), dtype=dtype, device=DEV)
    ops.prefill_attn(q, k.view(-1, d), v.view(-1, d), ln, cap, out, hkv, d ** -0.5, cap, status)
    assert ops.read_status(status) == 0, tag
    got = out.float().cpu().numpy()
    assert np.isfinite(got).all(), tag
    assert np.abs(got - want).max() <= tol, tag
    if ql * group <= 1024:                          # the split-KV kernels (16 or 32 rows per CTA) on the same problem
        out2 = torch.full_like(out, float("nan"))
        ops.decode_attn_multi(q, k.view(-1, d), v.view(-1, d), ln, cap, out2, hkv, d ** -0.5, cap, status=status)
        assert ops.read_status(status) == 0, tag
        got2 = out2.float().cpu().numpy()
        assert np.isfinite(got2).all(), tag
        assert np.abs(got2 - want).max() <= tol, tag
