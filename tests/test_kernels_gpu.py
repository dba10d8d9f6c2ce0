"""Parity of the CUDA path (called through the C ABI) against the numpy oracle.  Needs a B200."""
import os

import numpy as np
import pytest
import torch

from oracle import trimkv_oracle as orc

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from trimkv_b200 import ops as _ops
    _ops.lib()  # fail loudly if the library is missing
    return _ops


def _slab(nseg, cap, d, dtype):
    return (torch.zeros(nseg * cap, d, dtype=dtype, device=DEV), torch.zeros(nseg * cap, d, dtype=dtype, device=DEV),
            torch.zeros(nseg * cap, dtype=torch.float32, device=DEV), torch.zeros(nseg * cap, dtype=torch.int32, device=DEV),
            torch.zeros(nseg, dtype=torch.int32, device=DEV), torch.zeros(nseg + 1, dtype=torch.int32, device=DEV))


def _logbeta(gen, *shape):
    return torch.nn.functional.logsigmoid(torch.randn(*shape, generator=gen) * 1.5 + 3.0)


# ---------------------------------------------------------------- append
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("b,h,d,steps", [(1, 8, 128, [5, 1, 1, 3, 40, 1]), (3, 2, 64, [1, 1, 9, 1]), (2, 1, 128, [17])])
def test_append_matches_oracle(ops, dtype, b, h, d, steps):
    gen = torch.Generator().manual_seed(7)
    nseg, cap = b * h, sum(steps) + 3
    k, v, beta, pos, ln, cu = _slab(nseg, cap, d, dtype)
    status = ops.new_status(DEV)
    ref_k = [np.zeros((0, d), np.float32) for _ in range(nseg)]
    ref_b = [np.zeros((0,), np.float32) for _ in range(nseg)]
    ref_p = [np.zeros((0,), np.int64) for _ in range(nseg)]
    seen = 0
    for s in steps:
        # [B,S,H,D] storage viewed as [B,H,S,D]: the strided layout the model hands over.
        kn = torch.randn(b, s, h, d, generator=gen).to(dtype).to(DEV).transpose(1, 2)
        vn = (kn.float() * 2).to(dtype)
        bn = _logbeta(gen, b, s, h).to(dtype).to(DEV).transpose(1, 2)
        pn = torch.arange(seen, seen + s, device=DEV)
        ops.append(k, v, beta, pos, ln, cu, kn, vn, bn, pn, cap, status)
        for sg in range(nseg):
            ref_k[sg] = np.concatenate([ref_k[sg], kn[sg // h, sg % h].float().cpu().numpy()])
            ref_b[sg] = np.concatenate([ref_b[sg], bn[sg // h, sg % h].float().cpu().numpy()])
            ref_p[sg] = np.concatenate([ref_p[sg], np.arange(seen, seen + s)])
        seen += s
    assert ops.read_status(status) == 0
    assert ln.cpu().tolist() == [seen] * nseg
    assert cu.cpu().tolist() == list(range(0, nseg * seen + 1, seen))
    kk, vv = k.view(nseg, cap, d).float().cpu().numpy(), v.view(nseg, cap, d).float().cpu().numpy()
    for sg in range(nseg):
        assert np.array_equal(kk[sg, :seen], ref_k[sg])
        assert np.array_equal(vv[sg, :seen], (torch.from_numpy(ref_k[sg]) * 2).to(dtype).float().numpy())
        assert np.array_equal(beta.view(nseg, cap)[sg, :seen].cpu().numpy(), ref_b[sg])
        assert np.array_equal(pos.view(nseg, cap)[sg, :seen].cpu().numpy(), ref_p[sg])


def test_append_over_capacity_sets_status_and_skips(ops):
    k, v, beta, pos, ln, cu = _slab(2, 4, 128, torch.bfloat16)
    status = ops.new_status(DEV)
    kn = torch.ones(1, 2, 3, 128, dtype=torch.bfloat16, device=DEV)
    bn = torch.zeros(1, 2, 3, dtype=torch.bfloat16, device=DEV)
    ops.append(k, v, beta, pos, ln, None, kn, kn, bn, torch.arange(3, device=DEV), 4, status)
    assert ops.read_status(status) == 0 and ln.cpu().tolist() == [3, 3]
    ops.append(k, v, beta, pos, ln, None, kn, kn, bn, torch.arange(3, 6, device=DEV), 4, status)
    assert ops.read_status(status) == 1      # TKV_DEV_CAPACITY
    assert ln.cpu().tolist() == [3, 3]       # nothing written
    assert ops.read_status(status) == 0      # cleared by the read


# ---------------------------------------------------------------- eviction
def _fill(gen, nseg, cap, d, lens, dtype, beta_fn, step):
    k, v, beta, pos, ln, cu = _slab(nseg, cap, d, dtype)
    kv = torch.randn(nseg, cap, d, generator=gen).to(dtype)
    k.copy_(kv.view(-1, d)); v.copy_((kv.float() + 1).to(dtype).view(-1, d))
    b = beta_fn(gen, nseg, cap)
    beta.copy_(b.view(-1))
    p = torch.stack([torch.sort(torch.randperm(step, generator=gen)[:cap])[0] for _ in range(nseg)]).to(torch.int32)
    pos.copy_(p.view(-1))
    ln.copy_(torch.tensor(lens, dtype=torch.int32))
    return (k, v, beta, pos, ln, cu), kv.float().numpy(), b.numpy(), p.numpy().astype(np.int64)


def _bf16_logbeta(gen, *shape):
    return _logbeta(gen, *shape).to(torch.bfloat16).float()


def _coarse_logbeta(gen, *shape):
    vals = torch.tensor([-0.5, -0.25, -0.125, -0.0, 0.0])
    return vals[torch.randint(0, 5, shape, generator=gen)]


CASES = [
    # nseg, cap, d, M, trigger, lens-spec, dtype, beta generator
    (8, 640, 128, 512, 640, "full", torch.float32, _logbeta),            # config-1 steady state n = M+B
    (4, 4096, 128, 512, 640, "full", torch.float32, _logbeta),           # prefill-like n >> M
    (6, 700, 128, 256, 320, "ragged", torch.bfloat16, _bf16_logbeta),    # some segments below the trigger
    (5, 333, 64, 100, 101, "ragged", torch.bfloat16, _coarse_logbeta),   # heavy ties, -0.0/+0.0, odd sizes
    (1, 130, 128, 129, 130, "full", torch.bfloat16, _bf16_logbeta),      # evict exactly one token
    (3, 77, 128, 1, 2, "full", torch.float16, _coarse_logbeta),          # keep a single token
    (2, 4224, 128, 4096, 4224, "full", torch.bfloat16, _bf16_logbeta),   # config-2 steady state
    (2, 16512, 128, 16384, 16512, "full", torch.bfloat16, _bf16_logbeta),  # long segments: the 512-thread variant
    (3, 20000, 64, 15000, 15001, "ragged", torch.bfloat16, _coarse_logbeta),
    (2, 57000, 128, 4096, 57000, "full", torch.bfloat16, _bf16_logbeta),  # the longest segment the selection accepts
]


def _tail_heavy_logbeta(gen, *shape):
    """The newest rows score lowest: the kept rows are a prefix and nothing has to move."""
    b = torch.full(shape, -0.001)
    b[..., -40:] = -50.0
    return b


MULTI_CASES = [
    # nseg, cap, d, M, trigger, lens-spec, dtype, beta generator, CTAs per segment
    (8, 640, 128, 512, 640, "full", torch.float32, _logbeta, 4),
    (6, 384, 128, 256, 320, "ragged", torch.bfloat16, _bf16_logbeta, 3),
    (5, 133, 64, 100, 101, "ragged", torch.bfloat16, _coarse_logbeta, 8),     # ranges shorter than a tile
    (1, 130, 128, 129, 130, "full", torch.bfloat16, _bf16_logbeta, 2),
    (2, 4224, 128, 4096, 4224, "full", torch.bfloat16, _bf16_logbeta, 16),
    (3, 4224, 128, 4096, 4224, "full", torch.bfloat16, _coarse_logbeta, 5),
    (3, 2100, 64, 2000, 2001, "ragged", torch.float16, _coarse_logbeta, 7),
    (4, 1064, 128, 1024, 1064, "full", torch.bfloat16, _tail_heavy_logbeta, 4),  # kept rows are a prefix
    (2, 16512, 128, 16384, 16512, "full", torch.bfloat16, _bf16_logbeta, 32),
    (100, 384, 128, 256, 320, "ragged", torch.bfloat16, _bf16_logbeta, 8),      # more evicting segments than rows of the move grid
    (700, 160, 64, 128, 129, "ragged", torch.float16, _coarse_logbeta, 2),      # 2 x 296 blocks walk up to 700 segments
]


@pytest.mark.parametrize("nseg,cap,d,m,trigger,spec,dtype,beta_fn,ctas", MULTI_CASES)
def test_evict_with_several_ctas_per_segment_bit_exact(ops, nseg, cap, d, m, trigger, spec, dtype, beta_fn, ctas):
    _evict_case(ops, nseg, cap, d, m, trigger, spec, dtype, beta_fn, ctas)


@pytest.mark.parametrize("nseg,cap,d,m,trigger,spec,dtype,beta_fn", CASES)
def test_evict_inplace_bit_exact(ops, nseg, cap, d, m, trigger, spec, dtype, beta_fn):
    _evict_case(ops, nseg, cap, d, m, trigger, spec, dtype, beta_fn, 1)


def _evict_case(ops, nseg, cap, d, m, trigger, spec, dtype, beta_fn, ctas):
    gen = torch.Generator().manual_seed(11)
    if spec == "full":
        lens = [cap] * nseg
    else:
        lens = [int(x) for x in torch.randint(m // 2, cap + 1, (nseg,), generator=gen)]
        lens[0], lens[-1] = cap, trigger
    step = 4 * cap
    (k, v, beta, pos, ln, cu), kv, b, p = _fill(gen, nseg, cap, d, lens, dtype, beta_fn, step)
    status = ops.new_status(DEV)
    kept = torch.full((nseg, m), -1, dtype=torch.int32, device=DEV)
    q_idx = step + 1
    if ctas == 1:
        ops.evict(k, v, beta, pos, ln, cu, nseg, nseg, cap, q_idx, m, trigger, cap, kept, status)
    else:
        ws = ops.evict_multi_workspace(nseg, m, ctas, DEV)
        ws.fill_(0x5a5a5a5a)                       # the call must not depend on what the scratch holds
        ops.evict_multi(k, v, beta, pos, ln, cu, nseg, nseg, cap, q_idx, m, trigger, cap, ctas, ws,
                        kept_idx_out=kept, status=status)
    assert ops.read_status(status) == 0
    new_len = ln.cpu().numpy()
    kk = k.view(nseg, cap, d).float().cpu().numpy()
    vv = v.view(nseg, cap, d).float().cpu().numpy()
    bb, pp = beta.view(nseg, cap).cpu().numpy(), pos.view(nseg, cap).cpu().numpy()
    v_src = (torch.from_numpy(kv) + 1).to(dtype).float().numpy()
    for s in range(nseg):
        n = lens[s]
        if n >= trigger and n > m:
            sc = orc.retention_scores(b[s, :n], p[s, :n], q_idx)
            want = orc.canonical_topm(sc[None], m)[0]
            assert np.array_equal(kept[s].cpu().numpy(), want)
            assert new_len[s] == m
        else:
            want = np.arange(n)
            assert new_len[s] == n
        assert np.array_equal(pp[s, :len(want)], p[s, want])
        assert np.array_equal(bb[s, :len(want)], b[s, want])
        assert np.array_equal(kk[s, :len(want)], kv[s, want])
        assert np.array_equal(vv[s, :len(want)], v_src[s, want])
    assert np.array_equal(cu.cpu().numpy(), np.concatenate([[0], np.cumsum(new_len)]))
    # idempotence: nothing reaches the trigger any more unless trigger <= M was asked for
    before = (k.clone(), pos.clone(), ln.clone())
    ops.evict(k, v, beta, pos, ln, cu, nseg, nseg, cap, q_idx, m, max(trigger, m + 1), cap, None, status)
    assert torch.equal(before[0], k) and torch.equal(before[1], pos) and torch.equal(before[2], ln)


def test_select_at_the_longest_supported_prompt(ops):
    """Prompt hand-off at the size limit of the selection (57 000 tokens per segment: the keys fill the shared memory a
    block may have); one token more is refused on the host."""
    gen = torch.Generator().manual_seed(13)
    nseg, n, m = 3, 57000, 4096
    b = _coarse_logbeta(gen, nseg, n).to(DEV)
    p = torch.arange(n, dtype=torch.int32, device=DEV)
    kept = torch.empty(nseg, m, dtype=torch.int32, device=DEV)
    cnt = torch.empty(nseg, dtype=torch.int32, device=DEV)
    status = ops.new_status(DEV)
    ops.evict_select(b, p, None, n, nseg, n + 1, m, m + 128, n, kept, cnt, status)
    assert ops.read_status(status) == 0
    want = orc.canonical_topm(orc.retention_scores(b.cpu().numpy(), np.arange(n), n + 1), m)
    assert np.array_equal(kept.cpu().numpy(), want) and cnt.cpu().tolist() == [m] * nseg
    b1 = torch.zeros(1, n + 1, device=DEV)
    with pytest.raises(Exception):
        ops.evict_select(b1, torch.arange(n + 1, dtype=torch.int32, device=DEV), None, n + 1, 1, n + 2, m, m + 128, n + 1,
                         kept[:1], cnt[:1], status)


def test_evict_grouped_cu_seqlens(ops):
    """Several layers in one launch: cu_seqlens is rebuilt per group of B*Hkv segments."""
    gen = torch.Generator().manual_seed(5)
    layers, nseg, cap, d, m = 3, 4, 96, 128, 64
    total = layers * nseg
    (k, v, beta, pos, ln, _), kv, b, p = _fill(gen, total, cap, d, [cap] * total, torch.bfloat16, _bf16_logbeta, 500)
    cu = torch.zeros(layers, nseg + 1, dtype=torch.int32, device=DEV)
    ops.evict(k, v, beta, pos, ln, cu, nseg, total, cap, 501, m, cap, cap, None, None)
    assert cu.cpu().tolist() == [list(range(0, nseg * m + 1, m))] * layers
    want = orc.canonical_topm(orc.retention_scores(b, p, 501), m)
    assert np.array_equal(pos.view(total, cap)[:, :m].cpu().numpy(), np.take_along_axis(p, want, -1))


def test_select_then_compact_from_dense_prompt(ops):
    """Prefill hand-off: select on the dense prompt, gather into a capacity-strided cache."""
    gen = torch.Generator().manual_seed(3)
    bsz, h, n, d, m, cap = 2, 3, 1000, 128, 300, 364
    nseg = bsz * h
    kd = torch.randn(bsz, n, h, d, generator=gen).to(torch.bfloat16).to(DEV).transpose(1, 2)  # strided view
    vd = (kd.float() - 1).to(torch.bfloat16)
    b = _bf16_logbeta(gen, nseg, n).to(DEV)
    p = torch.arange(n, dtype=torch.int32, device=DEV)
    kept = torch.empty(nseg, m, dtype=torch.int32, device=DEV)
    cnt = torch.empty(nseg, dtype=torch.int32, device=DEV)
    status = ops.new_status(DEV)
    ops.evict_select(b, p, None, n, nseg, n + 1, m, m + 64, n, kept, cnt, status)
    want = orc.canonical_topm(orc.retention_scores(b.cpu().numpy(), np.arange(n), n + 1), m)
    assert np.array_equal(kept.cpu().numpy(), want) and cnt.cpu().tolist() == [m] * nseg
    k, v, beta, pos, ln, cu = _slab(nseg, cap, d, torch.bfloat16)
    ops.compact(k, v, beta, pos, cap, kd, vd, b, p.expand(nseg, n).contiguous(), kept, cnt, ln, cu, nseg, status)
    assert ops.read_status(status) == 0
    assert ln.cpu().tolist() == [m] * nseg and cu.cpu().tolist() == list(range(0, nseg * m + 1, m))
    kk = k.view(bsz, h, cap, d)[:, :, :m].float().cpu().numpy()
    src = kd.float().cpu().numpy()
    assert np.array_equal(kk, np.take_along_axis(src, want.reshape(bsz, h, m)[..., None], axis=2))
    assert np.array_equal(pos.view(nseg, cap)[:, :m].cpu().numpy(), want)


def test_full_size_eviction_properties(ops):
    """Benchmark-spec configs[2] sizes (2048 segments, M=4096, B=128): properties that hold for all segments, and the
    oracle's selection on a sample of them."""
    gen = torch.Generator(device=DEV).manual_seed(0)
    nseg, m, bsz, d = 2048, 4096, 128, 128
    cap = m + bsz
    k = torch.randn(nseg * cap, d, generator=gen, device=DEV, dtype=torch.bfloat16)
    v = torch.randn(nseg * cap, d, generator=gen, device=DEV, dtype=torch.bfloat16)
    beta = torch.nn.functional.logsigmoid(torch.randn(nseg, cap, generator=gen, device=DEV) * 1.5 + 3).bfloat16().float()
    step = 4 * m
    pos = torch.sort(torch.rand(nseg, step, generator=gen, device=DEV).argsort(-1)[:, :cap], -1)[0].to(torch.int32)
    ln = torch.randint(m, cap + 1, (nseg,), generator=gen, device=DEV, dtype=torch.int32)
    cu = torch.zeros(nseg + 1, dtype=torch.int32, device=DEV)
    k0, v0, b0, p0, l0 = k.clone(), v.clone(), beta.clone(), pos.clone(), ln.clone()
    status = ops.new_status(DEV)
    ops.evict(k, v, beta.view(-1), pos.view(-1), ln, cu, nseg, nseg, cap, step + 1, m, m + 1, cap, None, status)
    assert ops.read_status(status) == 0
    fired = l0 > m
    assert torch.equal(ln, torch.where(fired, torch.full_like(l0, m), l0))
    assert torch.equal(cu[1:].long(), ln.long().cumsum(0))
    valid = torch.arange(cap, device=DEV)[None, :] < l0[:, None]
    score = (beta.new_tensor(float(step + 1)) - p0.float()) * b0
    score = torch.where(valid, score, torch.full_like(score, -float("inf")))
    # kept positions ascending and a subset of the old ones; kept set = M best scores (threshold property)
    kp = pos[:, :m]
    assert bool((kp[:, 1:] > kp[:, :-1]).all())
    thr = torch.topk(score, m, dim=-1).values[:, -1]
    new_score = (float(step + 1) - kp.float()) * beta[:, :m]
    assert bool((new_score[fired] >= thr[fired, None]).all())
    assert torch.equal(new_score.sort(-1, descending=True)[0][fired], torch.topk(score, m, -1).values[fired])
    # payload moved with its row: look each kept position up in the original segment
    idx = torch.searchsorted(p0.contiguous(), kp.contiguous())
    rows = (torch.arange(nseg, device=DEV)[:, None] * cap + idx).view(-1)
    assert torch.equal(k.view(nseg, cap, d)[:, :m].reshape(-1, d), k0[rows])
    assert torch.equal(v.view(nseg, cap, d)[:, :m].reshape(-1, d), v0[rows])
    # the oracle's canonical selection (ties to the lower index) on a sample of 96 segments: kept positions,
    # log beta and the K/V payload bit for bit
    rng = np.random.default_rng(1)
    sample = np.unique(np.concatenate([rng.choice(nseg, 94, replace=False), [0, nseg - 1]]))
    l0_h, b0_h, p0_h = l0.cpu().numpy(), b0.cpu().numpy(), p0.cpu().numpy()
    for sgm in sample:
        n = int(l0_h[sgm])
        if n <= m:
            continue
        idx = orc.canonical_topm(orc.retention_scores(b0_h[sgm, :n], p0_h[sgm, :n], step + 1), m)
        assert np.array_equal(pos[sgm, :m].cpu().numpy(), p0_h[sgm, idx]), sgm
        assert np.array_equal(beta[sgm, :m].cpu().numpy(), b0_h[sgm, idx]), sgm
        src = torch.from_numpy(idx).to(DEV) + sgm * cap
        assert torch.equal(k.view(nseg, cap, d)[sgm, :m], k0[src]) and torch.equal(v.view(nseg, cap, d)[sgm, :m], v0[src]), sgm


# ---------------------------------------------------------------- decode attention
@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 2e-2), (torch.float16, 5e-3)])
@pytest.mark.parametrize("bsz,hq,hkv,d,cap,lens_spec", [
    (2, 16, 8, 128, 300, "ragged"), (1, 8, 8, 128, 70, "ragged"), (3, 40, 8, 128, 1100, "ragged"),
    (2, 32, 8, 128, 2100, "full"), (2, 8, 2, 64, 257, "ragged"), (1, 2, 1, 128, 5, "tiny"),
])
def test_decode_attention_vs_oracle(ops, dtype, tol, bsz, hq, hkv, d, cap, lens_spec):
    gen = torch.Generator().manual_seed(21)
    nseg = bsz * hkv
    if lens_spec == "full":
        lens = [cap] * nseg
    elif lens_spec == "tiny":
        lens = [1] * nseg
    else:
        lens = [int(x) for x in torch.randint(1, cap + 1, (nseg,), generator=gen)]
        lens[0] = 0 if nseg > 1 else lens[0]  # an empty segment yields zeros
        lens[-1] = cap
    q = torch.randn(bsz, 1, hq, d, generator=gen).to(dtype).to(DEV).transpose(1, 2)  # [B,Hq,1,D] strided
    k = torch.randn(nseg, cap, d, generator=gen).to(dtype).to(DEV)
    v = torch.randn(nseg, cap, d, generator=gen).to(dtype).to(DEV)
    ln = torch.tensor(lens, dtype=torch.int32, device=DEV)
    out = torch.empty(bsz, hq, d, dtype=dtype, device=DEV)
    max_len = max(lens)
    ws = torch.empty(ops.decode_attn_workspace_bytes(bsz, hq, hkv, d, max_len), dtype=torch.uint8, device=DEV)
    status = ops.new_status(DEV)
    ops.decode_attn(q[:, :, 0, :], k, v, ln, None, cap, out, ws, hkv, d ** -0.5, max_len, status)
    assert ops.read_status(status) == 0
    # oracle on the packed equivalent
    kf = torch.cat([k[s, :lens[s]] for s in range(nseg)]).float().cpu().numpy()
    vf = torch.cat([v[s, :lens[s]] for s in range(nseg)]).float().cpu().numpy()
    cu = np.concatenate([[0], np.cumsum(lens)])
    want = orc.varlen_gqa_attention(q.float().cpu().numpy(), kf, vf, cu, bsz, hkv)[:, 0]
    got = out.float().cpu().numpy()
    assert np.max(np.abs(got - want)) <= tol
    # packed layout addressed through cu_seqlens_k, as the reference's flat caches present it
    kp = torch.cat([k[s, :lens[s]] for s in range(nseg)]).contiguous()
    vp = torch.cat([v[s, :lens[s]] for s in range(nseg)]).contiguous()
    out2 = torch.empty_like(out)
    ops.decode_attn(q[:, :, 0, :], kp, vp, ln, torch.tensor(cu[:-1], dtype=torch.int32, device=DEV), 0, out2, ws, hkv,
                    d ** -0.5, max_len, status)
    # (a different split kernel may serve this layout, so compare with the oracle rather than bit for bit)
    assert np.max(np.abs(out2.float().cpu().numpy() - want)) <= tol


@pytest.mark.parametrize("bsz,hq,hkv,cap", [(4, 16, 8, 2100), (2, 32, 8, 4200), (1, 8, 8, 1030)])
def test_decode_attention_ragged_work_list(ops, bsz, hq, hkv, cap):
    """Grid sized by a bound on the total tokens: same partials, so the same bits as the dense grid; an insufficient
    bound is reported through the status word."""
    gen = torch.Generator().manual_seed(23)
    d, dtype, nseg = 128, torch.bfloat16, bsz * hkv
    lens = [int(x) for x in torch.randint(1, cap // 3, (nseg,), generator=gen)]
    lens[0], lens[1], lens[2], lens[-1] = 0, 256, 257, cap      # empty, exactly one chunk, one token more, the longest
    q = torch.randn(bsz, hq, d, generator=gen).to(dtype).to(DEV)
    k = torch.randn(nseg * cap, d, generator=gen).to(dtype).to(DEV)
    v = torch.randn(nseg * cap, d, generator=gen).to(dtype).to(DEV)
    ln = torch.tensor(lens, dtype=torch.int32, device=DEV)
    status = ops.new_status(DEV)
    dense = torch.empty_like(q)
    ws = torch.empty(ops.decode_attn_workspace_bytes(bsz, hq, hkv, d, cap), dtype=torch.uint8, device=DEV)
    ops.decode_attn(q, k, v, ln, None, cap, dense, ws, hkv, d ** -0.5, cap, status)
    total = sum(lens)
    for bound in (total, total + 1000):
        out = torch.full_like(q, float("nan"))
        wsr = torch.empty(ops.decode_attn_workspace_bytes_ragged(bsz, hq, hkv, d, cap, bound), dtype=torch.uint8, device=DEV)
        wsr.fill_(0xA5)
        ops.decode_attn(q, k, v, ln, None, cap, out, wsr, hkv, d ** -0.5, cap, status, total_len_bound=bound)
        assert ops.read_status(status) == 0
        assert torch.equal(out, dense)
    kf = torch.cat([k.view(nseg, cap, d)[s, :lens[s]] for s in range(nseg)]).float().cpu().numpy()
    vf = torch.cat([v.view(nseg, cap, d)[s, :lens[s]] for s in range(nseg)]).float().cpu().numpy()
    want = orc.varlen_gqa_attention(q[:, :, None].float().cpu().numpy(), kf, vf, np.concatenate([[0], np.cumsum(lens)]), bsz, hkv)[:, 0]
    assert np.max(np.abs(dense.float().cpu().numpy() - want)) <= 2e-2
    # a bound below the true total: the surplus work items are dropped and the status word says so
    small = total // 2
    wsr = torch.empty(ops.decode_attn_workspace_bytes_ragged(bsz, hq, hkv, d, cap, small), dtype=torch.uint8, device=DEV)
    ops.decode_attn(q, k, v, ln, None, cap, torch.empty_like(q), wsr, hkv, d ** -0.5, cap, status, total_len_bound=small)
    assert ops.read_status(status) == 2


def test_decode_attention_over_a_very_long_segment(ops):
    """70 000 and 300 cached tokens side by side (274 chunks for the long one: beyond the 255 the compact work list can
    address, so the call with a token bound must fall back to the full grid and give the same bits)."""
    gen = torch.Generator().manual_seed(29)
    bsz, hq, hkv, d, cap, dtype = 1, 8, 2, 128, 70000, torch.bfloat16
    lens = [cap, 300]
    q = torch.randn(bsz, hq, d, generator=gen).to(dtype).to(DEV)
    k = torch.randn(hkv * cap, d, generator=gen).to(dtype).to(DEV)
    v = torch.randn(hkv * cap, d, generator=gen).to(dtype).to(DEV)
    ln = torch.tensor(lens, dtype=torch.int32, device=DEV)
    status = ops.new_status(DEV)
    out = torch.full_like(q, float("nan"))
    ws = torch.empty(ops.decode_attn_workspace_bytes(bsz, hq, hkv, d, cap), dtype=torch.uint8, device=DEV)
    ops.decode_attn(q, k, v, ln, None, cap, out, ws, hkv, d ** -0.5, cap, status)
    assert ops.read_status(status) == 0
    kf = torch.cat([k.view(hkv, cap, d)[s, :lens[s]] for s in range(hkv)]).float().cpu().numpy()
    vf = torch.cat([v.view(hkv, cap, d)[s, :lens[s]] for s in range(hkv)]).float().cpu().numpy()
    want = orc.varlen_gqa_attention(q[:, :, None].float().cpu().numpy(), kf, vf, np.concatenate([[0], np.cumsum(lens)]), bsz, hkv)[:, 0]
    assert np.max(np.abs(out.float().cpu().numpy() - want)) <= 2e-2
    out2 = torch.full_like(q, float("nan"))
    wsr = torch.empty(ops.decode_attn_workspace_bytes_ragged(bsz, hq, hkv, d, cap, sum(lens)), dtype=torch.uint8, device=DEV)
    ops.decode_attn(q, k, v, ln, None, cap, out2, wsr, hkv, d ** -0.5, cap, status, total_len_bound=sum(lens))
    assert ops.read_status(status) == 0
    assert torch.equal(out2, out)


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 2e-2), (torch.float16, 5e-3)])
@pytest.mark.parametrize("bsz,hq,hkv,ql,cap", [(2, 16, 8, 3, 700), (1, 8, 4, 8, 300), (2, 16, 4, 7, 1100), (3, 2, 2, 5, 200),
                                               (1, 16, 8, 20, 600), (1, 8, 2, 48, 900), (2, 4, 4, 70, 400), (1, 16, 8, 32, 130)])
def test_multi_token_attention_vs_oracle(ops, dtype, tol, bsz, hq, hkv, ql, cap):
    """Several query tokens per request against caches that already hold them: bottom-right aligned causal mask per
    segment, query rows (token, head) on the MMA's N dimension: up to 16 rows on the decode kernel, more on the
    kernel with 64 rows per CTA (several row groups beyond that)."""
    gen = torch.Generator().manual_seed(29)
    d, nseg = 128, bsz * hkv
    lens = [int(x) for x in torch.randint(ql, cap + 1, (nseg,), generator=gen)]
    lens[0], lens[-1] = ql, cap                      # only the new tokens; a full segment (several chunks)
    if nseg > 2 and cap >= 256 + ql:
        lens[1] = 256 + ql - 1                       # the first new token sits exactly at a chunk boundary
    q = torch.randn(bsz, ql, hq, d, generator=gen).to(dtype).to(DEV)
    k = torch.randn(nseg, cap, d, generator=gen).to(dtype).to(DEV)
    v = torch.randn(nseg, cap, d, generator=gen).to(dtype).to(DEV)
    ln = torch.tensor(lens, dtype=torch.int32, device=DEV)
    out = torch.full((bsz, ql, hq, d), float("nan"), dtype=dtype, device=DEV)
    status = ops.new_status(DEV)
    ops.decode_attn_multi(q, k, v, ln, cap, out, hkv, d ** -0.5, max(lens), status=status)
    assert ops.read_status(status) == 0
    kf = torch.cat([k[s, :lens[s]] for s in range(nseg)]).float().cpu().numpy()
    vf = torch.cat([v[s, :lens[s]] for s in range(nseg)]).float().cpu().numpy()
    want = orc.varlen_gqa_attention(q.transpose(1, 2).float().cpu().numpy(), kf, vf, np.concatenate([[0], np.cumsum(lens)]), bsz, hkv)
    assert np.max(np.abs(out.float().cpu().numpy() - want)) <= tol
    # one query token through this entry point is the decode kernel's result
    out1 = torch.empty(bsz, 1, hq, d, dtype=dtype, device=DEV)
    ops.decode_attn_multi(q[:, -1:], k, v, ln, cap, out1, hkv, d ** -0.5, max(lens), status=status)
    assert np.max(np.abs(out1[:, 0].float().cpu().numpy() - want[:, -1])) <= tol


# ---------------------------------------------------------------- weight-streaming GEMM and its consumers
@pytest.mark.parametrize("m,n,k", [(32, 4224, 2048), (32, 2048, 2048), (32, 12288, 2048), (32, 2048, 6144),
                                   (5, 300, 128), (1, 128, 64), (17, 1000, 4096)])
def test_skinny_gemm_partials_sum_to_the_product(ops, m, n, k):
    gen = torch.Generator().manual_seed(m * 1000 + n)
    x = torch.randn(m, k, generator=gen).bfloat16().to(DEV)
    w = (torch.randn(n, k, generator=gen) * 0.05).bfloat16().to(DEV)
    splits = ops.skinny_gemm_splits(m, n, k)
    assert splits >= 1
    part = torch.full((splits, m, n), float("nan"), dtype=torch.float32, device=DEV)
    status = ops.new_status(DEV)
    assert ops.skinny_gemm(x, w, part, status) == splits
    assert ops.read_status(status) == 0
    got = part.sum(0)
    want = x.float() @ w.float().t()
    assert torch.isfinite(got).all()
    assert float((got - want).abs().max()) <= 1e-3 * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,n,k", [(32, 2048, 6144), (5, 384, 512), (16, 256, 64)])
def test_skinny_gemm_with_swiglu_prologue(ops, dtype, m, n, k):
    """SiLU(gate) * up computed inside the GEMM: the activation tile is bit-identical to tkv_silu_mul's output, so the
    partial sums equal those of tkv_skinny_gemm fed that output, and the sum is the eager product."""
    gen = torch.Generator().manual_seed(m + n + k)
    gu = torch.randn(m, 2 * k, generator=gen).to(dtype).to(DEV)
    w = (torch.randn(n, k, generator=gen) * 0.05).to(dtype).to(DEV)
    splits = ops.skinny_gemm_splits(m, n, k)
    status = ops.new_status(DEV)
    fused = torch.full((splits, m, n), float("nan"), dtype=torch.float32, device=DEV)
    assert ops.skinny_gemm_swiglu(gu, w, fused, status) == splits
    act = torch.empty(m, k, dtype=dtype, device=DEV)
    ops.silu_mul(gu, act)
    two_step = torch.empty_like(fused)
    ops.skinny_gemm(act, w, two_step, status)
    assert ops.read_status(status) == 0
    assert torch.equal(fused, two_step)
    eager = (torch.nn.functional.silu(gu[:, :k]) * gu[:, k:]).float() @ w.float().t()
    assert float((fused.sum(0) - eager).abs().max()) <= 2e-3 * max(1.0, float(eager.abs().max()))


def test_consumers_accept_gemm_partials(ops):
    """add_rmsnorm and silu_mul fed with fp32 partials + bias equal the same kernels fed with the rounded sum."""
    gen = torch.Generator().manual_seed(4)
    rows, cols, splits = 7, 512, 3
    part = torch.randn(splits, rows, cols, generator=gen).to(DEV)
    bias = torch.randn(cols, generator=gen).bfloat16().to(DEV)
    rounded = (part.sum(0) + bias.float()).bfloat16()
    res1 = torch.randn(rows, cols, generator=gen).bfloat16().to(DEV)
    res2 = res1.clone()
    w = torch.randn(cols, generator=gen).bfloat16().to(DEV)
    o1, o2 = torch.empty_like(res1), torch.empty_like(res1)
    ops.add_rmsnorm(res1, part, w, o1, 1e-6, splits, bias)
    ops.add_rmsnorm(res2, rounded, w, o2, 1e-6)
    assert torch.equal(res1, res2) and torch.equal(o1, o2)
    gu_part = torch.randn(splits, rows, 2 * cols, generator=gen).to(DEV)
    a1 = torch.empty(rows, cols, dtype=torch.bfloat16, device=DEV)
    a2 = torch.empty_like(a1)
    ops.silu_mul(gu_part, a1, splits)
    ops.silu_mul(gu_part.sum(0).bfloat16(), a2)
    assert torch.equal(a1, a2)


def _oracle_attention_sample(q, k_seg, v_seg, lens, hkv, sample):
    """fp32 oracle outputs [len(sample), G, D] for the sampled segments; k_seg(s) / v_seg(s) return that segment's rows."""
    bsz, hq, d = q.shape
    g = hq // hkv
    want = np.zeros((len(sample), g, d), np.float32)
    for i, s in enumerate(sample):
        b, h = divmod(int(s), hkv)
        n = int(lens[s])
        qs = q[b, h * g:(h + 1) * g].float().cpu().numpy()[None, :, None, :]   # [1, G, 1, D]: one request, one KV head
        ks, vs = k_seg(s)[:n].float().cpu().numpy(), v_seg(s)[:n].float().cpu().numpy()
        want[i] = orc.varlen_gqa_attention(qs, ks, vs, np.asarray([0, n], np.int32), 1, 1)[0, 0]
    return want


def test_full_size_attention_cross_check(ops):
    """benchmark-spec configs[3] sizes (batch 64, 32/8 heads, lognormal lengths in [64, 8192]): the tensor-core kernel on the
    capacity-strided layout and on the packed copy of the same cache (the reference's own layout), and the CUDA-core
    kernel on the packed copy, each against the fp32 oracle on a sample of 96 segments (the shortest, the longest and
    random ones) and against one another on all 512; plus two properties that need no second implementation
    (constant V gives that constant; the output is a convex combination of V rows)."""
    gen = torch.Generator(device=DEV).manual_seed(0)
    bsz, hq, hkv, d, cap = 64, 32, 8, 128, 8192
    nseg, g = bsz * hkv, hq // hkv
    lens = torch.exp(torch.randn(nseg, generator=gen, device=DEV) + 7.6246).clamp(64, 8192).round().to(torch.int32)
    q = torch.randn(bsz, hq, d, generator=gen, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(nseg * cap, d, generator=gen, device=DEV, dtype=torch.bfloat16)
    v = torch.randn(nseg * cap, d, generator=gen, device=DEV, dtype=torch.bfloat16)
    out = torch.empty(bsz, hq, d, dtype=torch.bfloat16, device=DEV)
    ws = torch.empty(ops.decode_attn_workspace_bytes(bsz, hq, hkv, d, cap), dtype=torch.uint8, device=DEV)
    status = ops.new_status(DEV)
    ops.decode_attn(q, k, v, lens, None, cap, out, ws, hkv, d ** -0.5, cap, status)
    mask = (torch.arange(cap, device=DEV)[None, :] < lens[:, None]).view(-1)
    kp, vp = k[mask].contiguous(), v[mask].contiguous()
    cu = torch.zeros(nseg + 1, dtype=torch.int32, device=DEV)
    cu[1:] = lens.cumsum(0)
    starts = cu[:-1].contiguous()
    out_packed_tc, out_packed_cc = torch.empty_like(out), torch.empty_like(out)
    ops.decode_attn(q, kp, vp, lens, starts, 0, out_packed_tc, ws, hkv, d ** -0.5, cap, status)                  # tensor cores
    ops.decode_attn(q, kp, vp, lens, starts, 0, out_packed_cc, ws, hkv, d ** -0.5, cap, status, packed_rows=0)   # CUDA cores
    assert ops.read_status(status) == 0
    assert float((out.float() - out_packed_cc.float()).abs().max()) <= 2e-2
    assert torch.equal(out, out_packed_tc)      # same tiles, same arithmetic: the layout changes addresses only
    lens_h = lens.cpu().numpy()
    order = np.argsort(lens_h)
    rng = np.random.default_rng(0)
    sample = np.unique(np.concatenate([order[:8], order[-8:], rng.choice(nseg, 80, replace=False)]))
    k3, v3 = k.view(nseg, cap, d), v.view(nseg, cap, d)
    want = _oracle_attention_sample(q, lambda s: k3[s], lambda s: v3[s], lens_h, hkv, sample)
    for name, o in (("strided/tc", out), ("packed/tc", out_packed_tc), ("packed/cuda-core", out_packed_cc)):
        got = o.float().view(bsz, hkv, g, d).cpu().numpy().reshape(nseg, g, d)[sample]
        assert np.max(np.abs(got - want)) <= 2e-2, name
    vmax = v.view(nseg, cap, d).float().masked_fill(~mask.view(nseg, cap, 1), -1e30).amax(1)   # per segment, per dim
    vmin = v.view(nseg, cap, d).float().masked_fill(~mask.view(nseg, cap, 1), 1e30).amin(1)
    o = out.float().view(bsz, hkv, hq // hkv, d)
    assert bool((o <= vmax.view(bsz, hkv, 1, d) + 2e-2).all()) and bool((o >= vmin.view(bsz, hkv, 1, d) - 2e-2).all())
    v.fill_(0.75)
    ops.decode_attn(q, k, v, lens, None, cap, out, ws, hkv, d ** -0.5, cap, status)
    assert float((out.float() - 0.75).abs().max()) <= 4e-3


def test_decode_attention_vs_flash_attn_varlen(ops):
    """Same-box cross-check against the library the reference calls: flash_attn_varlen_func with every
    (request, KV head) pair as one varlen sequence of an MQA problem, causal, default softmax scale
    (src/trimkv/attn/flash_attn.py:104-151).  Skipped where the installed wheel cannot run on this GPU."""
    try:
        from flash_attn.flash_attn_interface import flash_attn_varlen_func
    except Exception as e:  # not installed / not importable
        pytest.skip(f"flash_attn unavailable: {e}")
    gen = torch.Generator().manual_seed(12)
    bsz, hq, hkv, d, cap = 4, 16, 8, 128, 1500
    g, nseg = hq // hkv, bsz * hkv
    lens = [int(x) for x in torch.randint(1, cap + 1, (nseg,), generator=gen)]
    q = torch.randn(bsz, hq, d, generator=gen).bfloat16().to(DEV)
    k = torch.randn(nseg, cap, d, generator=gen).bfloat16().to(DEV)
    v = torch.randn(nseg, cap, d, generator=gen).bfloat16().to(DEV)
    ln = torch.tensor(lens, dtype=torch.int32, device=DEV)
    out = torch.empty(bsz, hq, d, dtype=torch.bfloat16, device=DEV)
    ws = torch.empty(ops.decode_attn_workspace_bytes(bsz, hq, hkv, d, cap), dtype=torch.uint8, device=DEV)
    ops.decode_attn(q, k, v, ln, None, cap, out, ws, hkv, d ** -0.5, max(lens), None)
    # the reference's packing: sequence s = b*Hkv + h holds the G query heads of KV head h as G "heads" of one query token
    packed_q = q.view(bsz, hkv, g, d).reshape(nseg, g, d).contiguous()
    kp = torch.cat([k[s, :lens[s]] for s in range(nseg)]).unsqueeze(1).contiguous()
    vp = torch.cat([v[s, :lens[s]] for s in range(nseg)]).unsqueeze(1).contiguous()
    cu_k = torch.zeros(nseg + 1, dtype=torch.int32, device=DEV)
    cu_k[1:] = ln.cumsum(0)
    cu_q = torch.arange(0, nseg + 1, dtype=torch.int32, device=DEV)
    try:
        ref = flash_attn_varlen_func(packed_q, kp, vp, cu_q, cu_k, max_seqlen_q=1, max_seqlen_k=max(lens), dropout_p=0.0,
                                     causal=True)
        torch.cuda.synchronize()
    except Exception as e:
        pytest.skip(f"flash_attn cannot run here: {type(e).__name__}: {e}")
    want = ref.view(bsz, hkv, g, d).reshape(bsz, hq, d)
    assert float((out.float() - want.float()).abs().max()) <= 2e-2


def test_peer_wait_gives_up_when_no_peer_answers(ops):
    """The receiving side of the head-sharded exchange never waits without a bound: with flags nobody raises, the wait
    kernel runs out of polls, reports TKV_DEV_TIMEOUT through the status word and the stream stays usable."""
    flags = torch.zeros(4, dtype=torch.int32, device=DEV)
    sync = torch.zeros(3, dtype=torch.int32, device=DEV)
    status = ops.new_status(DEV)
    ops.peer_wait(flags, sync, 4, 1, status, max_polls=2000)          # about a millisecond
    assert ops.read_status(status) == 4
    assert sync.tolist() == [0, 0, 1]                                  # the exchange is counted all the same
    # flags already at the expected count: returns at once with a clean status
    flags.fill_(2)
    ops.peer_wait(flags, sync, 4, 1, status, max_polls=2000)
    assert ops.read_status(status) == 0 and sync.tolist() == [0, 0, 2]
    x = torch.arange(8, device=DEV).sum().item()                       # the context is fine
    assert x == 28


def test_push_exchange_two_ranks_emulated_on_one_gpu(ops):
    """The head-sharded exchange with both "ranks" on one GPU, one after the other on one stream: each rank's gathered
    buffer and flag array live in this GPU's memory, rank 0's merge kernel stores its column block into both buffers
    and raises its flag in rank 1's array, then rank 1's does the same; only then do the wait kernels run, so
    they find their flags raised and never spin.  Both buffers must hold what the oracle computes for all heads.
    Two exchanges in a row (the counters advance): one chunk per segment (the split kernel writes the output itself)
    and several chunks (merged partials)."""
    import ctypes
    gen = torch.Generator().manual_seed(31)
    bsz, hq, hkv, d, world = 3, 8, 4, 128, 2          # per rank: 8 query / 4 KV heads; 16 / 8 in total
    width = world * hq * d
    flags = [torch.zeros(world, dtype=torch.int32, device=DEV) for _ in range(world)]
    sync = [torch.zeros(3, dtype=torch.int32, device=DEV) for _ in range(world)]
    status = ops.new_status(DEV)
    flag_ptrs = (ctypes.c_void_p * world)(*[f.data_ptr() for f in flags])
    for call, cap in enumerate((200, 1300)):
        nseg = bsz * hkv
        gathered = [torch.full((bsz, width), 7.0, dtype=torch.bfloat16, device=DEV) for _ in range(world)]
        out_ptrs = (ctypes.c_void_p * world)(*[g.data_ptr() for g in gathered])
        want = np.zeros((bsz, width), np.float32)
        for rank in range(world):
            lens = torch.randint(1, cap + 1, (nseg,), generator=gen).to(torch.int32)
            lens[-1] = cap
            q = torch.randn(bsz, hq, d, generator=gen).bfloat16().to(DEV)
            k = torch.randn(nseg * cap, d, generator=gen).bfloat16().to(DEV)
            v = torch.randn(nseg * cap, d, generator=gen).bfloat16().to(DEV)
            local = torch.empty(bsz, hq, d, dtype=torch.bfloat16, device=DEV)
            ws = torch.empty(ops.decode_attn_workspace_bytes(bsz, hq, hkv, d, cap), dtype=torch.uint8, device=DEV)
            ops.decode_attn_push(q, k, v, lens.to(DEV), cap, local, ws, hkv, d ** -0.5, cap, out_ptrs, flag_ptrs, world, rank,
                                 width, rank * hq * d, sync[rank], status)
            mask = (torch.arange(cap)[None, :] < lens[:, None]).view(-1)
            cu = np.concatenate([[0], np.cumsum(lens.numpy())]).astype(np.int32)
            want[:, rank * hq * d:(rank + 1) * hq * d] = orc.varlen_gqa_attention(
                q.float().cpu().numpy()[:, :, None, :], k.float().cpu()[mask].numpy(), v.float().cpu()[mask].numpy(),
                cu, bsz, hkv)[:, 0].reshape(bsz, hq * d)
        for rank in range(world):
            ops.peer_wait(flags[rank], sync[rank], world, rank, status, max_polls=1000)
        assert ops.read_status(status) == 0
        for rank in range(world):
            peer = 1 - rank
            assert int(flags[rank][peer]) == call + 1 and int(flags[rank][rank]) == 0   # a rank raises flags on peers only
            assert sync[rank].tolist() == [0, call + 1, call + 1]
            assert np.abs(gathered[rank].float().cpu().numpy() - want).max() <= 2e-2, (call, rank)


# ---------------------------------------------------------------- query-resident attention (many query tokens)
@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 2e-2), (torch.float16, 5e-3)])
@pytest.mark.parametrize("bsz,hq,hkv,cap,ql,lens_spec", [
    (2, 4, 2, 700, 40, "ragged"),        # 80 query rows: one block, padded
    (2, 4, 2, 900, 100, "ragged"),       # 200 rows: two blocks, the second partly filled
    (1, 8, 2, 300, 300, "dense"),        # a prompt pass: seg_len NULL, every token is new, 1200 rows
    (3, 2, 2, 260, 64, "first"),         # G = 1; one segment holds nothing but the new tokens
    (1, 16, 8, 1500, 8, "ragged"),       # 16 rows against long segments: many tiles, few rescales
])
def test_prefill_attention_vs_oracle(ops, dtype, tol, bsz, hq, hkv, cap, ql, lens_spec):
    d = 128
    gen = torch.Generator().manual_seed(41)
    nseg = bsz * hkv
    if lens_spec == "dense":
        lens = [cap] * nseg
    else:
        lens = [int(x) for x in torch.randint(ql, cap + 1, (nseg,), generator=gen)]
        lens[-1] = cap
        if lens_spec == "first":
            lens[0] = ql
    q = (torch.randn(bsz, ql, hq, d, generator=gen) * 1.5).to(dtype).to(DEV)
    k = torch.randn(nseg, cap, d, generator=gen).to(dtype).to(DEV)
    v = torch.randn(nseg, cap, d, generator=gen).to(dtype).to(DEV)
    for s_, n in enumerate(lens):            # rows beyond a segment's length hold garbage that must not leak
        k[s_, n:] = float("nan")
        v[s_, n:] = float("inf")
    ln = None if lens_spec == "dense" else torch.tensor(lens, dtype=torch.int32, device=DEV)
    out = torch.full((bsz, ql, hq, d), float("nan"), dtype=dtype, device=DEV)
    status = ops.new_status(DEV)
    ops.prefill_attn(q, k, v, ln, cap, out, hkv, d ** -0.5, cap, status)
    assert ops.read_status(status) == 0
    kp = torch.cat([k[s_, :n] for s_, n in enumerate(lens)]).float().cpu().numpy()
    vp = torch.cat([v[s_, :n] for s_, n in enumerate(lens)]).float().cpu().numpy()
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    want = orc.varlen_gqa_attention(q.float().cpu().numpy().transpose(0, 2, 1, 3), kp, vp, cu, bsz, hkv)
    got = out.float().cpu().numpy()
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= tol


def test_prefill_attention_strided_queries_and_multi_token_kernels_agree(ops):
    """The query tensor as the model hands it over ([B,Hq,Q,D] transposed to token-major strides), and the same
    problem through tkv_decode_attn_multi (32 rows per CTA, split-KV partials): two kernels, one result."""
    gen = torch.Generator().manual_seed(43)
    bsz, hq, hkv, d, cap, ql = 2, 4, 2, 128, 1100, 16
    nseg = bsz * hkv
    lens = torch.randint(ql, cap + 1, (nseg,), generator=gen).to(torch.int32)
    q = torch.randn(bsz, hq, ql, d, generator=gen).bfloat16().to(DEV).transpose(1, 2)      # [B,Q,Hq,D] view
    k = torch.randn(nseg * cap, d, generator=gen).bfloat16().to(DEV)
    v = torch.randn(nseg * cap, d, generator=gen).bfloat16().to(DEV)
    ln = lens.to(DEV)
    a = torch.empty(bsz, ql, hq, d, dtype=torch.bfloat16, device=DEV)
    b_ = torch.empty_like(a)
    status = ops.new_status(DEV)
    ops.prefill_attn(q, k, v, ln, cap, a, hkv, d ** -0.5, cap, status)
    ops.decode_attn_multi(q, k, v, ln, cap, b_, hkv, d ** -0.5, cap, status=status)
    assert ops.read_status(status) == 0
    assert float((a.float() - b_.float()).abs().max()) <= 2e-2
