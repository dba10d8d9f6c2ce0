"""The fused kernels of the decode step (tkv_add_rmsnorm, tkv_silu_mul, tkv_decode_prep) one by one against the plain
PyTorch ops they replace, in the model dtype, on seeded random shapes.  The kernels round where the eager sequence rounds
(src/trimkv/models/qwen3/modeling_trimkv_qwen3.py:328-353, 414-437), so the results agree to one or two units in the last place
of the 16-bit type (reduction orders differ).  Needs a B200."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _ulp_close(got, want, ulps=1.0, floor=1e-3):
    """|got - want| <= ulps units in the last place (of the 16-bit dtype, at the magnitude of `want` or of `floor`)."""
    mant = 7 if got.dtype == torch.bfloat16 else 10
    g, w = got.float(), want.float()
    ulp = torch.exp2(torch.floor(torch.log2(torch.maximum(w.abs(), torch.full_like(w, floor)))) - mant)
    bad = (g - w).abs() > ulps * ulp
    assert not bool(bad.any()), (int(bad.sum()), float((g - w).abs().max()))


def _rmsnorm(x, w, eps):
    dt = x.dtype
    xf = x.float()
    xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return w * xf.to(dt)


@pytest.mark.parametrize("seed", range(8))
def test_add_rmsnorm_matches_the_eager_ops(seed):
    from trimkv_b200 import ops
    rng = np.random.default_rng(seed)
    dtype = [torch.bfloat16, torch.float16][seed % 2]
    rows, cols = int(rng.integers(1, 40)), int(rng.choice([64, 128, 1024, 2048, 5120]))
    gen = torch.Generator().manual_seed(seed)
    res = torch.randn(rows, cols, generator=gen).to(dtype).to(DEV)
    delta = (torch.randn(rows, cols, generator=gen) * 0.5).to(dtype).to(DEV)
    w = (1 + 0.1 * torch.randn(cols, generator=gen)).to(dtype).to(DEV)
    want_res = res + delta
    want_out = _rmsnorm(want_res, w, 1e-6)
    out = torch.empty_like(res)
    ops.add_rmsnorm(res, delta, w, out, 1e-6)
    assert torch.equal(res, want_res)                 # one rounded addition: exact
    _ulp_close(out, want_out, ulps=2.0)               # the normalised value may round the other way, then times the weight
    # without a delta the residual stream is left alone
    res2, out2 = want_res.clone(), torch.empty_like(res)
    ops.add_rmsnorm(res2, None, w, out2, 1e-6)
    assert torch.equal(res2, want_res) and torch.equal(out2, out)


@pytest.mark.parametrize("seed", range(6))
def test_silu_mul_matches_the_eager_ops(seed):
    from trimkv_b200 import ops
    rng = np.random.default_rng(100 + seed)
    dtype = [torch.bfloat16, torch.float16][seed % 2]
    rows, inter = int(rng.integers(1, 40)), int(rng.choice([8, 96, 512, 6144]))
    gu = (torch.randn(rows, 2 * inter, generator=torch.Generator().manual_seed(seed)) * 2).to(dtype).to(DEV)
    out = torch.empty(rows, inter, dtype=dtype, device=DEV)
    ops.silu_mul(gu, out)
    _ulp_close(out, F.silu(gu[:, :inter]) * gu[:, inter:])


@pytest.mark.parametrize("seed", range(12))
def test_decode_prep_matches_the_eager_ops(seed):
    """q/k RMSNorm (or none), RoPE, the gate's tail and the append, against the module-level ops on the same inputs."""
    from trimkv_b200 import ops
    from trimkv_b200.modeling_trimkv import apply_rotary_pos_emb
    rng = np.random.default_rng(200 + seed)
    dtype = [torch.bfloat16, torch.float16][seed % 2]
    bsz, hkv, group = int(rng.integers(1, 6)), int(rng.choice([1, 2, 4, 8])), int(rng.choice([1, 2, 4]))
    hq, d, gi = hkv * group, 128, int(rng.choice([16, 32, 128, 256]))
    with_norm = bool(seed % 3)
    cap, old_len, position = 40, int(rng.integers(0, 39)), int(rng.integers(0, 100000))
    gen = torch.Generator().manual_seed(seed)
    cols = (hq + 2 * hkv) * d + gi
    qkvg = torch.randn(bsz, cols, generator=gen).to(dtype).to(DEV)
    qw = (1 + 0.1 * torch.randn(d, generator=gen)).to(dtype).to(DEV) if with_norm else None
    kw = (1 + 0.1 * torch.randn(d, generator=gen)).to(dtype).to(DEV) if with_norm else None
    w2 = (torch.randn(hkv, gi, generator=gen) * 0.2).to(dtype).to(DEV)
    gbias = (3 + torch.randn(hkv, generator=gen)).to(dtype).to(DEV)
    inv_freq = 1.0 / (1e6 ** (torch.arange(0, d, 2).float() / d))
    ang = position * inv_freq
    emb = torch.cat([ang, ang])
    cos, sin = emb.cos().to(dtype).to(DEV), emb.sin().to(dtype).to(DEV)
    nseg = bsz * hkv
    k_c = torch.zeros(nseg * cap, d, dtype=dtype, device=DEV)
    v_c = torch.zeros_like(k_c)
    b_c = torch.zeros(nseg * cap, dtype=torch.float32, device=DEV)
    p_c = torch.full((nseg * cap,), -7, dtype=torch.int32, device=DEV)
    ln = torch.full((nseg,), old_len, dtype=torch.int32, device=DEV)
    cu = (torch.arange(nseg + 1, dtype=torch.int32) * old_len).to(DEV)
    q_out = torch.empty(bsz, hq, 1, d, dtype=dtype, device=DEV)
    status = ops.new_status(DEV)
    ops.decode_prep(qkvg, qw, kw, 1e-6, cos, sin, w2, gbias, torch.tensor([position], device=DEV), q_out,
                    k_c, v_c, b_c, p_c, ln, cu, cap, hq, hkv, status)
    assert ops.read_status(status) == 0
    # the eager sequence
    q = qkvg[:, :hq * d].view(bsz, 1, hq, d)
    k = qkvg[:, hq * d:(hq + hkv) * d].view(bsz, 1, hkv, d)
    v = qkvg[:, (hq + hkv) * d:(hq + 2 * hkv) * d].view(bsz, 1, hkv, d)
    g = qkvg[:, (hq + 2 * hkv) * d:]
    if with_norm:
        q, k = _rmsnorm(q, qw, 1e-6), _rmsnorm(k, kw, 1e-6)
    q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    qr, kr = apply_rotary_pos_emb(q, k, cos.view(1, 1, d), sin.view(1, 1, d))
    logb = F.logsigmoid(F.linear(F.silu(g), w2) + gbias)                 # [B, Hkv]
    _ulp_close(q_out, qr, ulps=2.0, floor=1.0)                           # two rounded products and a rounded sum of O(1) terms
    rows = torch.arange(nseg, device=DEV) * cap + old_len
    _ulp_close(k_c[rows].view(bsz, hkv, d), kr[:, :, 0], ulps=2.0, floor=1.0)
    assert torch.equal(v_c[rows].view(bsz, hkv, d), v[:, :, 0])
    assert float((b_c[rows].view(bsz, hkv) - logb.float()).abs().max()) <= 2e-2     # a dot product of gi terms in 16 bits
    assert p_c[rows].cpu().tolist() == [position] * nseg
    assert ln.cpu().tolist() == [old_len + 1] * nseg
    assert cu.cpu().tolist() == [i * (old_len + 1) for i in range(nseg + 1)]
    untouched = torch.ones(nseg * cap, dtype=torch.bool, device=DEV)
    untouched[rows] = False
    assert not bool(k_c[untouched].any()) and bool((p_c[untouched] == -7).all())
