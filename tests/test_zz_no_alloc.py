"""The allocation-free decode-attention entry point against the regular one.

`tkv_decode_attn_static` exists for hosts that cannot give the library a workspace (an arena that already owns
the device, a plug-in slot without an allocator, a loop that must not hit cudaMalloc's synchronisation): its
scratch is a fixed array inside the library.  Here it is called straight through the C ABI, twice in a row on
different inputs, and must reproduce `tkv_decode_attn` (which serves these shapes from the tensor-core kernel) and
the fp32 oracle within the 2e-2 bf16 tolerance of the other attention tests; the shapes only the CUDA-core kernel
serves (packed layout, head_dim 64, f16) are checked against the oracle too; a problem larger than the built-in
array must be refused cleanly.
This file sorts last on purpose so a run that stops at the first failure has already run everything else.
"""
import numpy as np
import pytest
import torch

from oracle import trimkv_oracle as orc

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TOL = 2e-2  # same bound as tests/test_kernels_gpu.py::test_decode_attention_vs_oracle for bf16


def _problem(seed, bsz, hq, hkv, d, cap):
    gen = torch.Generator().manual_seed(seed)
    nseg = bsz * hkv
    q = torch.randn(bsz, hq, d, generator=gen).bfloat16().to(DEV)
    k = torch.randn(nseg * cap, d, generator=gen).bfloat16().to(DEV)
    v = torch.randn(nseg * cap, d, generator=gen).bfloat16().to(DEV)
    ln = torch.randint(1, cap + 1, (nseg,), generator=gen).to(torch.int32).to(DEV)
    return q, k, v, ln


def test_static_scratch_entry_point_matches_workspace_entry_point():
    from trimkv_b200 import _lib, ops
    lib = _lib.lib()
    stream = torch.cuda.current_stream(torch.device(DEV)).cuda_stream
    for call, (seed, bsz, hq, hkv, d, cap) in enumerate([(1, 4, 16, 8, 128, 1500), (2, 3, 40, 8, 128, 700)]):
        q, k, v, ln = _problem(seed, bsz, hq, hkv, d, cap)
        want = torch.empty(bsz, hq, d, dtype=torch.bfloat16, device=DEV)
        ws = torch.empty(ops.decode_attn_workspace_bytes(bsz, hq, hkv, d, cap), dtype=torch.uint8, device=DEV)
        ops.decode_attn(q, k, v, ln, None, cap, want, ws, hkv, d ** -0.5, cap, None)
        got = torch.full_like(want, float("nan"))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc = lib.tkv_decode_attn_static(q.data_ptr(), q.stride(0), q.stride(1), k.data_ptr(), v.data_ptr(),
                                        ln.data_ptr(), None, cap, got.data_ptr(), bsz, hq, hkv, d, _lib.TKV_BF16,
                                        d ** -0.5, cap, None, stream)
        assert rc == 0, lib.tkv_last_error()
        torch.cuda.synchronize()
        # the call took nothing from the device's free memory
        assert torch.cuda.mem_get_info()[0] >= free_before - (1 << 20), f"call {call}"
        assert torch.isfinite(got.float()).all(), f"call {call}"
        assert float((got.float() - want.float()).abs().max()) <= TOL, f"call {call}"
        assert _oracle_gap(got, q, k, v, ln, hkv, cap) <= TOL, f"call {call}"


def _oracle_gap(got, q, k, v, ln, hkv, cap, starts=None):
    """Largest absolute difference to orc.varlen_gqa_attention (fp32) over all segments."""
    bsz, hq, d = q.shape
    lens = ln.cpu().numpy()
    if starts is None:   # capacity-strided: pack the live rows as the oracle expects them
        mask = (torch.arange(cap, device=k.device)[None, :] < ln[:, None]).view(-1)
        k, v = k[mask], v[mask]
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    want = orc.varlen_gqa_attention(q.float().cpu().numpy()[:, :, None, :], k.float().cpu().numpy(), v.float().cpu().numpy(),
                                    cu, bsz, hkv)[:, 0]
    return float(np.abs(got.float().cpu().numpy() - want).max())


@pytest.mark.parametrize("dtype,d,tol", [(torch.bfloat16, 128, 2e-2), (torch.float16, 64, 5e-3)])
def test_static_scratch_entry_point_packed_layout_and_small_heads(dtype, d, tol):
    """The packed [sum n, D] layout with seg_start (the reference's flat caches) and head_dim 64 / f16."""
    from trimkv_b200 import _lib
    lib = _lib.lib()
    stream = torch.cuda.current_stream(torch.device(DEV)).cuda_stream
    gen = torch.Generator().manual_seed(7)
    bsz, hq, hkv, cap = 3, 8, 4, 900
    nseg = bsz * hkv
    lens = torch.randint(1, cap + 1, (nseg,), generator=gen).to(torch.int32)
    lens[1] = 0
    total = int(lens.sum())
    q = torch.randn(bsz, hq, d, generator=gen).to(dtype).to(DEV)
    k = torch.randn(total, d, generator=gen).to(dtype).to(DEV)
    v = torch.randn(total, d, generator=gen).to(dtype).to(DEV)
    cu = torch.zeros(nseg + 1, dtype=torch.int32)
    cu[1:] = lens.cumsum(0)
    ln, starts = lens.to(DEV), cu[:-1].contiguous().to(DEV)
    got = torch.full((bsz, hq, d), float("nan"), dtype=dtype, device=DEV)
    rc = lib.tkv_decode_attn_static(q.data_ptr(), q.stride(0), q.stride(1), k.data_ptr(), v.data_ptr(), ln.data_ptr(),
                                    starts.data_ptr(), 0, got.data_ptr(), bsz, hq, hkv, d,
                                    _lib.TKV_BF16 if dtype == torch.bfloat16 else _lib.TKV_F16, d ** -0.5, cap, None, stream)
    assert rc == 0, lib.tkv_last_error()
    torch.cuda.synchronize()
    assert torch.isfinite(got.float()).all()
    assert _oracle_gap(got, q, k, v, ln, hkv, cap, starts=starts) <= tol


def test_static_scratch_entry_point_refuses_oversized_problems():
    from trimkv_b200 import _lib, ops
    lib = _lib.lib()
    bsz, hq, hkv, d, cap = 256, 64, 8, 128, 8192
    # 2048 segments x 16 chunks of 512 tokens x 8 heads x 130 floats = 136 MB of partials
    assert ops.decode_attn_workspace_bytes(bsz, hq, hkv, d, cap) > (32 << 20)
    dummy = torch.zeros(64, dtype=torch.bfloat16, device=DEV)
    ln = torch.zeros(bsz * hkv, dtype=torch.int32, device=DEV)
    rc = lib.tkv_decode_attn_static(dummy.data_ptr(), hq * d, d, dummy.data_ptr(), dummy.data_ptr(), ln.data_ptr(),
                                    None, cap, dummy.data_ptr(), bsz, hq, hkv, d, _lib.TKV_BF16, 1.0, cap, None,
                                    torch.cuda.current_stream(torch.device(DEV)).cuda_stream)
    assert rc == -2
    assert b"built-in array" in lib.tkv_last_error()
