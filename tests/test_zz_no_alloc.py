"""The allocation-free decode-attention entry point against the regular one.

`tkv_decode_attn_static` exists for hosts that cannot give the library a workspace (an arena that already owns
the device, a plug-in slot without an allocator, a loop that must not hit cudaMalloc's synchronisation): its
scratch is a fixed array inside the library.  Here it is called straight through the C ABI, twice in a row on
different inputs, and must reproduce `tkv_decode_attn` (same kernels, so the 2e-2 bf16 tolerance of the other
attention tests is met with room to spare); a problem larger than the built-in array must be refused cleanly.
This file sorts last on purpose so a run that stops at the first failure has already run everything else.
"""
import pytest
import torch

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


def test_static_scratch_entry_point_refuses_oversized_problems():
    from trimkv_b200 import _lib, ops
    lib = _lib.lib()
    bsz, hq, hkv, d, cap = 256, 64, 8, 128, 8192
    assert ops.decode_attn_workspace_bytes(bsz, hq, hkv, d, cap) > (32 << 20)
    dummy = torch.zeros(64, dtype=torch.bfloat16, device=DEV)
    ln = torch.zeros(bsz * hkv, dtype=torch.int32, device=DEV)
    rc = lib.tkv_decode_attn_static(dummy.data_ptr(), hq * d, d, dummy.data_ptr(), dummy.data_ptr(), ln.data_ptr(),
                                    None, cap, dummy.data_ptr(), bsz, hq, hkv, d, _lib.TKV_BF16, 1.0, cap, None,
                                    torch.cuda.current_stream(torch.device(DEV)).cuda_stream)
    assert rc == -2
    assert b"built-in array" in lib.tkv_last_error()
