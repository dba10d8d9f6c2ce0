"""CPU stand-ins for the native calls `TrimKVCache` makes, for testing the HOST logic of the cache class without a GPU.

TEST INFRASTRUCTURE ONLY: the product has no CPU path (`TrimKVCache` refuses CPU tensors, the library is CUDA only).
Each function below follows the contract its entry point states in include/trimkv_b200.h, on CPU tensors, with the
selection taken from the oracle (`canonical_topm`: larger score first, ties to the lower index).  What they let a CPU
test exercise is everything the Python class decides by itself: capacity and slab sizing, the prompt hand-off (deferred
and per layer), counters, the compress trigger, which launch form it picks, views, batch splitting.  The kernels
themselves are compared with the oracle on a GPU (tests/test_kernels_gpu.py).
"""
import numpy as np
import torch

from oracle import trimkv_oracle as orc

launch_count = 0
_lib = __import__("trimkv_b200._lib", fromlist=["_lib"])   # TrimKVNativeError for the class's own raises


class DeviceTensor(torch.Tensor):
    """A CPU tensor that says it lives on a CUDA device, for the one check `update` makes on its input."""

    @property
    def is_cuda(self):
        return True


def on_device(t: torch.Tensor) -> torch.Tensor:
    return t.as_subclass(DeviceTensor)


def new_status(device):
    return torch.zeros(1, dtype=torch.int32)


def read_status(status):
    code = int(status.item())
    status.zero_()
    return code


def _report(status, code):
    if status is not None:
        status[0] = max(int(status[0]), code)


def append(k_cache, v_cache, beta_cache, pos_cache, seg_len, cu_seqlens, k_new, v_new, beta_new, pos_new, cap, status=None):
    b, h, s, d = k_new.shape
    if pos_new.dim() == 1:
        pos_new = pos_new[None, None, :].expand(b, h, s)
    for seg in range(b * h):
        n = int(seg_len[seg])
        if n + s > cap:
            _report(status, 1)
            continue
        lo = seg * cap + n
        k_cache[lo:lo + s] = k_new[seg // h, seg % h]
        v_cache[lo:lo + s] = v_new[seg // h, seg % h]
        beta_cache[lo:lo + s] = beta_new[seg // h, seg % h].to(torch.float32)
        pos_cache[lo:lo + s] = pos_new[seg // h, seg % h].to(torch.int32)
        seg_len[seg] = n + s
    if cu_seqlens is not None:
        cu_seqlens += torch.arange(cu_seqlens.numel(), dtype=torch.int32) * s


def _select(beta_row, pos_row, q_idx, m, protect_last=0):
    sc = orc.retention_scores(beta_row.numpy(), pos_row.numpy(), q_idx)
    if protect_last:
        sc[len(sc) - protect_last:] = np.inf
    return torch.from_numpy(orc.canonical_topm(sc, m))


def evict_select(beta, pos, seg_len, n_uniform, nseg, q_idx, memory_size, trigger_len, max_len, kept_idx, kept_cnt, status=None):
    for seg in range(nseg):
        n = int(seg_len[seg]) if seg_len is not None else n_uniform
        if n >= trigger_len and n > memory_size:
            p = pos if pos.dim() == 1 else pos[seg]
            kept_idx[seg] = _select(beta[seg, :n], p[:n], q_idx, memory_size).to(torch.int32)
            kept_cnt[seg] = memory_size
        else:
            kept_cnt[seg] = n


def _rebuild_cu(seg_len, cu_seqlens, group):
    if cu_seqlens is None:
        return
    lens = seg_len.view(-1, group).to(torch.int64)
    cu = cu_seqlens.view(-1, group + 1)
    cu[:, 0] = 0
    cu[:, 1:] = lens.cumsum(1).to(torch.int32)


def compact(k_dst, v_dst, beta_dst, pos_dst, cap, k_src, v_src, beta_src, pos_src, kept_idx, kept_cnt, seg_len, cu_seqlens,
            group, status=None):
    b, h, n, d = k_src.shape
    for seg in range(b * h):
        cnt = int(kept_cnt[seg]) if kept_cnt is not None else n
        if cnt > cap:
            _report(status, 1)
            continue
        idx = torch.arange(cnt) if (kept_idx is None or cnt == n) else kept_idx[seg, :cnt].long()
        lo = seg * cap
        k_dst[lo:lo + cnt] = k_src[seg // h, seg % h][idx]
        v_dst[lo:lo + cnt] = v_src[seg // h, seg % h][idx]
        beta_dst[lo:lo + cnt] = beta_src[seg][idx]
        p = pos_src if pos_src.dim() == 1 else pos_src[seg]
        pos_dst[lo:lo + cnt] = p[idx]
        seg_len[seg] = cnt
    _rebuild_cu(seg_len, cu_seqlens, group)


def evict_ex(k_cache, v_cache, beta_cache, pos_cache, seg_len, cu_seqlens, group, nseg, cap, q_idx, max_len, keep_cnt,
             protect_last=0, memory_size=1, trigger_len=0, kept_idx_out=None, kept_stride=0, status=None, knorm=False,
             score_dtype=0, scores=None):
    assert not knorm and score_dtype == 0 and scores is None, "the emulation covers strategy 'alpha' in fp32"
    k2, v2 = k_cache.view(-1, k_cache.shape[-1]), v_cache.view(-1, v_cache.shape[-1])
    b1, p1, ln = beta_cache.view(-1), pos_cache.view(-1), seg_len.view(-1)
    keep_cnt = keep_cnt.view(-1) if keep_cnt is not None else None
    for seg in range(nseg):
        n = int(ln[seg])
        if n > max_len:
            _report(status, 2)
            continue
        m = int(keep_cnt[seg]) if keep_cnt is not None else memory_size
        if keep_cnt is None and n < trigger_len:
            continue
        if m >= n:
            continue
        lo = seg * cap
        idx = _select(b1[lo:lo + n], p1[lo:lo + n], q_idx, m, protect_last)
        for t in (k2, v2, b1, p1):
            t[lo:lo + m] = t[lo:lo + n][idx].clone()
        ln[seg] = m
        if kept_idx_out is not None:
            kept_idx_out.view(nseg, -1)[seg, :m] = idx.to(torch.int32)
    if cu_seqlens is not None:
        _rebuild_cu(ln, cu_seqlens.view(-1), group)


def evict(k_cache, v_cache, beta_cache, pos_cache, seg_len, cu_seqlens, group, nseg, cap, q_idx, memory_size, trigger_len,
          max_len, kept_idx_out=None, status=None):
    evict_ex(k_cache, v_cache, beta_cache, pos_cache, seg_len, cu_seqlens, group, nseg, cap, q_idx, max_len, None, 0,
             memory_size, trigger_len, kept_idx_out, 0, status)


def evict_multi_workspace(nseg, memory_size, ctas_per_segment, device):
    return torch.zeros(1, dtype=torch.uint8)


multi_calls = []   # (nseg, ctas) of every several-CTAs-per-segment launch the class chose


def evict_multi(k_cache, v_cache, beta_cache, pos_cache, seg_len, cu_seqlens, group, nseg, cap, q_idx, memory_size,
                trigger_len, max_len, ctas, workspace, protect_last=0, knorm=False, kept_idx_out=None, status=None):
    multi_calls.append((nseg, ctas))
    evict_ex(k_cache, v_cache, beta_cache, pos_cache, seg_len, cu_seqlens, group, nseg, cap, q_idx, max_len, None,
             protect_last, memory_size, trigger_len, kept_idx_out, 0, status, knorm)


def group_budget(beta_cache, pos_cache, seg_len, cap, groups, inner, n_outer, outer_stride, q_idx, k_total, keep_cnt,
                 threshold=None, floor_mode=0, floor_cnt=0, status=None, score_dtype=0, scores=None):
    """Keep counts under a shared budget (fp32 scores; the contract of tkv_group_budget), from the oracle's
    concatenated top-k: group g = segments {g*inner + o*outer_stride + i}, o outer, i inner."""
    assert score_dtype == 0 and scores is None, "the emulation covers fp32 scores without key norms"
    beta, pos, ln, keep = beta_cache.reshape(-1), pos_cache.reshape(-1), seg_len.reshape(-1), keep_cnt.view(-1)
    for g in range(groups):
        segs = [g * inner + o * outer_stride + i for o in range(n_outer) for i in range(inner)]
        sc = []
        for s in segs:
            n = int(ln[s])
            sc.append(orc.retention_scores(beta[s * cap:s * cap + n].numpy(), pos[s * cap:s * cap + n].numpy(), q_idx))
        counts = orc._group_keep_counts(sc, k_total=k_total, threshold=threshold, bucketize_attribution=(floor_mode == 1))
        for s, c, x in zip(segs, counts, sc):
            if floor_mode == 1:
                c = min(len(x), c + floor_cnt)
            elif floor_mode == 2:
                c = max(c, min(floor_cnt, len(x)))
            keep[s] = c
