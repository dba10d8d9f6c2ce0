"""Generate the golden vectors under tests/golden/ from the reference's own Python.

Run in a container that has the reference checkout (pass its ``src`` directory as
argv[1]); the GPU box does not have it, which is why the outputs are committed.

    python tests/golden/make_golden.py <reference>/src

The reference package cannot be imported whole under transformers 5.x (its model
files import a class that was removed), so an empty ``trimkv`` package whose
``__path__`` points at the checkout is registered first and only
``trimkv.cache_utils`` / ``trimkv.attn.eager_attn`` are imported.  The flat cache
classes call a CUDA-only Triton append; on CPU it is rebound to a per-head
concatenation with the same semantics (src/trimkv/triton/db_cache_utils.py:97-117).
"""
import os
import sys
import types

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))


def import_reference(src_dir):
    pkg = types.ModuleType("trimkv")
    pkg.__path__ = [os.path.join(src_dir, "trimkv")]
    sys.modules["trimkv"] = pkg
    import trimkv.cache_utils as cu
    attn_pkg = types.ModuleType("trimkv.attn")
    attn_pkg.__path__ = [os.path.join(src_dir, "trimkv", "attn")]
    sys.modules["trimkv.attn"] = attn_pkg
    import trimkv.attn.eager_attn as ea

    def cat_append(cache, state, headlens, cu_headlens):
        _, h_, s_, _ = state.shape
        parts = []
        for h in range(h_):
            a = int(cu_headlens[h]); n = int(headlens[h])
            parts += [cache[a:a + n], state[0, h]]
        return torch.cat(parts, 0)

    cu.update_flatten_view_triton = cat_append
    return cu, ea


def config1(cu):
    """Benchmark-spec configs[0]: batch 1, 8 KV heads, D 128, fp32, M 512, B 128, 4096 prefill + 256 steps."""
    torch.manual_seed(0)
    H, D, S, M, B, T = 8, 128, 4096, 512, 128, 256
    cache = cu.TrimKVCache(device="cpu")
    logb = F.logsigmoid(torch.randn(1, H, S + T) * 1.5 + 3.0)
    kept, lens, evict_steps = [], [], []

    def step(lo, hi, tag):
        n = hi - lo
        # K/V content does not influence selection; small deterministic rows keep this fast.
        k = torch.arange(lo, hi, dtype=torch.float32)[None, None, :, None].expand(1, H, n, D).contiguous()
        cache.update(k, k.clone(), logb[:, :, lo:hi].contiguous(), torch.arange(lo, hi), 0)
        before = cache.get_cache_length(0)
        cache.compress(memory_size=M, buffer_size=B)
        after = cache.get_cache_length(0)
        lens.append(after)
        if after != before:
            kept.append(cache.kv_positions[0][0].numpy().astype(np.int32).copy())
            evict_steps.append(tag)

    step(0, S, 0)
    for t in range(T):
        step(S + t, S + t + 1, t + 1)
    np.savez_compressed(
        os.path.join(HERE, "config1_lockstep.npz"),
        log_beta=logb[0].numpy(), kept_positions=np.stack(kept), lens=np.asarray(lens, np.int32),
        evict_steps=np.asarray(evict_steps, np.int32), M=M, B=B, S=S, T=T)
    print("config1: evictions at", evict_steps, "final len", lens[-1])


def ties_bf16(cu):
    """bf16-stored log beta makes equal scores common; pin the kept-score multiset and the lengths."""
    torch.manual_seed(1)
    Bt, H, D, S, M, B, T = 2, 4, 16, 700, 256, 64, 200
    cache = cu.TrimKVCache(device="cpu")
    logb = F.logsigmoid(torch.randn(Bt, H, S + T) * 1.5 + 3.0).to(torch.bfloat16)
    out_scores, out_pos_ref, steps = [], [], []
    for t in range(T + 1):
        lo, hi = (0, S) if t == 0 else (S + t - 1, S + t)
        n = hi - lo
        k = torch.zeros(Bt, H, n, D, dtype=torch.bfloat16)
        cache.update(k, k.clone(), logb[:, :, lo:hi].contiguous(), torch.arange(lo, hi), 0)
        before = cache.get_cache_length(0)
        q_idx = cache.get_seq_length(0) + 1
        cache.compress(memory_size=M, buffer_size=B)
        if cache.get_cache_length(0) != before:
            rw = cache.retention_weights[0].to(torch.float32)
            sc = rw * (q_idx - cache.kv_positions[0])
            out_scores.append(np.sort(sc.numpy().reshape(Bt * H, M), axis=-1))
            out_pos_ref.append(cache.kv_positions[0].numpy().reshape(Bt * H, M).astype(np.int32))
            steps.append(t)
    np.savez_compressed(
        os.path.join(HERE, "ties_bf16.npz"),
        log_beta_bits=logb.view(torch.int16).numpy(), kept_scores_sorted=np.stack(out_scores),
        kept_positions_reference=np.stack(out_pos_ref), evict_steps=np.asarray(steps, np.int32),
        M=M, B=B, S=S, T=T)
    print("ties_bf16: evictions at", steps)


def ties_single_shot(cu):
    """Independent evictions whose boundary falls inside a class of equal scores."""
    torch.manual_seed(4)
    R, n, M = 64, 300, 200
    vals = torch.tensor([-0.5, -0.25, -0.125, -0.0625])
    logb = vals[torch.randint(0, 4, (1, R, n))]
    cache = cu.TrimKVCache(device="cpu")
    k = torch.zeros(1, R, n, 2)
    cache.update(k, k.clone(), logb, torch.arange(n), 0)
    q_idx = cache.get_seq_length(0) + 1
    cache.compress(memory_size=M, buffer_size=n - M)
    pos = cache.kv_positions[0][0]
    sc = cache.retention_weights[0][0] * (q_idx - pos)
    np.savez_compressed(
        os.path.join(HERE, "ties_single_shot.npz"), log_beta=logb[0].numpy(),
        kept_positions_reference=pos.numpy().astype(np.int32),
        kept_scores_sorted=np.sort(sc.numpy(), axis=-1), M=M)
    print("ties_single_shot: ok")


def flat_layout(cu):
    """Flat varlen layout of BatchedDynamicBudgetTrimKVCache after a prefill and three appends."""
    torch.manual_seed(2)
    Bt, H, D, S = 2, 3, 8, 5
    cache = cu.BatchedDynamicBudgetTrimKVCache(device="cpu")
    k = torch.randn(Bt, H, S + 4, D)
    b = F.logsigmoid(torch.randn(Bt, H, S + 4))
    cache.update(k[:, :, :S], k[:, :, :S] * 2, b[:, :, :S], torch.arange(S), 0)
    for t in range(3):
        lo, hi = (S + t, S + t + 1) if t < 2 else (S + 2, S + 4)
        _, _, _, _, kw = cache.update(k[:, :, lo:hi], k[:, :, lo:hi] * 2, b[:, :, lo:hi], torch.arange(lo, hi), 0)
    np.savez_compressed(
        os.path.join(HERE, "flat_layout.npz"),
        k=k.numpy(), log_beta=b.numpy(), key_flat=cache.key_cache[0].numpy(),
        value_flat=cache.value_cache[0].numpy(), rw_flat=cache.retention_weights[0].numpy(),
        pos_flat=cache.kv_positions[0].numpy(), head_lens=kw["head_lens"].numpy(),
        cu_seqlens_k=kw["cu_seqlens_k"].numpy(), S=S)
    print("flat_layout: head_lens", kw["head_lens"].tolist())


def sliding_window(cu):
    """TrimKVCache with sliding_window_size: the newest rows are never evicted."""
    torch.manual_seed(6)
    Bt, H, D, S, M, B, T, W = 2, 3, 4, 50, 16, 4, 20, 6
    cache = cu.TrimKVCache(device="cpu")
    cache.sliding_window_size = W
    logb = F.logsigmoid(torch.randn(Bt, H, S + T) * 1.5 + 3.0)
    pos = []
    for t in range(T + 1):
        lo, hi = (0, S) if t == 0 else (S + t - 1, S + t)
        k = torch.zeros(Bt, H, hi - lo, D)
        cache.update(k, k.clone(), logb[:, :, lo:hi].contiguous(), torch.arange(lo, hi), 0)
        before = cache.get_cache_length(0)
        cache.compress(memory_size=M, buffer_size=B)
        if cache.get_cache_length(0) != before:
            pos.append(cache.kv_positions[0].numpy().astype(np.int32).copy())
    np.savez_compressed(os.path.join(HERE, "sliding_window.npz"), log_beta=logb.numpy(), kept_positions=np.stack(pos),
                        M=M, B=B, S=S, T=T, W=W)
    print("sliding_window: evictions", len(pos))


def knorm_alpha(cu):
    """TrimKVCache with strategy "knorm_alpha" on fp32 keys of widely varying norm."""
    torch.manual_seed(8)
    Bt, H, D, S, M, B, T = 2, 2, 32, 60, 20, 5, 15
    cache = cu.TrimKVCache(device="cpu")
    logb = F.logsigmoid(torch.randn(Bt, H, S + T) * 1.5 + 3.0)
    keys = torch.randn(Bt, H, S + T, D) * torch.exp(torch.randn(Bt, H, S + T, 1))
    pos = []
    for t in range(T + 1):
        lo, hi = (0, S) if t == 0 else (S + t - 1, S + t)
        cache.update(keys[:, :, lo:hi].contiguous(), keys[:, :, lo:hi].contiguous() * 0.5, logb[:, :, lo:hi].contiguous(),
                     torch.arange(lo, hi), 0)
        before = cache.get_cache_length(0)
        cache.compress(strategy="knorm_alpha", memory_size=M, buffer_size=B)
        if cache.get_cache_length(0) != before:
            pos.append(cache.kv_positions[0].numpy().astype(np.int32).copy())
    np.savez_compressed(os.path.join(HERE, "knorm_alpha.npz"), log_beta=logb.numpy(), keys=keys.numpy(),
                        kept_positions=np.stack(pos), M=M, B=B, S=S, T=T)
    print("knorm_alpha: evictions", len(pos))


def flat_budget(cu):
    """Budget-sharing compress of the two flat cache classes (fp32 tensors, so scores are fp32 as on the CUDA path)."""
    L, B, H, D, S, T, M, Bf = 2, 2, 3, 4, 40, 30, 8, 4
    out = {}
    cases = [("batched", "alpha", 0.0, 0.0), ("batched", "layer_wise_alpha", 0.0, 0.0),
             ("batched", "layer_wise_alpha", 0.25, 0.0), ("batched", "alpha_threshold", 0.0, 0.35),
             ("single", "alpha", 0.0, 0.0), ("single", "alpha", 0.25, 0.0), ("single", "layer_wise_alpha", 0.0, 0.0)]
    for ci, (kind, strategy, floor, thr) in enumerate(cases):
        torch.manual_seed(10 + ci)
        bsz = B if kind == "batched" else 1
        cls = cu.BatchedDynamicBudgetTrimKVCache if kind == "batched" else cu.DynamicBudgetTrimKVCache
        cache = cls(device="cpu")
        logb = F.logsigmoid(torch.randn(L, bsz, H, S + T) * 1.5 + 3.0)
        lens, poss = [], []
        for t in range(T + 1):
            lo, hi = (0, S) if t == 0 else (S + t - 1, S + t)
            for l in range(L):
                k = torch.arange(lo, hi, dtype=torch.float32)[None, None, :, None].expand(bsz, H, hi - lo, D) + 1000 * l
                cache.update(k.contiguous(), -k.contiguous(), logb[l, :, :, lo:hi].contiguous(), torch.arange(lo, hi), l)
            cache.compress(strategy=strategy, memory_size=M, buffer_size=Bf, floor_budget_ratio=floor,
                           alpha_threshold=thr, num_layers=L, num_key_value_heads=H)
            lens.append(torch.stack([cache.head_lens[l] for l in range(L)]).numpy().copy())
            poss.append([cache.kv_positions[l][:, 0].numpy().astype(np.int32).copy() for l in range(L)])
        out[f"c{ci}_logb"] = logb.numpy()
        out[f"c{ci}_lens"] = np.stack(lens)
        for t in (0, T // 2, T):
            for l in range(L):
                out[f"c{ci}_pos_t{t}_l{l}"] = poss[t][l]
    out["meta"] = np.asarray([L, B, H, D, S, T, M, Bf])
    out["cases"] = np.asarray([f"{k}|{s}|{f}|{a}" for k, s, f, a in cases])
    np.savez_compressed(os.path.join(HERE, "flat_budget.npz"), **out)
    print("flat_budget: ok")


def flat_budget_bf16(cu):
    """The flat classes on bf16 tensors: they score in bf16 (no upcast), which makes equal scores frequent.  One
    prefill + one compress per case; pinned are the per-group multisets of kept scores, the lengths and positions
    (exactly comparable where no tie straddles the group's budget)."""
    L, B, H, D, S, M, Bf = 2, 2, 3, 4, 300, 64, 16
    cases = [("batched", "alpha", 0.0), ("batched", "layer_wise_alpha", 0.0), ("single", "alpha", 0.0),
             ("single", "layer_wise_alpha", 0.0), ("batched", "alpha_threshold", 0.35)]
    out = {}
    for ci, (kind, strategy, thr) in enumerate(cases):
        torch.manual_seed(30 + ci)
        bsz = B if kind == "batched" else 1
        cls = cu.BatchedDynamicBudgetTrimKVCache if kind == "batched" else cu.DynamicBudgetTrimKVCache
        cache = cls(device="cpu")
        logb = F.logsigmoid(torch.randn(L, bsz, H, S) * 1.5 + 3.0).to(torch.bfloat16)
        for l in range(L):
            k = (torch.arange(S, dtype=torch.float32)[None, None, :, None].expand(bsz, H, S, D) + 1000 * l).to(torch.bfloat16)
            cache.update(k.contiguous(), -k.contiguous(), logb[l].contiguous(), torch.arange(S), l)
        q_idx = cache.get_seq_length() + 1
        cache.compress(strategy=strategy, memory_size=M, buffer_size=Bf, floor_budget_ratio=0.0, alpha_threshold=thr,
                       num_layers=L, num_key_value_heads=H)
        assert cache.retention_weights[0].dtype == torch.bfloat16
        lens = torch.stack([cache.head_lens[l] for l in range(L)]).numpy()
        # kept scores, recomputed the way the class does (bf16 product), per (layer, segment)
        for l in range(L):
            sc = ((q_idx - cache.kv_positions[l].squeeze(-1)) * cache.retention_weights[l].squeeze(-1)).float().numpy()
            out[f"c{ci}_scores_l{l}"] = sc
            out[f"c{ci}_pos_l{l}"] = cache.kv_positions[l][:, 0].numpy().astype(np.int32)
        out[f"c{ci}_logb_bits"] = logb.view(torch.int16).numpy()
        out[f"c{ci}_lens"] = lens
    out["meta"] = np.asarray([L, B, H, D, S, M, Bf])
    out["cases"] = np.asarray([f"{k}|{s}|{t}" for k, s, t in cases])
    np.savez_compressed(os.path.join(HERE, "flat_budget_bf16.npz"), **out)
    print("flat_budget_bf16: lens", [out[f"c{ci}_lens"].tolist() for ci in range(len(cases))])


def flat_budget_knorm(cu):
    """"knorm_alpha" strategies of the flat classes (score = log_alpha + log ||k||, in the tensors' dtype), on fp32
    and on bf16 tensors.  One prefill + one compress per case."""
    L, B, H, D, S, M, Bf = 2, 2, 3, 8, 128, 32, 8
    cases = []
    for dt in ("float32", "bfloat16"):
        cases += [("batched", "knorm_alpha", 0.0, dt), ("batched", "layer_wise_knorm_alpha", 0.0, dt),
                  ("single", "knorm_alpha", 0.0, dt), ("single", "layer_wise_knorm_alpha", 0.0, dt),
                  ("single", "knorm_alpha_threshold", 0.35, dt), ("batched", "knorm_alpha_threshold", 0.35, dt)]
    out = {}
    for ci, (kind, strategy, thr, dt) in enumerate(cases):
        torch.manual_seed(50 + ci)
        tdt = getattr(torch, dt)
        bsz = B if kind == "batched" else 1
        cls = cu.BatchedDynamicBudgetTrimKVCache if kind == "batched" else cu.DynamicBudgetTrimKVCache
        cache = cls(device="cpu")
        logb = F.logsigmoid(torch.randn(L, bsz, H, S) * 1.5 + 3.0).to(tdt)
        keys = (torch.randn(L, bsz, H, S, D) * torch.exp(torch.randn(L, bsz, H, S, 1))).to(tdt)
        for l in range(L):
            cache.update(keys[l].contiguous(), (keys[l] * 0.5).contiguous(), logb[l].contiguous(), torch.arange(S), l)
        q_idx = cache.get_seq_length() + 1
        cache.compress(strategy=strategy, memory_size=M, buffer_size=Bf, floor_budget_ratio=0.0, alpha_threshold=thr,
                       num_layers=L, num_key_value_heads=H)
        for l in range(L):
            la = (q_idx - cache.kv_positions[l].squeeze(-1)) * cache.retention_weights[l].squeeze(-1)
            sc = la + torch.log(cache.key_cache[l].norm(dim=-1).reshape(-1).clamp_min(1e-12))
            assert sc.dtype == tdt
            out[f"c{ci}_scores_l{l}"] = sc.float().numpy()
            out[f"c{ci}_pos_l{l}"] = cache.kv_positions[l][:, 0].numpy().astype(np.int32)
        if dt == "bfloat16":   # exact and half the size: the bit patterns
            out[f"c{ci}_logb"] = logb.view(torch.int16).numpy()
            out[f"c{ci}_keys"] = keys.view(torch.int16).numpy()
        else:
            out[f"c{ci}_logb"] = logb.numpy()
            out[f"c{ci}_keys"] = keys.numpy()
        out[f"c{ci}_lens"] = torch.stack([cache.head_lens[l] for l in range(L)]).numpy()
    out["meta"] = np.asarray([L, B, H, D, S, M, Bf])
    out["cases"] = np.asarray([f"{k}|{s}|{t}|{d}" for k, s, t, d in cases])
    np.savez_compressed(os.path.join(HERE, "flat_budget_knorm.npz"), **out)
    print("flat_budget_knorm: lens", [out[f"c{ci}_lens"].sum() for ci in range(len(cases))])


def eager_attention(ea):
    """Dense GQA attention from the reference's eager function (fp32), Q=1 and Q=3."""
    torch.manual_seed(3)
    Bt, Hq, Hkv, D, n = 2, 8, 2, 128, 37
    out = {}
    for ql in (1, 3):
        q = torch.randn(Bt, Hq, ql, D); k = torch.randn(Bt, Hkv, n, D); v = torch.randn(Bt, Hkv, n, D)
        mask = torch.full((ql, n), float("-inf")).triu(n - ql + 1)[None, None]
        mod = types.SimpleNamespace(num_key_value_groups=Hq // Hkv, training=False)
        o, _, _ = ea.eager_attention_forward(mod, q, k, v, mask, scaling=D ** -0.5)
        out[f"q{ql}"] = q.numpy(); out[f"k{ql}"] = k.numpy(); out[f"v{ql}"] = v.numpy(); out[f"o{ql}"] = o.numpy()
    np.savez_compressed(os.path.join(HERE, "eager_attention.npz"), **out)
    print("eager_attention: ok")


if __name__ == "__main__":
    cu_, ea_ = import_reference(sys.argv[1])
    config1(cu_)
    ties_bf16(cu_)
    ties_single_shot(cu_)
    flat_layout(cu_)
    sliding_window(cu_)
    knorm_alpha(cu_)
    flat_budget(cu_)
    flat_budget_bf16(cu_)
    flat_budget_knorm(cu_)
    eager_attention(ea_)
