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

The model files (``models/{qwen3,llama,phi3}/modeling_trimkv_*.py``) import under the installed
transformers after two additions to transformers' own namespaces, made by ``import_reference_models``:
an empty ``transformers.cache_utils.SlidingWindowCache`` (imported, never used on this path) and the
plain ``ROPE_INIT_FUNCTIONS["default"]`` (inverse frequencies ``theta^(-2i/d)``, scale 1) that older
transformers registered.  Nothing of the reference is edited.
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


def import_reference_models():
    """The reference's three model families (call after ``import_reference``)."""
    import importlib
    import transformers.cache_utils as tcu
    from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS
    if not hasattr(tcu, "SlidingWindowCache"):
        tcu.SlidingWindowCache = type("SlidingWindowCache", (), {})
    if "default" not in ROPE_INIT_FUNCTIONS:
        def default_rope(config, device=None, seq_len=None, **kw):
            d = getattr(config, "head_dim", None) or config.hidden_size // config.num_attention_heads
            rp = getattr(config, "rope_parameters", None) or {}
            theta = rp.get("rope_theta", getattr(config, "rope_theta", 10000.0))
            d = int(d * rp.get("partial_rotary_factor", getattr(config, "partial_rotary_factor", 1.0)))
            return 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.int64).to(device=device, dtype=torch.float) / d)), 1.0
        ROPE_INIT_FUNCTIONS["default"] = default_rope
    for name in ("trimkv.models", "trimkv.models.qwen3", "trimkv.models.llama", "trimkv.models.phi3"):
        pkg = types.ModuleType(name)
        pkg.__path__ = [os.path.join(sys.modules["trimkv"].__path__[0], *name.split(".")[1:])]
        sys.modules[name] = pkg
    # the reference's own attention package (its __init__ holds the registry the models call)
    del sys.modules["trimkv.attn"]
    importlib.import_module("trimkv.attn")
    out = {}
    for fam, cfg_name, cls_name in (("qwen3", "TrimKVQwen3Config", "TrimKVQwen3ForCausalLM"),
                                    ("llama", "TrimKVLlamaConfig", "TrimKVLlamaForCausalLM"),
                                    ("phi3", "TrimKVPhi3Config", "TrimKVPhi3ForCausalLM")):
        mod = importlib.import_module(f"trimkv.models.{fam}.modeling_trimkv_{fam}")
        out[fam] = (getattr(mod, cfg_name), getattr(mod, cls_name))
    return out


def model_goldens(cu, models):
    """Prompt + teacher-forced greedy decode through the reference's own model classes and ``TrimKVCache`` on CPU.

    Per case (tiny_models.CASES: the three families with the ``rg`` gate, Qwen3 with ``rg2`` and ``rg3``): fp32 and
    bf16 runs on the same token ids (the fp32 run's own greedy choices); after every forward the logits of the last
    position, every layer's cache length and kept positions; plus the ids HF ``generate`` returns for the fp32 model
    with a fresh reference cache.  Weights and prompt come from tiny_models.py."""
    import tiny_models as tm
    import warnings
    warnings.filterwarnings("ignore")
    for case, (fam, extra, T) in tm.CASES.items():
        Cfg, Cls = models[fam]
        cfg = Cfg(**dict(tm.FAMILIES[fam], **extra), attn_implementation="sdpa", pad_token_id=0,
                  eos_token_id=None, bos_token_id=None)  # no end-of-sequence id: no row ever "finishes" under generate
        model = Cls(cfg).eval()
        shapes = {k: tuple(v.shape) for k, v in model.state_dict().items()}
        sd = {k: torch.from_numpy(v) for k, v in tm.fill_state_dict(shapes).items()}
        prompt = torch.from_numpy(tm.prompt_ids(fam, cfg.vocab_size))
        L, Hkv, cap = cfg.num_hidden_layers, cfg.num_key_value_heads, cfg.memory_size + cfg.buffer_size
        out = {"param_names": np.array(sorted(shapes)), "param_shapes": np.array([str(shapes[k]) for k in sorted(shapes)])}

        def fresh(dt):
            model.to(torch.float32).load_state_dict(sd, strict=True)       # .to() converts in place
            m = model.to(dt)
            # .to(bf16) also rounds the rotary inverse frequencies (a non-persistent buffer); a checkpoint loaded with
            # from_pretrained(torch_dtype=bfloat16) keeps them in fp32, so put the fp32 values back.
            m.model.rotary_emb.inv_freq = m.model.rotary_emb.original_inv_freq.clone().float()
            return m

        forced = None
        for tag, dt in (("fp32", torch.float32), ("bf16", torch.bfloat16)):
            m = fresh(dt)
            cache = cu.TrimKVCache(device="cpu")
            logits = np.zeros((T + 1, tm.BATCH, cfg.vocab_size), np.float32)
            lens = np.zeros((T + 1, L), np.int32)
            pos = np.full((T + 1, L, tm.BATCH, Hkv, cap), -1, np.int16)
            ids, chosen = prompt, []
            with torch.no_grad():
                for t in range(T + 1):
                    o = m(input_ids=ids, past_key_values=cache, logits_to_keep=1)
                    logits[t] = o.logits[:, -1].float().numpy()
                    for l in range(L):
                        n = cache.get_cache_length(l)
                        lens[t, l] = n
                        pos[t, l, :, :, :n] = cache.kv_positions[l].numpy()
                    nxt = o.logits[:, -1].argmax(-1, keepdim=True) if forced is None else forced[:, t:t + 1]
                    chosen.append(nxt)
                    ids = nxt
            if forced is None:
                forced = torch.cat(chosen, 1)          # [B, T+1]; the last one is never fed
            out[f"logits_{tag}"], out[f"lens_{tag}"], out[f"pos_{tag}"] = logits, lens, pos
        out["ids"] = torch.cat([prompt, forced[:, :T]], 1).numpy()
        m = fresh(torch.float32)
        with torch.no_grad():
            gen = m.generate(prompt, attention_mask=torch.ones_like(prompt), max_new_tokens=24, do_sample=False,
                             past_key_values=cu.TrimKVCache(device="cpu"))
        out["generate_ids"] = gen.numpy()
        assert np.array_equal(out["generate_ids"][:, tm.PROMPT_LEN:], forced[:, :24].numpy()), "generate != forward loop"
        np.savez_compressed(os.path.join(HERE, f"model_{case}.npz"), **out)
        d = np.abs(out["logits_fp32"] - out["logits_bf16"]).max()
        print(f"model_{case}: lens {out['lens_fp32'][0].tolist()} -> {out['lens_fp32'][-1].tolist()}, |logits| max "
              f"{np.abs(out['logits_fp32']).max():.2f}, fp32-bf16 max diff {d:.4f}, bf16 positions equal fp32: "
              f"{np.array_equal(out['pos_fp32'], out['pos_bf16'])}")


if __name__ == "__main__":
    sys.path.insert(0, HERE)
    cu_, ea_ = import_reference(sys.argv[1])
    if len(sys.argv) > 2 and sys.argv[2] == "models":      # only the model-level vectors
        model_goldens(cu_, import_reference_models())
        sys.exit(0)
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
    model_goldens(cu_, import_reference_models())
