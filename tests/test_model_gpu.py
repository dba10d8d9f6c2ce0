"""Model-level parity on a B200: the callers (Qwen3, Llama, Phi-3) + cache + kernels against golden vectors made by
the reference's own model classes (tests/golden/model_*.npz) and against the eager CPU restatement."""
import os
import sys
import warnings

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import tiny_models as tm  # noqa: E402

warnings.filterwarnings("ignore")


def _golden_model(case, dtype, attn):
    import trimkv_b200 as t
    fam, extra, steps = tm.CASES[case]
    Cfg, Cls = {"qwen3": (t.TrimKVQwen3Config, t.TrimKVQwen3ForCausalLM), "llama": (t.TrimKVLlamaConfig, t.TrimKVLlamaForCausalLM),
                "phi3": (t.TrimKVPhi3Config, t.TrimKVPhi3ForCausalLM)}[fam]
    cfg = Cfg(**dict(tm.FAMILIES[fam], **extra), attn_implementation=attn, pad_token_id=0, eos_token_id=None, bos_token_id=None)
    model = Cls(cfg).eval()
    shapes = {k: tuple(v.shape) for k, v in model.state_dict().items()}
    model.load_state_dict({k: torch.from_numpy(v) for k, v in tm.fill_state_dict(shapes).items()}, strict=True)
    return model.to(dtype).to(DEV), cfg, np.load(os.path.join(HERE, "golden", f"model_{case}.npz")), steps


def _feed(g, step):
    ids, P = torch.from_numpy(g["ids"]), tm.PROMPT_LEN
    return (ids[:, :P] if step == 0 else ids[:, P + step - 1: P + step]).to(DEV)


def _check_cache(cache, cfg, g, tag, step, exact):
    """Lengths must equal the reference's; returns the number of (layer, request, head) rows whose kept positions
    differ (asserted zero when ``exact``)."""
    bad = 0
    for l in range(cfg.num_hidden_layers):
        n = cache.get_cache_length(l)
        assert n == g[f"lens_{tag}"][step, l], (step, l)
        mine = cache.kv_positions[l][:, :, :n].cpu().numpy()
        diff = (mine != g[f"pos_{tag}"][step, l, :, :, :n]).any(-1)
        if exact:
            assert not diff.any(), (step, l)
        bad += int(diff.sum())
    return bad


@pytest.mark.parametrize("case", sorted(tm.CASES))
def test_cache_kernels_under_reference_model_fp32_exact(case):
    """fp32 weights, fp32 K/V through the CUDA append and eviction kernels, dense library attention (the decode
    attention kernels are 16-bit): kept positions and lengths equal the reference model's at every step, logits to
    2e-4.  Pins the caller order and the cache kernels on the GPU against the reference itself."""
    from trimkv_b200 import TrimKVCache
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    model, cfg, g, steps = _golden_model(case, torch.float32, "sdpa")
    cache = TrimKVCache(device=DEV)
    worst = 0.0
    with torch.inference_mode():
        for step in range(steps + 1):
            out = model(input_ids=_feed(g, step), past_key_values=cache, logits_to_keep=1)
            worst = max(worst, float((out.logits[:, -1].cpu() - torch.from_numpy(g["logits_fp32"][step])).abs().max()))
            _check_cache(cache, cfg, g, "fp32", step, exact=True)
    cache.check_status()
    assert worst <= 2e-4, worst


@pytest.mark.parametrize("case", sorted(tm.CASES))
def test_cuda_path_matches_reference_model_bf16(case):
    """bf16 end to end through update / decode attention / compress: logits within 2e-2 of the reference model's bf16
    run on CPU, lengths identical at every step.  Kept positions may differ where bf16 GEMM rounding (cuBLAS vs the
    CPU) moves a log beta across a near-tie; the count of such rows is bounded."""
    from trimkv_b200 import TrimKVCache
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    model, cfg, g, steps = _golden_model(case, torch.bfloat16, "tkv_b200")
    cache = TrimKVCache(device=DEV)
    worst, bad, rows = 0.0, 0, 0
    with torch.inference_mode():
        for step in range(steps + 1):
            out = model(input_ids=_feed(g, step), past_key_values=cache, logits_to_keep=1)
            worst = max(worst, float((out.logits[:, -1].float().cpu() - torch.from_numpy(g["logits_bf16"][step])).abs().max()))
            bad += _check_cache(cache, cfg, g, "bf16", step, exact=False)
            rows += cfg.num_hidden_layers * tm.BATCH * cfg.num_key_value_heads
    cache.check_status()
    assert worst <= 2e-2, worst
    assert bad <= rows // 4, (bad, rows)


@pytest.mark.parametrize("case,use_graph", [("qwen3", False), ("qwen3", True), ("llama", True), ("phi3", True)])
def test_fused_decode_step_matches_reference_model_bf16(case, use_graph):
    """The fused CUDA decode step (add+RMSNorm, decode_prep, attention, SiLU*up; captured in a CUDA graph) fed the
    reference run's tokens: same bounds as the module path."""
    from trimkv_b200 import TrimKVCache
    from trimkv_b200.decoder import GreedyDecoder
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    model, cfg, g, steps = _golden_model(case, torch.bfloat16, "tkv_b200")
    cache = model.new_cache(DEV)
    worst, bad, rows = 0.0, 0, 0
    with torch.inference_mode():
        out = model(input_ids=_feed(g, 0), past_key_values=cache, logits_to_keep=1)
        worst = float((out.logits[:, -1].float().cpu() - torch.from_numpy(g["logits_bf16"][0])).abs().max())
        dec = GreedyDecoder(model, cache, use_graph=use_graph, fused=True)
        assert dec.fused is not None
        for step in range(1, steps + 1):
            dec.step(_feed(g, step), eager=(step < 3))
            worst = max(worst, float((dec.logits.float().cpu() - torch.from_numpy(g["logits_bf16"][step])).abs().max()))
            bad += _check_cache(cache, cfg, g, "bf16", step, exact=False)
            rows += cfg.num_hidden_layers * tm.BATCH * cfg.num_key_value_heads
    cache.check_status()
    assert worst <= 2e-2, worst
    assert bad <= rows // 4, (bad, rows)


@pytest.mark.parametrize("case", ["qwen3", "phi3"])
def test_hf_generate_with_the_cuda_cache(case):
    """``GenerationMixin.generate`` driving ``trimkv_b200.TrimKVCache`` on the GPU, as examples/test_qwen3.py:51-55
    drives the reference's cache: fp32 so that the greedy tokens are the reference's own."""
    from trimkv_b200 import TrimKVCache
    torch.backends.cuda.matmul.allow_tf32 = False
    model, cfg, g, _ = _golden_model(case, torch.float32, "sdpa")
    prompt = torch.from_numpy(g["ids"][:, :tm.PROMPT_LEN]).to(DEV)
    out = model.generate(prompt, attention_mask=torch.ones_like(prompt), max_new_tokens=24, do_sample=False,
                         past_key_values=TrimKVCache(device=DEV))
    assert np.array_equal(out.cpu().numpy(), g["generate_ids"])
    # and in bf16 through the decode-attention kernels: runs, right shape, cache bounded by M + B
    model, cfg, g, _ = _golden_model(case, torch.bfloat16, "tkv_b200")
    cache = TrimKVCache(device=DEV)
    out = model.generate(prompt, attention_mask=torch.ones_like(prompt), max_new_tokens=40, do_sample=False,
                         past_key_values=cache)
    assert out.shape == (tm.BATCH, tm.PROMPT_LEN + 40)
    assert cache.get_cache_length(0) < cfg.memory_size + cfg.buffer_size
    cache.check_status()


def _tiny(memory_size=96, buffer_size=16, layers=2):
    from trimkv_b200 import TrimKVQwen3Config, TrimKVQwen3ForCausalLM
    cfg = TrimKVQwen3Config(
        vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=layers, num_attention_heads=4,
        num_key_value_heads=2, head_dim=128, retention_gate_intermediate_size=32, retention_gate_bias_init=3.0,
        memory_size=memory_size, buffer_size=buffer_size, initializer_range=0.02)
    torch.manual_seed(0)
    model = TrimKVQwen3ForCausalLM(cfg).to(torch.bfloat16).eval()
    return model, cfg


def test_generate_matches_cpu_restatement():
    """Greedy decode through update/attention/compress: logits within 2e-2 of the eager CPU path (bf16),
    cache lengths identical at every step, kept positions identical unless scores tie within bf16 noise."""
    from oracle.qwen3_oracle import EagerTrimKVCache, OracleQwen3
    from trimkv_b200 import TrimKVCache
    # cuBLAS may reduce bf16 GEMM partials in bf16 by default; that noise is not what this test is about.
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    model, cfg = _tiny(layers=2)
    ref = OracleQwen3(model.state_dict(), cfg, dtype=torch.bfloat16)
    model = model.to(DEV)
    gen = torch.Generator().manual_seed(5)
    ids = torch.randint(0, cfg.vocab_size, (2, 150), generator=gen)
    cache, rcache = TrimKVCache(device=DEV), EagerTrimKVCache(canonical=True)
    worst, mismatched_rows = 0.0, 0
    with torch.inference_mode():
        for t in range(40):
            out = model(input_ids=ids.to(DEV), past_key_values=cache, logits_to_keep=1)
            want = ref.forward(ids, rcache)
            got = out.logits.float().cpu()
            worst = max(worst, float((got - want.float()).abs().max()))
            assert cache.get_seq_length() == rcache.get_seq_length()
            diverged = False
            for l in range(cfg.num_hidden_layers):
                assert cache.get_cache_length(l) == rcache.get_cache_length(l)
                mine = cache.kv_positions[l].cpu().to(torch.int64)
                rows = int((mine != rcache.kv_positions[l]).any(-1).sum())
                mismatched_rows += rows
                diverged |= rows > 0
            if diverged:
                # log beta comes out of bf16 GEMMs that round differently on CPU and GPU, so a near-tie at the
                # eviction boundary can fall either way; adopt the GPU state and keep comparing in lock-step.
                for l in range(cfg.num_hidden_layers):
                    rcache.key_cache[l] = cache.key_cache[l].cpu().clone()
                    rcache.value_cache[l] = cache.value_cache[l].cpu().clone()
                    rcache.retention_weights[l] = cache.retention_weights[l].cpu().to(torch.bfloat16)
                    rcache.kv_positions[l] = cache.kv_positions[l].cpu().to(torch.int64)
            ids = want.argmax(-1)  # feed both with the same token so the comparison stays in lock-step
    cache.check_status()
    assert worst <= 2e-2, worst
    assert mismatched_rows <= 6, mismatched_rows  # of 40 steps x 2 layers x 4 segments


@pytest.mark.parametrize("use_graph,tc_gemm,fused_down", [(False, False, False), (True, False, False), (True, True, False),
                                                         (True, False, True)])
def test_fused_decode_step_matches_module_path(use_graph, tc_gemm, fused_down):
    """The fused kernels (add+RMSNorm, decode_prep, SiLU*up; optionally the tensor-core GEMMs, or SiLU*up inside the
    down projection) against the PyTorch-op layer on the same weights."""
    from trimkv_b200 import TrimKVCache
    from trimkv_b200.decoder import GreedyDecoder
    model, cfg = _tiny(memory_size=64, buffer_size=8, layers=3)
    model = model.to(DEV)
    gen = torch.Generator().manual_seed(9)
    prompt = torch.randint(0, cfg.vocab_size, (3, 100), generator=gen).to(DEV)
    outs = []
    with torch.inference_mode():
        for fused in (False, True):
            cache = TrimKVCache(device=DEV, memory_size=cfg.memory_size, buffer_size=cfg.buffer_size)
            out = model(input_ids=prompt, past_key_values=cache, logits_to_keep=1)
            dec = GreedyDecoder(model, cache, use_graph=use_graph and fused, fused=fused, tc_gemm=tc_gemm, fused_down=fused_down)
            dec.ids.copy_(out.logits[:, -1].argmax(-1, keepdim=True))
            toks, logits = [], []
            forced = torch.randint(0, cfg.vocab_size, (30, 3, 1), generator=torch.Generator().manual_seed(1)).to(DEV)
            for t in range(30):
                if dec.use_graph and dec.graph is None and t == 2:
                    pass
                dec.step(forced[t], eager=(t < 2))  # same input tokens for both paths
                logits.append(dec.logits.float().clone())
                toks.append(dec.next_ids.clone())
            cache.check_status()
            n = cache.get_cache_length(0)  # a graph-captured decoder exposes full-capacity views: cut to the live rows
            outs.append((torch.stack(logits), cache.kv_positions[0][:, :, :n].clone(),
                         cache.key_cache[0][:, :, :n].float().clone(), cache.retention_weights[0][:, :, :n].clone(), n))
    (l0, p0, k0, b0, n0), (l1, p1, k1, b1, n1) = outs
    assert n0 == n1
    assert float((l0 - l1).abs().max()) <= 2e-2
    assert torch.equal(p0, p1)
    assert float((k0 - k1).abs().max()) <= 2e-2
    assert float((b0 - b1).abs().max()) <= 1e-2


def _module_path_rates_choices(model, cfg, prompt, ids, new_tokens):
    """The module path, fed the tokens another path chose greedily, must rate each of them within twice the paths'
    logit tolerance of its own best token."""
    from trimkv_b200 import TrimKVCache
    from trimkv_b200.decoder import GreedyDecoder
    plen = prompt.shape[1]
    with torch.inference_mode():
        ref_cache = TrimKVCache(device=DEV, memory_size=cfg.memory_size, buffer_size=cfg.buffer_size)
        logits = model(input_ids=prompt, past_key_values=ref_cache, logits_to_keep=1).logits[:, -1].float()
        dec = GreedyDecoder(model, ref_cache, use_graph=False, fused=False)
        for t in range(new_tokens):
            chosen = ids[:, plen + t: plen + t + 1]
            gap = logits.max(-1, keepdim=True).values - logits.gather(-1, chosen)
            assert float(gap.max()) <= 4e-2, (t, float(gap.max()))
            if t + 1 < new_tokens:
                dec.step(chosen, eager=True)
                logits = dec.logits.float()


def test_hf_generate_through_the_fused_step():
    """``config.fused_decode_step = True``: HF ``generate`` (greedy, then sampling) whose one-token forward passes run
    as the fused CUDA step; without the flag the module path runs and no fused step is built."""
    from trimkv_b200 import TrimKVCache
    model, cfg = _tiny(memory_size=64, buffer_size=8, layers=3)
    model = model.to(DEV)
    new_tokens, plen = 40, 100
    prompt = torch.randint(0, cfg.vocab_size, (3, plen), generator=torch.Generator().manual_seed(6)).to(DEV)
    mask = torch.ones_like(prompt)
    kw = dict(attention_mask=mask, max_new_tokens=new_tokens, pad_token_id=0)
    model.generation_config.eos_token_id = model.config.eos_token_id = None      # no early stop
    plain = TrimKVCache(device=DEV)
    model.generate(prompt, do_sample=False, past_key_values=plain, **kw)
    assert "_fused_step" not in plain.__dict__
    model.config.fused_decode_step = True
    cache = TrimKVCache(device=DEV)
    ids = model.generate(prompt, do_sample=False, past_key_values=cache, **kw)
    assert "_fused_step" in cache.__dict__
    assert ids.shape == (3, plen + new_tokens) and torch.equal(ids[:, :plen], prompt)
    assert cache.get_seq_length() == plen + new_tokens - 1
    assert cache.get_cache_length(0) < cfg.memory_size + cfg.buffer_size
    cache.check_status()
    _module_path_rates_choices(model, cfg, prompt, ids, new_tokens)
    assert model.config.fused_decode_step is True                  # the module-path decoder put the flag back
    torch.manual_seed(0)
    cache = TrimKVCache(device=DEV)
    sampled = model.generate(prompt, do_sample=True, temperature=0.8, top_k=20, past_key_values=cache, **kw)
    assert sampled.shape == (3, plen + new_tokens) and int(sampled.max()) < cfg.vocab_size
    cache.check_status()
    # launched from Python instead of replayed from a graph
    model.config.fused_decode_step = "eager"
    short = model.generate(prompt, do_sample=False, past_key_values=TrimKVCache(device=DEV),
                           **dict(kw, max_new_tokens=8))
    _module_path_rates_choices(model, cfg, prompt, short, 8)
    model.config.fused_decode_step = True
    # without eviction the slabs grow: the step that would exceed the capacity runs plainly and the graph is recorded again
    model.config.compress_memory = False
    grown = TrimKVCache(device=DEV)
    long = model.generate(prompt, do_sample=False, past_key_values=grown, **dict(kw, max_new_tokens=30))
    assert grown.get_cache_length(0) == plen + 29
    grown.check_status()
    _module_path_rates_choices(model, cfg, prompt, long, 30)
    model.config.compress_memory = True
    # a forward pass the fused step does not cover takes the module path
    out = model(input_ids=ids[:, -1:], past_key_values=cache, output_hidden_states=True)
    assert out.logits.shape == (3, 1, cfg.vocab_size)
    with torch.no_grad():
        assert model._fused_step_for(ids[:, -1:], cache, None, {}) is not None
        assert model._fused_step_for(ids[:, -2:], cache, None, {}) is None              # two tokens
    with torch.enable_grad():
        assert model._fused_step_for(ids[:, -1:], cache, None, {}) is None              # autograd would record nothing
    # a cache that carries a fused step is still freed by its last reference (no cycle for the collector to find)
    import gc
    import weakref
    gc.collect()
    gc.disable()
    try:
        with torch.inference_mode():
            c = TrimKVCache(device=DEV)
            model(input_ids=prompt, past_key_values=c, logits_to_keep=1)
            model(input_ids=prompt[:, :1], past_key_values=c)
        assert "_fused_step" in c.__dict__
        alive = weakref.ref(c)
        del c
        assert alive() is None
    finally:
        gc.enable()


def test_generate_with_fused_decode():
    """``generate(..., fused_decode=True)``: greedy decoding through the fused, graph-replayed step.  The module path,
    fed the tokens it chose, must rate each of them within twice the paths' logit tolerance of its own best token; a
    second call reuses the fused weights."""
    from trimkv_b200 import TrimKVCache
    from trimkv_b200.decoder import GreedyDecoder
    model, cfg = _tiny(memory_size=64, buffer_size=8, layers=3)
    model = model.to(DEV)
    new_tokens, plen = 40, 100
    prompt = torch.randint(0, cfg.vocab_size, (3, plen), generator=torch.Generator().manual_seed(4)).to(DEV)
    cache = TrimKVCache(device=DEV, memory_size=cfg.memory_size, buffer_size=cfg.buffer_size)
    ids = model.generate(prompt, max_new_tokens=new_tokens, fused_decode=True, past_key_values=cache)
    assert ids.shape == (3, plen + new_tokens) and torch.equal(ids[:, :plen], prompt)
    assert cache.get_seq_length() == plen + new_tokens - 1
    assert cache.get_cache_length(0) < cfg.memory_size + cfg.buffer_size
    cache.check_status()
    _module_path_rates_choices(model, cfg, prompt, ids, new_tokens)
    fused = {k: v[0].data_ptr() for k, v in model._tkv_fused_weights.items()}
    again = model.generate(prompt, max_new_tokens=new_tokens, fused_decode=True,
                           past_key_values=TrimKVCache(device=DEV, memory_size=cfg.memory_size, buffer_size=cfg.buffer_size))
    assert torch.equal(again, ids)
    assert fused == {k: v[0].data_ptr() for k, v in model._tkv_fused_weights.items()}
    assert model.generate(prompt, max_new_tokens=5, fused_decode=True).shape == (3, plen + 5)   # cache made by the model
    with pytest.raises(NotImplementedError):
        model.float().generate(prompt, max_new_tokens=2, fused_decode=True)


@pytest.mark.parametrize("strategy", ["alpha", "layer_wise_alpha"])
def test_flat_budget_cache_through_the_fused_decoder(strategy):
    """A budget-sharing flat cache stepped by the fused decode step (decode_prep instead of update) across several
    shared-budget evictions: same lengths, kept positions and logits as the module path that calls update(); the
    host-side row totals that trigger compress() and size the ragged attention grid stay in step with the device."""
    from trimkv_b200 import BatchedDynamicBudgetTrimKVCache
    from trimkv_b200.decoder import GreedyDecoder
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    model, cfg = _tiny(memory_size=64, buffer_size=8, layers=3)
    cfg.compress_strategy = strategy
    model = model.to(DEV)
    gen = torch.Generator().manual_seed(11)
    prompt = torch.randint(0, cfg.vocab_size, (3, 100), generator=gen).to(DEV)
    forced = torch.randint(0, cfg.vocab_size, (40, 3, 1), generator=gen).to(DEV)
    outs = []
    with torch.inference_mode():
        for fused in (False, True):
            cache = BatchedDynamicBudgetTrimKVCache(device=DEV)
            out = model(input_ids=prompt, past_key_values=cache, logits_to_keep=1)
            dec = GreedyDecoder(model, cache, use_graph=False, fused=fused)
            assert (dec.fused is not None) == fused
            logits, lens = [], []
            for t in range(40):
                dec.step(forced[t])
                logits.append(dec.logits.float().clone())
                lens.append(torch.stack([cache.head_lens[l].clone() for l in range(len(cache))]))
                # the host copy of the row totals equals the device's
                assert cache._rows == [int(cache.head_lens[l].sum()) for l in range(len(cache))], (fused, t)
            cache.check_status()
            pos = [cache.kv_positions[l].clone() for l in range(len(cache))]
            outs.append((torch.stack(logits), torch.stack(lens), pos))
    (l0, n0, p0), (l1, n1, p1) = outs
    assert int(n0.min()) < int(n0.max()), "the budget was shared unevenly between heads (what this cache is for)"
    assert float((l0 - l1).abs().max()) <= 2e-2
    same = (n0 == n1).float().mean().item()
    assert same >= 0.9, same   # a near-tie in bf16 may move a row between heads; the lengths then differ by one


@pytest.mark.parametrize("resident_min_ctas", [96, 1])
def test_chunked_prefill_matches_cpu_restatement(resident_min_ctas, monkeypatch):
    """(Second parameter value: the query-resident kernel serves every piece instead of the 32-row split-KV kernel or
    the library.)  The prompt fed in pieces (multi-token queries against the cache, eviction after every piece, capacity growing
    past M+B while a piece is appended): logits of every piece within 2e-2 of the eager CPU path fed the same pieces."""
    from oracle.qwen3_oracle import EagerTrimKVCache, OracleQwen3
    from trimkv_b200 import TrimKVCache, attn as attn_mod
    monkeypatch.setattr(attn_mod, "RESIDENT_MIN_CTAS", resident_min_ctas)
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    model, cfg = _tiny(memory_size=96, buffer_size=16, layers=2)
    ref = OracleQwen3(model.state_dict(), cfg, dtype=torch.bfloat16)
    model = model.to(DEV)
    gen = torch.Generator().manual_seed(7)
    prompt = torch.randint(0, cfg.vocab_size, (2, 230), generator=gen)
    pieces = [prompt[:, lo:lo + 40] for lo in range(0, 230, 40)]            # 5 x 40 + 30; 40 tokens x G=2 = 80 query rows
    pieces += [prompt[:, :7], prompt[:, 7:10]]                              # short follow-ups: the decode kernel's multi-token form
    cache, rcache = TrimKVCache(device=DEV), EagerTrimKVCache(canonical=True)
    worst, mismatched_rows = 0.0, 0
    with torch.inference_mode():
        for ids in pieces:
            out = model(input_ids=ids.to(DEV), past_key_values=cache, logits_to_keep=1)
            want = ref.forward(ids, rcache)
            worst = max(worst, float((out.logits.float().cpu() - want.float()).abs().max()))
            assert cache.get_seq_length() == rcache.get_seq_length()
            diverged = False
            for l in range(cfg.num_hidden_layers):
                assert cache.get_cache_length(l) == rcache.get_cache_length(l)
                rows = int((cache.kv_positions[l].cpu().to(torch.int64) != rcache.kv_positions[l]).any(-1).sum())
                mismatched_rows += rows
                diverged |= rows > 0
            if diverged:   # a near-tie at the boundary fell the other way: adopt the GPU state, stay in lock-step
                for l in range(cfg.num_hidden_layers):
                    rcache.key_cache[l] = cache.key_cache[l].cpu().clone()
                    rcache.value_cache[l] = cache.value_cache[l].cpu().clone()
                    rcache.retention_weights[l] = cache.retention_weights[l].cpu().to(torch.bfloat16)
                    rcache.kv_positions[l] = cache.kv_positions[l].cpu().to(torch.int64)
    cache.check_status()
    assert worst <= 2e-2, worst
    assert mismatched_rows <= 4, mismatched_rows
    # generate() with prefill_chunk_size walks the same pieces
    with torch.inference_mode():
        a = model.generate(prompt.to(DEV), max_new_tokens=4, past_key_values=TrimKVCache(device=DEV), prefill_chunk_size=40)
        c2 = TrimKVCache(device=DEV)
        for lo in range(0, 230, 40):
            out = model(input_ids=prompt[:, lo:lo + 40].to(DEV), past_key_values=c2, logits_to_keep=1)
        assert torch.equal(a[:, 230], out.logits[:, -1].argmax(-1))
