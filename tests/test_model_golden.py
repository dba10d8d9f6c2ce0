"""Model-level pins on CPU: the oracle decoder and this library's model classes against outputs of the reference's
own model classes (tests/golden/model_*.npz, made by tests/golden/make_golden.py from the reference checkout).

The cache here is the oracle's eager cache: these tests cover the caller (projection layouts, gates, RoPE, the order
gate -> RoPE -> update -> attention -> ... -> compress, HF ``generate`` plumbing, ``from_pretrained``), not the CUDA
kernels; tests/test_model_gpu.py runs the same vectors through the CUDA path.
"""
import os
import sys
import warnings

import numpy as np
import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import tiny_models as tm  # noqa: E402

warnings.filterwarnings("ignore")


def build(case, dtype=torch.float32, attn="sdpa"):
    import trimkv_b200 as t
    fam, extra, steps = tm.CASES[case]
    Cfg, Cls = {"qwen3": (t.TrimKVQwen3Config, t.TrimKVQwen3ForCausalLM), "llama": (t.TrimKVLlamaConfig, t.TrimKVLlamaForCausalLM),
                "phi3": (t.TrimKVPhi3Config, t.TrimKVPhi3ForCausalLM)}[fam]
    cfg = Cfg(**dict(tm.FAMILIES[fam], **extra), attn_implementation=attn, pad_token_id=0, eos_token_id=None, bos_token_id=None)
    model = Cls(cfg).eval()
    shapes = {k: tuple(v.shape) for k, v in model.state_dict().items()}
    model.load_state_dict({k: torch.from_numpy(v) for k, v in tm.fill_state_dict(shapes).items()}, strict=True)
    return model.to(dtype), cfg, np.load(os.path.join(HERE, "golden", f"model_{case}.npz")), steps


def feed(g, step):
    ids, P = torch.from_numpy(g["ids"]), tm.PROMPT_LEN
    return ids[:, :P] if step == 0 else ids[:, P + step - 1: P + step]


@pytest.mark.parametrize("case", sorted(tm.CASES))
def test_parameter_names_and_shapes_are_the_reference_s(case):
    model, cfg, g, _ = build(case)
    mine = {k: str(tuple(v.shape)) for k, v in model.state_dict().items()}
    assert sorted(mine) == list(g["param_names"])
    assert [mine[k] for k in sorted(mine)] == list(g["param_shapes"])


@pytest.mark.parametrize("case", sorted(tm.CASES))
def test_oracle_decoder_equals_reference_model_fp32(case):
    from oracle.qwen3_oracle import EagerTrimKVCache, OracleDecoder
    model, cfg, g, steps = build(case)
    ref, cache = OracleDecoder(model.state_dict(), cfg), EagerTrimKVCache(canonical=True)
    for step in range(steps + 1):
        logits = ref.forward(feed(g, step), cache)[:, -1]
        assert float((logits - torch.from_numpy(g["logits_fp32"][step])).abs().max()) <= 1e-5, step
        for l in range(cfg.num_hidden_layers):
            n = cache.get_cache_length(l)
            assert n == g["lens_fp32"][step, l]
            assert np.array_equal(cache.kv_positions[l].numpy(), g["pos_fp32"][step, l, :, :, :n]), (step, l)


@pytest.mark.parametrize("case", ["qwen3", "llama", "phi3"])
def test_oracle_decoder_close_to_reference_model_bf16(case):
    """bf16 on the same CPU with the same torch ops: near-ties may still fall differently between the fused SDPA call
    the golden run used and the eager attention of the oracle, so positions are compared by count."""
    from oracle.qwen3_oracle import EagerTrimKVCache, OracleDecoder
    model, cfg, g, steps = build(case)
    ref, cache = OracleDecoder(model.state_dict(), cfg, dtype=torch.bfloat16), EagerTrimKVCache(canonical=True)
    worst, bad_rows, rows = 0.0, 0, 0
    for step in range(steps + 1):
        logits = ref.forward(feed(g, step), cache)[:, -1].float()
        worst = max(worst, float((logits - torch.from_numpy(g["logits_bf16"][step])).abs().max()))
        for l in range(cfg.num_hidden_layers):
            n = cache.get_cache_length(l)
            assert n == g["lens_bf16"][step, l]
            bad_rows += int((cache.kv_positions[l].numpy() != g["pos_bf16"][step, l, :, :, :n]).any(-1).sum())
            rows += cache.kv_positions[l].shape[0] * cache.kv_positions[l].shape[1]
    assert worst <= 2e-2, worst
    assert bad_rows <= rows // 4, (bad_rows, rows)


@pytest.mark.parametrize("case", sorted(tm.CASES))
def test_model_classes_equal_reference_model_fp32(case):
    """This library's model classes (dense attention, eager cache) reproduce the reference model's logits exactly."""
    from oracle.qwen3_oracle import EagerTrimKVCache
    model, cfg, g, steps = build(case)
    cache = EagerTrimKVCache(canonical=True)
    with torch.no_grad():
        for step in range(steps + 1):
            out = model(input_ids=feed(g, step), past_key_values=cache, logits_to_keep=1)
            assert float((out.logits[:, -1] - torch.from_numpy(g["logits_fp32"][step])).abs().max()) <= 1e-5, step
            for l in range(cfg.num_hidden_layers):
                n = cache.get_cache_length(l)
                assert n == g["lens_fp32"][step, l]
                assert np.array_equal(cache.kv_positions[l].numpy(), g["pos_fp32"][step, l, :, :, :n]), (step, l)


@pytest.mark.parametrize("case", ["qwen3", "llama", "phi3"])
def test_hf_generate_returns_the_reference_s_tokens(case):
    """``GenerationMixin.generate`` with a TRIM-KV cache passed in, as examples/test_qwen3.py:51-55 calls it."""
    from oracle.qwen3_oracle import EagerTrimKVCache
    model, cfg, g, _ = build(case)
    prompt = torch.from_numpy(g["ids"][:, :tm.PROMPT_LEN])
    out = model.generate(prompt, attention_mask=torch.ones_like(prompt), max_new_tokens=24, do_sample=False,
                         past_key_values=EagerTrimKVCache(canonical=True))
    assert np.array_equal(out.numpy(), g["generate_ids"])


def test_from_pretrained_base_checkpoint_plus_gate_weights(tmp_path):
    """The reference's loading convention (modeling_trimkv_qwen3.py:510-571): ``config.base_model`` names the base
    checkpoint, ``trimkv_weights.pth`` beside config.json holds the parameters matched by ``trainable_params``."""
    import trimkv_b200 as t
    model, cfg, g, _ = build("qwen3")
    base_dir, gate_dir = tmp_path / "base", tmp_path / "trimkv"
    model.save_pretrained(base_dir)
    gates = {k: v.clone() + 0.25 for k, v in model.state_dict().items() if "retention_gate" in k}
    cfg2 = t.TrimKVQwen3Config.from_pretrained(base_dir)
    cfg2.base_model, cfg2.trainable_params = str(base_dir), "retention_gate"
    os.makedirs(gate_dir)
    cfg2.save_pretrained(gate_dir)
    torch.save(gates, gate_dir / "trimkv_weights.pth")
    loaded = t.TrimKVQwen3ForCausalLM.from_pretrained(str(gate_dir), load_trimkv_weights=True, download_from="local",
                                                      memory_size=77)
    assert loaded.config.memory_size == 77 and loaded.config.base_model == str(base_dir)
    sd = loaded.state_dict()
    for k, v in model.state_dict().items():
        want = gates[k] if k in gates else v
        assert torch.equal(sd[k], want), k
    with pytest.raises(ValueError):
        t.TrimKVQwen3ForCausalLM.from_pretrained(str(gate_dir), download_from="huggingface")
