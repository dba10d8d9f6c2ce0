#!/usr/bin/env python
"""Benchmark of the TRIM-KV cache hot path on B200: decode tok/s of the Qwen3-1.7B-shaped model.

    python bench.py --gpus N --steps K --warmup W            # this library (CUDA kernels)
    python bench.py --impl reference --steps K --warmup W    # the reference's eager path on the host cores

One "step" is one greedy decode step of the whole batch: for each of the 28 layers retention gate ->
RoPE -> cache append -> split-KV decode attention, then LM head and argmax, then the eviction check
(`compress`, which fires every `buffer_size` steps).  The prompt pass (32 x 8192 tokens) and its
hand-off eviction to M = 4096 run before the timed region.  Inputs are synthetic (random-init weights,
uniform random prompt ids).  With N GPUs every rank runs its own 32 requests (batch partition, no
collective on the cache path): weak scaling, value = all ranks' tokens / max-over-ranks time.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # benchmark-spec configs[1]: Qwen3-1.7B architecture, batch 32, 8192-token prompt, M=4096, B=128.
    "qwen3-1.7b-decode": dict(
        hidden_size=2048, num_hidden_layers=28, num_attention_heads=16, num_key_value_heads=8, head_dim=128,
        intermediate_size=6144, vocab_size=151936, rope_theta=1e6, retention_gate_intermediate_size=128,
        retention_gate_bias_init=3.0, memory_size=4096, buffer_size=128, batch=32, prompt=8192),
    # benchmark-spec configs[4] per GPU at 8 GPUs: Qwen3-14B architecture, 16 of the 128 requests, M=8192, B=256.  The prompt is
    # lengthened from 1024 to M+B tokens so that the cache is saturated when decoding starts (the configured run only
    # saturates after 7424 decode steps); the timed window then covers steady-state steps and their evictions.
    "qwen3-14b-decode": dict(
        hidden_size=5120, num_hidden_layers=40, num_attention_heads=40, num_key_value_heads=8, head_dim=128,
        intermediate_size=17408, vocab_size=151936, rope_theta=1e6, retention_gate_intermediate_size=128,
        retention_gate_bias_init=3.0, memory_size=8192, buffer_size=256, batch=16, prompt=8448),
    # small variant for quick checks of the harness itself (not a bench line)
    "tiny": dict(
        hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
        intermediate_size=512, vocab_size=1024, rope_theta=1e6, retention_gate_intermediate_size=32,
        retention_gate_bias_init=3.0, memory_size=256, buffer_size=32, batch=4, prompt=512),
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f)["hbm_gbs"], "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int, period_ms: int = 20):
        self.index, self.rows, self.proc, self.period_ms = index, [], None, period_ms

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", str(self.period_ms)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [x.strip() for x in line.split(",")]))

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.thread.join(timeout=2)

    def summary(self, t0=None, t1=None):
        """Median SM clock and the throttle reasons seen between wall-clock times t0 and t1 (all samples if None)."""
        sm, mx, reasons = [], 0, set()
        for t, r in list(self.rows):
            if len(r) < 6 or not r[0].isdigit() or (t0 is not None and not (t0 <= t <= t1)):
                continue
            sm.append(int(r[0])); mx = max(mx, int(r[1]))
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm)}


def build_model(cfg_kw, device, dtype=torch.bfloat16):
    from trimkv_b200 import TrimKVQwen3Config, TrimKVQwen3ForCausalLM
    kw = {k: v for k, v in cfg_kw.items() if k not in ("batch", "prompt")}
    cfg = TrimKVQwen3Config(**kw, compress_memory=True, compress_strategy="alpha", attn_implementation="tkv_b200")
    torch.manual_seed(0)
    with torch.device(device):
        model = TrimKVQwen3ForCausalLM(cfg).to(dtype)
    return model.eval(), cfg


def cpu_reference_run(cfg_kw, steps, warmup, sample_batch, seed=0):
    """Times the eager restatement of the reference's decode step on the host cores (see oracle/qwen3_oracle.py).

    Sample: `sample_batch` requests of the workload's batch, all layers, cache pre-filled with M random
    rows per head (the 8192-token prompt pass is skipped on the CPU), then `steps` decode steps, each with the
    reference's torch.cat append, eager attention and the compress check (fires every B steps).
    """
    from types import SimpleNamespace
    from oracle.qwen3_oracle import EagerTrimKVCache, OracleQwen3
    c = SimpleNamespace(**{k: v for k, v in cfg_kw.items() if k not in ("batch", "prompt")}, rms_norm_eps=1e-6,
                        compress_memory=True, compress_strategy="alpha")
    g = torch.Generator().manual_seed(seed)
    dt = torch.bfloat16
    L, H, Hq, D, hid, inter = (c.num_hidden_layers, c.num_key_value_heads, c.num_attention_heads, c.head_dim,
                               c.hidden_size, c.intermediate_size)
    sd = {"model.embed_tokens.weight": torch.randn(c.vocab_size, hid, generator=g) * 0.02,
          "model.norm.weight": torch.ones(hid), "lm_head.weight": torch.randn(c.vocab_size, hid, generator=g) * 0.02}
    for l in range(L):
        p = f"model.layers.{l}."
        for name, shape in (("self_attn.q_proj", (Hq * D, hid)), ("self_attn.k_proj", (H * D, hid)),
                            ("self_attn.v_proj", (H * D, hid)), ("self_attn.o_proj", (hid, Hq * D)),
                            ("mlp.gate_proj", (inter, hid)), ("mlp.up_proj", (inter, hid)), ("mlp.down_proj", (hid, inter)),
                            ("self_attn.retention_gate.linear1", (c.retention_gate_intermediate_size, hid)),
                            ("self_attn.retention_gate.linear2", (H, c.retention_gate_intermediate_size))):
            sd[p + name + ".weight"] = torch.randn(*shape, generator=g) * 0.02
        sd[p + "self_attn.retention_gate.linear1.bias"] = torch.zeros(c.retention_gate_intermediate_size)
        sd[p + "self_attn.retention_gate.bias"] = torch.full((H,), float(c.retention_gate_bias_init))
        for n in ("input_layernorm", "post_attention_layernorm", "self_attn.q_norm", "self_attn.k_norm"):
            sd[p + n + ".weight"] = torch.ones(D if "norm.weight" in n + ".weight" and "self_attn" in n else hid)
    model = OracleQwen3(sd, c, dtype=dt)
    cache = EagerTrimKVCache(canonical=False)  # torch.topk, exactly the reference's call
    M, seen = c.memory_size, cfg_kw["prompt"]
    for l in range(L):
        cache.key_cache.append(torch.randn(sample_batch, H, M, D, generator=g).to(dt))
        cache.value_cache.append(torch.randn(sample_batch, H, M, D, generator=g).to(dt))
        cache.retention_weights.append(torch.nn.functional.logsigmoid(torch.randn(sample_batch, H, M, generator=g) * 1.5 + 3).to(dt))
        cache.kv_positions.append(torch.sort(torch.rand(sample_batch, H, seen, generator=g).argsort(-1)[..., :M], -1)[0])
        cache.n_seen_tokens.append(seen)
    cache._seen_tokens = seen
    ids = torch.randint(0, c.vocab_size, (sample_batch, 1), generator=g)
    for _ in range(warmup):
        ids = model.forward(ids, cache).argmax(-1)
    t0 = time.perf_counter()
    for _ in range(steps):
        ids = model.forward(ids, cache).argmax(-1)
    dt_s = time.perf_counter() - t0
    return sample_batch * steps / dt_s, dt_s / steps * 1e3


def shutdown_process_group(decoder=None, limit_s: float = 60.0):
    """Tears the NCCL communicator down.  A captured decode graph that holds collectives of the communicator must be
    destroyed first: NCCL's communicator destruction waits until every CUDA graph that captured its work is gone.  A
    watchdog bounds the wait and turns a teardown that does not return into exit code 3 instead of a silent stall."""
    import torch.distributed as dist
    if decoder is not None:
        decoder.close()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()

    def give_up():
        sys.stderr.write(f"bench.py: communicator teardown did not return within {limit_s:.0f} s\n")
        sys.stderr.flush()
        os._exit(3)
    t = threading.Timer(limit_s, give_up)
    t.daemon = True
    t.start()
    dist.destroy_process_group()
    t.cancel()


def host_threads():
    """All host cores for the CPU arms: torch.distributed.run exports OMP_NUM_THREADS=1 to its workers, which would
    otherwise leave the eager baseline on one core."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    torch.set_num_threads(max(1, n))
    return torch.get_num_threads()


def reference_batch(wl, requested):
    """Requests the host-core arm decodes per step: the workload's full batch when the host has the memory for the
    eager path's cache plus the transient copies torch.cat makes of it, else the largest power-of-two fraction."""
    if requested:
        return min(requested, wl["batch"])
    per_request = wl["num_hidden_layers"] * wl["num_key_value_heads"] * (wl["memory_size"] + wl["buffer_size"]) * wl["head_dim"] * 2 * 2
    try:
        import psutil
        avail = psutil.virtual_memory().available
    except Exception:
        avail = 32 << 30
    weights = 4 << 30 if wl["hidden_size"] <= 2048 else 32 << 30
    b = wl["batch"]
    while b > 1 and weights + 3 * b * per_request > 0.6 * avail:
        b //= 2
    return b


def run_reference(args, wl_name, wl):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = host_threads()
    sample_batch = reference_batch(wl, args.cpu_batch)
    tok_s, ms = cpu_reference_run(wl, args.steps, args.warmup, sample_batch)
    full = sample_batch == wl["batch"]
    sample = (f"{'all ' if full else ''}{sample_batch} of {wl['batch']} requests per step, all {wl['num_hidden_layers']} layers, "
              f"cache pre-filled with M={wl['memory_size']} random rows per head (the prompt pass is not part of a decode "
              f"step), {args.steps} decode steps in bf16 on {cores} host threads"
              + ("" if full else "; tok/s is that of the sample (per-step work is linear in the requests)"))
    line = {
        "impl": "reference", "metric": "decode_tok_per_s", "value": tok_s, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": wl_name, "global_batch": wl["batch"], "batch_per_gpu": wl["batch"], "prompt_len": wl["prompt"],
                   "memory_size": wl["memory_size"], "buffer_size": wl["buffer_size"],
                   "cpu_sample_batch": sample_batch, "ran_on": "host cores of rank 0 (eager PyTorch path of the reference, restated)"},
        "cpu_baseline": {"value": tok_s, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tok_s, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def micro_cache_phase(kind, M, nseg, steps, warmup, ctas=1, cpu_baseline=True, dev=None, Bf=128, D=128):
    """The forced-eviction ("evict") or append ("append") phase of the kernel-level workload of the benchmark
    specification (its configs[2]): nseg segments of bf16 K/V with live lengths uniform in [M, M+B], log beta =
    logsigmoid(N(3, 1.5)) rounded to bf16, creation steps drawn without replacement from [0, 4M).  Every timed launch
    works on a buffer the previous launch did not touch (buffers rotate; each exceeds L2).  Returns a dict with GB/s
    from the algorithmic bytes (evict: 8 n + 1032 M per segment; append: 2 * 520 per segment) and CUDA-event times."""
    from trimkv_b200 import ops
    dev = dev or torch.device("cuda", torch.cuda.current_device())
    peak, peak_src = measured_peaks()
    g = torch.Generator(device=dev).manual_seed(0)
    cap = M + Bf
    ws = ops.evict_multi_workspace(nseg, M, ctas, dev) if ctas > 1 else None
    nbuf = max(2, min(4, int(2e9 // (nseg * cap * 512)) or 2)) if kind == "evict" else 1
    bufs = []
    for _ in range(nbuf):
        k = torch.randn(nseg * cap, D, generator=g, device=dev, dtype=torch.bfloat16)
        v = torch.randn(nseg * cap, D, generator=g, device=dev, dtype=torch.bfloat16)
        beta = torch.nn.functional.logsigmoid(torch.randn(nseg * cap, generator=g, device=dev) * 1.5 + 3).bfloat16().float()
        pos = torch.sort(torch.rand(nseg, 4 * M, generator=g, device=dev).argsort(-1)[:, :cap], -1)[0].to(torch.int32).view(-1)
        bufs.append((k, v, beta, pos))
    # append: `chain` launches back to back in one CUDA graph per timed sample (lengths leave room for them), so that the
    # device time of a launch is measured and not the host's dispatch of it; an L2 flush precedes every sample.
    chain = 32 if kind == "append" else 1
    len0 = torch.randint(M + 1 if kind == "evict" else M, cap + (1 if kind == "evict" else 1 - chain),
                         (nseg,), generator=g, device=dev, dtype=torch.int32)
    ln, cu = len0.clone(), torch.zeros(nseg + 1, dtype=torch.int32, device=dev)
    status = ops.new_status(dev)
    kn = torch.randn(nseg // 8, 8, 1, D, generator=g, device=dev, dtype=torch.bfloat16)
    bn = torch.zeros(nseg // 8, 8, 1, device=dev, dtype=torch.bfloat16)
    pn = torch.tensor([4 * M], device=dev)
    times = []
    graph = flush = None
    if kind == "append":
        k, v, beta, pos = bufs[0]
        ops.append(k, v, beta, pos, ln, cu, kn, kn, bn, pn, cap, status)      # module load etc. before the capture
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(chain):
                ops.append(k, v, beta, pos, ln, cu, kn, kn, bn, pn, cap, status)
        flush = torch.empty(192 << 20, dtype=torch.uint8, device=dev)
    for i in range(warmup + steps):
        k, v, beta, pos = bufs[i % nbuf]
        ln.copy_(len0)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if graph is not None:
            flush.zero_()
            e0.record()
            graph.replay()
            e1.record()
            if i >= warmup:
                times.append((e0, e1))
            continue
        e0.record()
        if kind == "evict":
            if ctas > 1:
                ops.evict_multi(k, v, beta, pos, ln, cu, nseg, nseg, cap, 4 * M + 1, M, M + 1, cap, ctas, ws, status=status)
            else:
                ops.evict(k, v, beta, pos, ln, cu, nseg, nseg, cap, 4 * M + 1, M, M + 1, cap, None, status)
        else:
            ops.append(k, v, beta, pos, ln, cu, kn, kn, bn, pn, cap, status)
        e1.record()
        if i >= warmup:
            times.append((e0, e1))
    torch.cuda.synchronize()
    assert ops.read_status(status) == 0
    n_sum = int(len0.long().sum())
    alg = (8 * n_sum + nseg * 1032 * M) if kind == "evict" else nseg * 2 * 520
    res = {"kernel": "evict_inplace_kernel" if kind == "evict" else "append_warp_per_segment",
           "config": {"nseg": nseg, "M": M, "B": Bf, "head_dim": D, "dtype": "bf16", "buffers": nbuf},
           "ctas_per_segment": ctas, "peak": peak, "peak_source": peak_src, "unit": "GB/s"}
    del bufs
    if cpu_baseline:
        # The reference's eager ops for the same phase on the host cores, on a sample of the segments
        # (src/trimkv/cache_utils.py:104-108 for append, :172-198 for eviction), same algorithmic-byte formula.
        ns, n = min(64, nseg), M + Bf
        gc = torch.Generator().manual_seed(0)
        kc = torch.randn(1, ns, n, D, generator=gc).bfloat16(); vc = torch.randn(1, ns, n, D, generator=gc).bfloat16()
        bc = torch.nn.functional.logsigmoid(torch.randn(1, ns, n, generator=gc) * 1.5 + 3).bfloat16()
        pc = torch.sort(torch.rand(1, ns, 4 * M, generator=gc).argsort(-1)[..., :n], -1)[0]
        reps, t0 = 0, time.perf_counter()
        while reps < 3 or time.perf_counter() - t0 < 3.0:
            if kind == "evict":
                sc = bc.to(torch.float32) * (4 * M + 1 - pc)
                idx, _ = torch.sort(torch.topk(sc, M, dim=-1).indices, dim=-1)
                _ = (kc.gather(-2, idx.unsqueeze(-1).expand(-1, -1, -1, D)), vc.gather(-2, idx.unsqueeze(-1).expand(-1, -1, -1, D)),
                     bc.gather(-1, idx), pc.gather(-1, idx))
            else:
                _ = (torch.cat([kc, kc[:, :, :1]], dim=-2), torch.cat([vc, vc[:, :, :1]], dim=-2),
                     torch.cat([bc, bc[:, :, :1]], dim=-1), torch.cat([pc, pc[:, :, :1]], dim=-1))
            reps += 1
        sec = (time.perf_counter() - t0) / reps
        cpu_alg = ns * (8 * n + 1032 * M) if kind == "evict" else ns * 2 * 520
        res["cpu_baseline"] = {"value": cpu_alg / sec / 1e9, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
                               "sample": f"{ns} of {nseg} segments with n = M+B = {n}, eager torch ops of the reference "
                                         f"({'score/topk/sort/4 gathers' if kind == 'evict' else '4 torch.cat'}), {reps} repetitions"}
    ms = sorted(a.elapsed_time(b) / chain for a, b in times)
    avg = sum(ms) / len(ms)
    if kind == "append":
        res["timing"] = (f"{chain} launches back to back in a CUDA graph per sample, L2 flushed before each sample; "
                         "2 MB per launch: bound by launch latency, not by bandwidth (the decode step appends inside "
                         "decode_prep_kernel and never runs this launch)")
    res.update({"algorithmic_bytes_per_launch": alg, "avg_ms": avg, "median_ms": ms[len(ms) // 2],
                "achieved": alg / (avg * 1e-3) / 1e9, "frac": alg / (avg * 1e-3) / 1e9 / peak,
                "frac_of_nominal_8tbs": alg / (avg * 1e-3) / 1e9 / 8000.0})
    return res


def run_micro(args):
    """Kernel microbenchmarks on the kernel-level shapes of the benchmark specification (its configs[2] and configs[3]); one JSON line each.

    evict : nseg segments, live lengths uniform in [M, M+B], keep top-M on every segment (forced), bf16, D=128.
    attn  : one layer of decode attention, batch x 8 KV heads, lengths lognormal(median 2048, sigma 1) in [64, 8192].
    append: one token per segment.
    steady: append every step, evict only the segments that reached M+B.
    generate: generate() of the model classes on --workload, HF loop against fused_decode=True (wall clock per token).
    multi : --q-tokens new tokens per request against M cached ones (a piece of a chunked prefill, multi-token
            decoding): the multi-token kernels beside the library attention, causal and with a length mask.
    Each timed launch works on data that was not touched by the previous one (buffers rotate; each is > L2).
    """
    from trimkv_b200 import ops
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peak, peak_src = measured_peaks()
    g = torch.Generator(device=dev).manual_seed(0)
    D, M, Bf, nseg = 128, args.M, 128, args.nseg
    res = {"micro": args.micro, "steps": args.steps, "warmup": args.warmup, "peak": peak, "peak_source": peak_src}
    times = []
    ws = ops.evict_multi_workspace(nseg, M, args.ctas, dev) if args.ctas > 1 else None
    res["ctas_per_segment"] = args.ctas
    if args.micro == "prefill":
        # One layer of the prompt pass: batch x S new tokens, dense causal attention over their own K/V (no cache yet),
        # the query-resident kernel beside the library attention.  --nseg = batch * 8 KV heads, --M = S.
        from trimkv_b200.attn import _dense_causal
        batch, hq, hkv, S = nseg // 8, 16, 8, M
        k = torch.randn(batch, hkv, S, D, generator=g, device=dev, dtype=torch.bfloat16)
        v = torch.randn(batch, hkv, S, D, generator=g, device=dev, dtype=torch.bfloat16)
        qh = torch.randn(batch, hq, S, D, generator=g, device=dev, dtype=torch.bfloat16)
        out = torch.empty(batch, S, hq, D, device=dev, dtype=torch.bfloat16)

        def avg_ms(fn):
            for _ in range(args.warmup):
                fn()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize(); e0.record()
            for _ in range(args.steps):
                fn()
            e1.record(); torch.cuda.synchronize()
            return e0.elapsed_time(e1) / args.steps
        ours = avg_ms(lambda: ops.prefill_attn(qh.transpose(1, 2), k, v, None, S, out, hkv, D ** -0.5, S))
        lib_ms = avg_ms(lambda: _dense_causal(qh, k, v, D ** -0.5))
        flops = 4.0 * batch * hq * D * S * (S + 1) / 2
        diff = float((_dense_causal(qh, k, v, D ** -0.5).float() - out.float()).abs().max())
        res.update({"config": {"batch": batch, "hq": hq, "hkv": hkv, "head_dim": D, "dtype": "bf16", "prompt_tokens": S},
                    "causal_flops": flops, "avg_ms": ours, "tflops": flops / (ours * 1e-3) / 1e12,
                    "library_causal_ms": lib_ms, "library_tflops": flops / (lib_ms * 1e-3) / 1e12,
                    "max_abs_diff_vs_library": diff})
        print(json.dumps(res))
        return
    if args.micro == "multi":
        from trimkv_b200.attn import _dense_causal, _ragged_causal
        batch, hq, hkv, Q = nseg // 8, 16, 8, args.q_tokens
        n, cap = M + Q, M + max(256, Q)
        k = torch.randn(nseg * cap, D, generator=g, device=dev, dtype=torch.bfloat16)
        v = torch.randn(nseg * cap, D, generator=g, device=dev, dtype=torch.bfloat16)
        lens = torch.full((nseg,), n, device=dev, dtype=torch.int32)
        q = torch.randn(batch, Q, hq, D, generator=g, device=dev, dtype=torch.bfloat16)
        out = torch.empty_like(q)
        wsm = torch.empty(ops._lib.lib().tkv_decode_attn_multi_workspace_bytes(batch, hq, hkv, D, n, Q), dtype=torch.uint8, device=dev)
        k4, v4, qh = k.view(batch, hkv, cap, D)[:, :, :n], v.view(batch, hkv, cap, D)[:, :, :n], q.transpose(1, 2)

        def avg_ms(fn):
            for _ in range(args.warmup):
                fn()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize(); e0.record()
            for _ in range(args.steps):
                fn()
            e1.record(); torch.cuda.synchronize()
            return e0.elapsed_time(e1) / args.steps
        ours = avg_ms(lambda: ops.decode_attn_multi(q, k, v, lens, cap, out, hkv, D ** -0.5, n, workspace=wsm))
        out_pf = torch.empty_like(out)
        resident = avg_ms(lambda: ops.prefill_attn(q, k, v, lens, cap, out_pf, hkv, D ** -0.5, n))
        res.update({"query_resident_ms": resident, "query_resident_kv_gbs": nseg * n * 4 * D / (resident * 1e-3) / 1e9,
                    "max_abs_diff_resident_vs_split": float((out_pf.float() - out.float()).abs().max())})
        res.update({"config": {"batch": batch, "hq": hq, "hkv": hkv, "head_dim": D, "dtype": "bf16", "q_tokens": Q,
                               "query_rows_per_segment": Q * hq // hkv, "cached_tokens": n},
                    "kv_bytes": nseg * n * 4 * D, "avg_ms": ours,
                    "library_causal_ms": avg_ms(lambda: _dense_causal(qh, k4, v4, D ** -0.5)),
                    "library_masked_ms": avg_ms(lambda: _ragged_causal(qh, k4, v4, lens, D ** -0.5)),
                    "max_abs_diff_vs_library": float((_dense_causal(qh, k4, v4, D ** -0.5).float() - out.float()).abs().max())})
        print(json.dumps(res))
        return
    if args.micro == "generate":
        # What a user of the model classes sees: tokens per second of generate() after the prompt pass, through the HF
        # loop over the module-by-module forward, the HF loop with config.fused_decode_step (the fused step, launched
        # from Python), and the fused, graph-replayed step (fused_decode=True).
        wl = WORKLOADS[args.workload]
        model, cfg = build_model(wl, dev)
        ids = torch.randint(0, cfg.vocab_size, (wl["batch"], wl["prompt"]), generator=g, device=dev)
        mask = torch.ones_like(ids)
        n_new = max(8, min(128, args.steps))

        def wall(n, **kw):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            out = model.generate(ids, attention_mask=mask, max_new_tokens=n, do_sample=False, **kw)
            torch.cuda.synchronize()
            assert out.shape == (wl["batch"], wl["prompt"] + n)
            return time.perf_counter() - t0

        res.update({"config": {"workload": args.workload, "batch": wl["batch"], "prompt": wl["prompt"],
                               "M": wl["memory_size"], "B": wl["buffer_size"], "new_tokens": n_new},
                    "timing": "HF loop: host time stamps of the streamer calls over the last n tokens; fused_decode: wall clock of generate(max_new_tokens=8+n) minus generate(max_new_tokens=8), the faster of two calls each"})
        class Stamps:
            """HF streamer that records when each step's tokens reached the host."""
            def __init__(self):
                self.t = []

            def put(self, value):
                self.t.append(time.perf_counter())

            def end(self):
                pass

        for name, kw, flag in (("hf_generate", {}, False), ("hf_generate_fused_step", {}, True),
                               ("fused_decode", {"fused_decode": True}, False)):
            model.config.fused_decode_step = flag           # True: one-token forward passes run as the fused CUDA step
            wall(4, **kw)                                   # warm-up: workspaces, kernel attributes, fused weights
            # every call builds a cache (and, on the fused paths, records a graph), whose cost varies from call to call
            # by more than the tokens in between take: the faster of two calls each
            if "fused_decode" not in kw:
                # the HF loop: time stamps of its streamer calls, from the 8th new token on (the graph of the fused step
                # has been recorded by then); a call's fixed costs (cache, graph) stay out of the figure
                st = Stamps()
                total = wall(8 + n_new, streamer=st, **kw)
                ms = (st.t[-1] - st.t[-1 - n_new]) / n_new * 1e3
                res[name] = {"ms_per_step": ms, "tok_per_s": wl["batch"] / (ms * 1e-3), "whole_call_s": total}
                continue
            # every call builds a cache and records a graph, whose cost varies from call to call by more than the tokens
            # in between take: the faster of two calls each
            short = min(wall(8, **kw), wall(8, **kw))
            full = min(wall(8 + n_new, **kw), wall(8 + n_new, **kw))
            ms = (full - short) / n_new * 1e3
            res[name] = {"ms_per_step": ms, "tok_per_s": wl["batch"] / (ms * 1e-3), "prompt_pass_and_8_tokens_s": short}
        print(json.dumps(res))
        return
    if args.micro == "steady":
        # Triggered steady state: every step appends one token to every segment, then evicts only the segments that
        # reached M+B (lengths start uniform in [M, M+B), so about 1/B of them fire per step).  Amortised per step.
        cap = M + Bf
        k = torch.randn(nseg * cap, D, generator=g, device=dev, dtype=torch.bfloat16)
        v = torch.randn(nseg * cap, D, generator=g, device=dev, dtype=torch.bfloat16)
        beta = torch.nn.functional.logsigmoid(torch.randn(nseg * cap, generator=g, device=dev) * 1.5 + 3).bfloat16().float()
        pos = torch.sort(torch.rand(nseg, 4 * M, generator=g, device=dev).argsort(-1)[:, :cap], -1)[0].to(torch.int32).view(-1)
        ln = torch.randint(M, cap, (nseg,), generator=g, device=dev, dtype=torch.int32)
        cu = torch.zeros(nseg + 1, dtype=torch.int32, device=dev)
        ops.rebuild_cu_seqlens(ln, cu, nseg, nseg)
        status = ops.new_status(dev)
        kn = torch.randn(nseg // 8, 8, 1, D, generator=g, device=dev, dtype=torch.bfloat16)
        bn = torch.full((nseg // 8, 8, 1), -0.05, device=dev, dtype=torch.bfloat16)
        # Lengths grow by one per step and fall back to M at M+B, so the firing pattern repeats every B steps: one period
        # is captured in a CUDA graph (append + eviction per step, nothing else) and replayed, which times the device
        # and not the host's dispatch of two to four small launches per step.  The scores' query index and the appended
        # position are those of the captured period; the work per step does not depend on them.
        ln_host, fired = ln.cpu().numpy().astype(np.int64), 0
        period = Bf
        args.warmup = max(1, args.warmup)      # the first call of a kernel (attribute set-up) stays outside the capture
        pns = [torch.full((1,), 4 * M + i, device=dev, dtype=torch.int64) for i in range(args.warmup + period)]

        def one_step(i):
            ops.append(k, v, beta, pos, ln, cu, kn, kn, bn, pns[i], cap, status)
            if args.ctas > 1:
                ops.evict_multi(k, v, beta, pos, ln, cu, nseg, nseg, cap, 4 * M + i + 1, M, cap, cap, args.ctas, ws,
                                status=status)
            else:
                ops.evict(k, v, beta, pos, ln, cu, nseg, nseg, cap, 4 * M + i + 1, M, cap, cap, None, status)

        for i in range(args.warmup):
            one_step(i)
            ln_host += 1
            ln_host[ln_host >= cap] = M
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(period):
                one_step(args.warmup + i)
        replays = max(2, args.steps // period)
        args.steps = replays * period
        fired = replays * nseg                 # every segment fires once per period
        graph.replay()                         # one untimed period (the state after it equals the state before it)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(); e0.record()
        for _ in range(replays):
            graph.replay()
        e1.record(); torch.cuda.synchronize()
        assert ops.read_status(status) == 0
        assert np.array_equal(ln.cpu().numpy(), ln_host)
        ms = e0.elapsed_time(e1) / args.steps
        alg = nseg * 2 * 520 + fired / args.steps * (8 * cap + 1032 * M)
        res.update({"config": {"nseg": nseg, "M": M, "B": Bf, "head_dim": D, "dtype": "bf16"},
                    "timing": f"{replays} replays of a CUDA graph holding one period of {period} steps",
                    "segments_evicted_per_step": fired / args.steps, "algorithmic_bytes_per_step": alg, "avg_ms_per_step": ms,
                    "achieved_gbs": alg / (ms * 1e-3) / 1e9, "frac_of_peak": alg / (ms * 1e-3) / 1e9 / peak})
        print(json.dumps(res))
        return
    if args.micro in ("evict", "append"):
        out = micro_cache_phase(args.micro, M, nseg, args.steps, args.warmup, args.ctas, not args.no_cpu_baseline, dev)
        out.update({"micro": args.micro, "steps": args.steps, "warmup": args.warmup, "achieved_gbs": out["achieved"],
                    "frac_of_peak": out["frac"]})
        print(json.dumps(out))
        return
    if True:
        if args.attn_shape == "config4":   # Qwen3-8B heads, ragged lengths
            batch, hq, hkv = args.nseg // 8, 32, 8
            lens = torch.exp(torch.randn(nseg, generator=g, device=dev) + 7.6246).clamp(64, 8192).round().to(torch.int32)
            cap = 8192
        else:                              # one layer of the decode benchmark: Qwen3-1.7B heads, n ~ M + B/2
            batch, hq, hkv = args.nseg // 8, 16, 8
            cap = M + Bf
            lens = torch.full((nseg,), M + Bf // 2, device=dev, dtype=torch.int32)
        nbuf = 2 if nseg * cap * 512 > (1 << 28) else 4
        bufs = [(torch.randn(nseg * cap, D, generator=g, device=dev, dtype=torch.bfloat16),
                 torch.randn(nseg * cap, D, generator=g, device=dev, dtype=torch.bfloat16)) for _ in range(nbuf)]
        q = torch.randn(batch, hq, D, generator=g, device=dev, dtype=torch.bfloat16)
        out = torch.empty_like(q)
        # With --token-bound the grid is sized by the total number of cached tokens (which the flat caches know on the
        # host) instead of by nseg * max_len.
        bound = int(lens.long().sum()) if args.token_bound else None
        res["token_bound"] = bound
        ws = torch.empty(ops.decode_attn_workspace_bytes(batch, hq, hkv, D, cap) if bound is None else
                         ops.decode_attn_workspace_bytes_ragged(batch, hq, hkv, D, cap, bound), dtype=torch.uint8, device=dev)
        seg_start = None
        if args.packed:   # the live rows of every segment back to back, as the reference's flat caches hold them
            mask = (torch.arange(cap, device=dev)[None, :] < lens[:, None]).view(-1)
            bufs = [(kk[mask].contiguous(), vv[mask].contiguous()) for kk, vv in bufs]
            cu = torch.zeros(nseg + 1, dtype=torch.int32, device=dev); cu[1:] = lens.cumsum(0)
            seg_start = cu[:-1].contiguous()
            res["layout"] = "packed"
        for i in range(args.warmup + args.steps):
            k, v = bufs[i % nbuf]
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            ops.decode_attn(q, k, v, lens, seg_start, cap, out, ws, hkv, D ** -0.5, cap, None, total_len_bound=bound)
            e1.record()
            if i >= args.warmup:
                times.append((e0, e1))
        torch.cuda.synchronize()
        alg = int(lens.long().sum()) * 4 * D + batch * hq * D * 4
        # The library kernel the reference calls for this step (flash_attn_varlen_func on the packed cache, every
        # (request, KV head) pair one sequence), timed the same way on the same lengths, for comparison.
        try:
            from flash_attn.flash_attn_interface import flash_attn_varlen_func
            mask = (torch.arange(cap, device=dev)[None, :] < lens[:, None]).view(-1)
            packs = ([(kk.unsqueeze(1), vv.unsqueeze(1)) for kk, vv in bufs] if args.packed else
                     [(kk[mask].unsqueeze(1).contiguous(), vv[mask].unsqueeze(1).contiguous()) for kk, vv in bufs])
            cu_k = torch.zeros(nseg + 1, dtype=torch.int32, device=dev); cu_k[1:] = lens.cumsum(0)
            cu_q = torch.arange(0, nseg + 1, dtype=torch.int32, device=dev)
            pq = q.view(batch, hkv, hq // hkv, D).reshape(nseg, hq // hkv, D).contiguous()
            mk = int(lens.max())
            fa = []
            for i in range(args.warmup + args.steps):
                kp, vp = packs[i % nbuf]
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                flash_attn_varlen_func(pq, kp, vp, cu_q, cu_k, max_seqlen_q=1, max_seqlen_k=mk, causal=True)
                e1.record()
                if i >= args.warmup:
                    fa.append((e0, e1))
            torch.cuda.synchronize()
            fa_ms = sum(a.elapsed_time(b) for a, b in fa) / len(fa)
            res["flash_attn_varlen"] = {"avg_ms": fa_ms, "achieved_gbs": alg / (fa_ms * 1e-3) / 1e9,
                                        "note": "kernel call only, Q already packed, max_seqlen_k precomputed"}
            del packs
        except Exception as e:  # wheel missing or not runnable on this GPU
            res["flash_attn_varlen"] = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
        res["config"] = {"batch": batch, "hq": hq, "hkv": hkv, "head_dim": D, "dtype": "bf16",
                         "mean_len": float(lens.float().mean()), "buffers": nbuf, "shape": args.attn_shape}
    ms = sorted(a.elapsed_time(b) for a, b in times)
    avg = sum(ms) / len(ms)
    res.update({"algorithmic_bytes_per_launch": alg, "avg_ms": avg, "median_ms": ms[len(ms) // 2],
                "achieved_gbs": alg / (avg * 1e-3) / 1e9, "frac_of_peak": alg / (avg * 1e-3) / 1e9 / peak})
    print(json.dumps(res))


def parse_args(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--micro", default=None, choices=["evict", "attn", "append", "steady", "multi", "prefill", "generate"],
                    help="run one kernel microbenchmark instead of the decode benchmark")
    ap.add_argument("--attn-shape", default="config4", choices=["config4", "config2"])
    ap.add_argument("--M", type=int, default=4096)
    ap.add_argument("--nseg", type=int, default=2048)
    ap.add_argument("--q-tokens", type=int, default=16, help="multi microbenchmark: new tokens per request")
    ap.add_argument("--packed", action="store_true",
                    help="attention microbenchmark: the reference's packed [sum n, D] layout (seg_start = cu_seqlens_k)")
    ap.add_argument("--token-bound", action="store_true",
                    help="attention microbenchmark: size the grid by the total token count (ragged lengths)")
    ap.add_argument("--ctas", type=int, default=1, help="CTAs sharing one segment in the eviction microbenchmarks")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--workload", default="qwen3-1.7b-decode", choices=sorted(WORKLOADS))
    ap.add_argument("--no-graph", action="store_true", help="dispatch every decode step from Python (no CUDA graph)")
    ap.add_argument("--no-fused", action="store_true", help="run the layer as separate PyTorch ops around the cache kernels")
    ap.add_argument("--head-sharded", action="store_true",
                    help="N > 1: all ranks decode the same requests, each owning Hkv/N KV heads (all-gather of attention "
                         "outputs per layer) instead of the default batch partition")
    ap.add_argument("--fused-gather", action="store_true",
                    help="with --head-sharded: the attention merge kernel stores into every rank's gathered buffer over "
                         "NVLink and raises a flag, instead of an NCCL all-gather per layer")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-batch", type=int, default=0,
                    help="requests per step of the host-core arm (--impl reference; 0 = the full batch if host memory allows)")
    ap.add_argument("--cpu-sample-batch", type=int, default=2, help="requests in the cpu_baseline sample of the native arm")
    ap.add_argument("--cpu-steps", type=int, default=12)
    ap.add_argument("--cache", default="per-head", choices=["per-head", "batched-budget"],
                    help="per-head: TrimKVCache (the benchmark's configuration).  batched-budget: "
                         "BatchedDynamicBudgetTrimKVCache with strategy 'alpha', the token budget shared between the heads "
                         "and layers of a request (ragged head lengths; evictions are not bracketed in this mode)")
    ap.add_argument("--blas", default="default", choices=["default", "cublas", "cublaslt"],
                    help="which library entry torch uses for the dense GEMMs of the decode step (torch.backends.cuda."
                         "preferred_blas_library); the GEMMs are library code either way")
    ap.add_argument("--tc-gemm", default="",
                    help="comma-separated subset of qkvg,o,gu,down: projections of the decode step that run on "
                         "tkv_skinny_gemm instead of the library GEMM")
    ap.add_argument("--no-evict-window", action="store_true",
                    help="do not advance the cache so that an eviction falls inside the timed windows (profiling runs)")
    ap.add_argument("--no-micro", action="store_true", help="skip the kernel-level evict / append phases of the default run")
    return ap.parse_args(argv)


def main():
    args = parse_args()
    wl = WORKLOADS[args.workload]
    if args.warmup < 3:
        args.warmup = 3
    if args.micro:
        return run_micro(args)
    if args.workload == "qwen3-14b-decode":
        args.cpu_sample_batch = 1
        args.cpu_batch = args.cpu_batch or 1
    if args.impl == "reference":
        if args.steps > 32:
            args.steps = 32  # bounded: the host-core run must end within minutes
        return run_reference(args, args.workload, wl)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the cache path has no CPU implementation "
                         "(use --impl reference for the host-core baseline)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    import torch.distributed as dist
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    if args.blas != "default":
        torch.backends.cuda.preferred_blas_library(args.blas)
    from trimkv_b200 import TrimKVCache, attn as tkv_attn, build as tkv_build, ops
    from trimkv_b200.decoder import GreedyDecoder
    if not os.path.exists(tkv_build.LIB) and local == 0:
        tkv_build.build()      # the library normally ships prebuilt; compile it where only the sources arrived
    if world > 1:
        dist.barrier()
    ops.lib()

    model, cfg = build_model(wl, dev)
    B, P, M, Bf = wl["batch"], wl["prompt"], wl["memory_size"], wl["buffer_size"]
    gen = torch.Generator().manual_seed(1000 + rank)
    prompt = torch.randint(0, cfg.vocab_size, (B, P), generator=gen).pin_memory()
    flat = args.cache == "batched-budget"
    if flat:
        from trimkv_b200 import BatchedDynamicBudgetTrimKVCache
        cache = BatchedDynamicBudgetTrimKVCache(device=dev)
        args.no_evict_window = True
    else:
        cache = TrimKVCache(device=dev, memory_size=M, buffer_size=Bf, num_layers=cfg.num_hidden_layers)
    with torch.inference_mode():
        out = model(input_ids=prompt.to(dev, non_blocking=True), past_key_values=cache, logits_to_keep=1)
        first = out.logits[:, -1].argmax(-1, keepdim=True)
        del out
        torch.cuda.empty_cache()
        sharded = args.head_sharded and world > 1
        if sharded:
            cache = cache.head_shard(rank, world)   # the prompt pass was replicated; keep this rank's KV heads only
            torch.cuda.empty_cache()
        dec = GreedyDecoder(model, cache, use_graph=not args.no_graph, fused=not args.no_fused,
                            head_shard_group=dist.group.WORLD if sharded else None,
                            fused_gather=sharded and args.fused_gather,
                            tc_gemm=frozenset(t for t in args.tc_gemm.split(",") if t))
        dec.ids.copy_(first)
        clocks = ClockSampler(local)
        clocks.__enter__()             # sampled from before the warm-up; the line reports the timed spans
        for _ in range(args.warmup):  # eager warm-up steps (allocate workspaces before any capture)
            dec.step(eager=True)
        if dec.use_graph:
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                dec.step(eager=True)
            torch.cuda.current_stream().wait_stream(s)
            dec.capture()
            for _ in range(3):
                dec.step()
        cache.check_status()

        def barrier():
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        def max_over_ranks(x):
            if world == 1:
                return x
            t = torch.tensor([x], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())

        def advance_to(steps_before_trigger):
            """Untimed steps until the cache is `steps_before_trigger` tokens short of M+B, so that a timed window
            of any length holds an all-layer eviction (it fires once per B steps; a short window would miss it)."""
            n = 0
            while not args.no_evict_window and (M + Bf - cache.get_cache_length(0)) % Bf != steps_before_trigger % Bf and n < Bf:
                dec.step(); n += 1
            return n

        def timed_steps(step_fn):
            """K steps between events; a step on which the eviction fires is split so that the eviction launch is
            bracketed by events of its own (graph replay, then compress: the same launches in the same order)."""
            evs = []
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            w0 = time.time()
            e0.record()
            for i in range(args.steps):
                if not flat and cache.get_cache_length(0) + 1 >= M + Bf:
                    n_before = cache.get_cache_length(0) + 1
                    comp, cfg.compress_memory = cfg.compress_memory, False
                    step_fn()
                    cfg.compress_memory = comp
                    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    ev0.record()
                    cache.compress(memory_size=M, buffer_size=Bf)
                    ev1.record()
                    evs.append((ev0, ev1, n_before))
                else:
                    step_fn()
            e1.record()
            barrier()
            return max_over_ranks(e0.elapsed_time(e1)), evs, (w0, time.time())

        # ---- timed region 1: device-resident decode (ids never leave the GPU); CUDA-graph replays only
        pre1 = advance_to(max(1, args.steps // 2))
        launches0 = ops.launch_count
        ms_total, evict_events, span1 = timed_steps(lambda: dec.step())
        launches = ops.launch_count - launches0

        # ---- timed region 2: end to end, ids cross PCIe both ways every step
        host_ids = torch.zeros(B, 1, dtype=torch.int64).pin_memory()
        host_ids.copy_(dec.next_ids)

        def e2e_step():
            nxt = dec.step(host_ids)                      # H2D of this step's input ids (pinned)
            host_ids.copy_(nxt, non_blocking=True)        # D2H of the step's result
            torch.cuda.current_stream().synchronize()
        pre2 = advance_to(max(1, args.steps // 2))
        ms_e2e, evict_events2, span2 = timed_steps(e2e_step)
        cache.check_status()

        # ---- untimed: the dominant kernel (decode attention) bracketed by events on the launching stream, on a few
        # eagerly dispatched steps (the graph replays above cannot be bracketed per kernel)
        attn_events, lens_at_sample = [], []
        for _ in range(4):
            tkv_attn.event_log = []
            # tokens per segment at this step (the budget-sharing cache keeps the layer's total on the host)
            lens_at_sample.append(cache._rows[0] / (B * cfg.num_key_value_heads) + 1 if flat else cache.get_cache_length(0) + 1)
            # Keep the GPU busy for a few milliseconds first so that the host queues the step's launches ahead of it;
            # otherwise the event pairs would also time the host's dispatch gaps between the two attention kernels.
            torch.cuda._sleep(20_000_000)
            dec.step(eager=True)
            attn_events.append(tkv_attn.event_log)
            tkv_attn.event_log = None
        torch.cuda.synchronize()
        clocks.__exit__(None, None, None)
        clk = clocks.summary(span1[0], span2[1])
        clk["samples_all"] = clocks.summary()["samples"]
        clk["window"] = "both timed regions"
        if clk["samples"] == 0:
            clk = dict(clocks.summary(), window="whole run (no sample fell inside the timed regions)")
        evict_events = evict_events + evict_events2

    tokens = B * args.steps * (1 if sharded else world)
    value = tokens / (ms_total * 1e-3)
    e2e = tokens / (ms_e2e * 1e-3)

    # ---- roofline of the dominant kernel (decode attention: reads every cached K/V row once per step)
    peak, peak_src = measured_peaks()
    Hq, Hkv, D, L = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.num_hidden_layers
    if sharded:  # per-rank kernels see this rank's heads only
        Hq, Hkv = Hq // world, Hkv // world
    ach = []
    for evs, n in zip(attn_events, lens_at_sample):
        bytes_per_launch = B * Hkv * n * 4 * D + B * Hq * D * 2 * 2
        for a, b in evs:
            ach.append((bytes_per_launch, a.elapsed_time(b) * 1e-3))
    roofline = None
    if ach:
        tot_b, tot_t = sum(x for x, _ in ach), sum(t for _, t in ach)
        gbs = tot_b / tot_t / 1e9
        # dram__bytes_read+write of one ncu capture of the same two kernels at this shape (batch 32, n = 4160):
        # 561.2 MB against 545.5 MB algorithmic; scaled by the bytes.
        traffic = tot_b / len(ach) * (561.19 / 545.52) if args.workload == "qwen3-1.7b-decode" else None
        roofline = {"bound": "hbm", "kernel": "decode_attn_tc_kernel+decode_attn_combine_kernel", "achieved": gbs,
                    "peak": peak, "unit": "GB/s", "frac": gbs / peak, "peak_source": peak_src,
                    "frac_of_nominal_8tbs": gbs / 8000.0, "traffic": traffic,
                    "launches_timed": len(ach), "avg_launch_us": tot_t / len(ach) * 1e6,
                    "bytes_per_launch": tot_b / len(ach)}
    evict = None
    if evict_events:
        nseg = L * B * Hkv
        eb = sum(nseg * (8 * n + (4 * D + 8) * 1 * M + 4 * D * M) for _, _, n in evict_events)  # 8n + 1032 M
        et = sum(a.elapsed_time(b) for a, b, _ in evict_events) * 1e-3
        evict = {"kernel": "evict_inplace_kernel", "segments": nseg, "achieved": eb / et / 1e9, "peak": peak,
                 "unit": "GB/s", "frac": eb / et / 1e9 / peak, "frac_of_nominal_8tbs": eb / et / 1e9 / 8000.0,
                 "launches_timed": len(evict_events),
                 "avg_launch_ms": et / len(evict_events) * 1e3}

    # ---- the second half of the metric, "cache update+evict GB/s": besides the in-window eviction above, the forced
    # eviction and the append phase of the kernel-level workload (2048 segments, M = 4096, B = 128) on rank 0.
    want_cpu = rank == 0 and world == 1 and not args.no_cpu_baseline
    evict_micro = append_micro = None
    if rank == 0 and not args.no_micro:
        if want_cpu:
            host_threads()
        with torch.inference_mode():
            evict_micro = micro_cache_phase("evict", 4096, 2048, 20, 5, 1, want_cpu, dev)
            append_micro = micro_cache_phase("append", 4096, 2048, 50, 10, 1, want_cpu, dev)
        append_micro["note"] = "2 MB per launch: bound by launch latency, not by bandwidth"

    # The window holds one eviction per `steps` steps although it fires once per B steps: the same measurement with
    # the eviction's share scaled to its true rate, for comparison with longer windows.
    ev1_ms = sum(a.elapsed_time(b) for a, b, _ in evict_events[:len(evict_events) - len(evict_events2)])
    steady_ms = (ms_total - ev1_ms) / args.steps + ev1_ms / max(1, len(evict_events) - len(evict_events2)) / Bf \
        if len(evict_events) > len(evict_events2) else ms_total / args.steps

    cpu = None
    if want_cpu:
        cores = host_threads()
        tok_s, ms = cpu_reference_run(wl, args.cpu_steps, 2, args.cpu_sample_batch)
        cpu = {"value": tok_s, "unit": "tok/s", "cores": cores, "kind": "port",
               "sample": f"{args.cpu_sample_batch} of {B} requests, all {L} layers, cache pre-filled with M={M} random rows per head, "
                         f"{args.cpu_steps} decode steps in bf16 ({ms:.0f} ms/step); tok/s of the sample (per-step work is "
                         "linear in the requests)"}

    if rank == 0:
        line = {
            "metric": "decode_tok_per_s", "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_total / args.steps, "higher_is_better": True,
            "scaling": "strong" if sharded else "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": args.workload, "global_batch": B * (1 if sharded else world), "batch_per_gpu": B, "prompt_len": P,
                       "memory_size": M, "buffer_size": Bf, "parallelism": ((f"kv-head-shard x{world}" + (" (merge kernel pushes to peers)" if args.fused_gather else " (NCCL all-gather)"))
                                       if sharded else f"batch-partition x{world}"),
                       "cache": args.cache, "blas": args.blas, "cuda_graph": dec.use_graph, "fused_layer_kernels": dec.fused is not None,
                       "untimed_steps_before_windows": [pre1, pre2],
                       "evictions_in_windows": len(evict_events),
                       "l2": "per-step working set (all weights + every cached K/V row, many GB) exceeds the 126 MB L2; no explicit flush"},
            "ms_per_step_at_true_eviction_rate": steady_ms,
            "roofline": roofline, "evict": evict, "evict_micro": evict_micro, "append": append_micro, "cpu_baseline": cpu,
            "e2e": {"value": e2e, "unit": "tok/s", "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": B * 8 * world, "d2h_bytes_per_step": B * 8 * world},
            "gpu_launches": launches * world, "clocks": clk,
        }
        print(json.dumps(line))
    if world > 1:
        sys.stdout.flush()
        shutdown_process_group(dec)


if __name__ == "__main__":
    main()
