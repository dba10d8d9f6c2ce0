"""Greedy decode loop around `TrimKVQwen3ForCausalLM` + `TrimKVCache`, optionally as a CUDA graph.

The reference decodes through HF ``generate`` (one Python-dispatched forward per token,
examples/test_qwen3.py:51).  Here the per-token forward (all layers: gate -> RoPE -> append ->
decode attention, then LM head and argmax) can be captured once in a CUDA graph and replayed; the
eviction (`cache.compress`) stays outside the graph because the host decides when it fires.
"""
from __future__ import annotations

import os
import weakref
from typing import Optional

import torch

from . import ops
from .cache_utils import TrimKVCache


class FusedDecodeStep:
    """One-token forward of the whole decoder with the fused CUDA kernels around the GEMMs.

    Per layer: add+RMSNorm -> one GEMM for q|k|v|gate.linear1 -> decode_prep (q/k-norm, RoPE, gate tail,
    append) -> split-KV decode attention -> o_proj -> add+RMSNorm -> one GEMM for gate|up -> SiLU*up ->
    down_proj: 10 launches instead of ~60.  The GEMMs stay cuBLAS (through torch); the concatenated
    weights replace the originals' storage (the module parameters become views of them).
    """

    @staticmethod
    def supports(model) -> bool:
        """Shapes the fused kernels cover: head_dim 128 rotated in full, the ``rg`` gate with at most 1024 hidden
        units, SiLU activations (and, when it runs, 16-bit weights).  Anything else decodes through the module path."""
        from .modeling_trimkv import head_dim_of, rotary_dim_of
        cfg = model.config
        return (head_dim_of(cfg) == 128 and rotary_dim_of(cfg) == 128 and cfg.retention_gate == "rg"
                and getattr(cfg, "hidden_act", "silu") == "silu")

    def __init__(self, model, cache: TrimKVCache, tc_gemm: bool = False, fused_down: bool = False):
        cfg = model.config
        if not self.supports(model):
            raise NotImplementedError("fused decode step needs head_dim 128 (fully rotated), retention_gate 'rg' and SiLU")
        # The cache is held weakly: a step may be stored on its cache (TrimKVForCausalLM.forward does), and a strong
        # reference back would keep gigabytes of slabs alive until the cycle collector happens to run.
        self.model, self._cache, self.cfg = model, weakref.ref(cache), cfg
        self.layers = []

        fused_before = model.__dict__.setdefault("_tkv_fused_weights", {})   # a second decoder of this model reuses them

        def fuse(parts):
            """One weight (and bias) for several Linear modules that read the same input; the modules' parameters
            become views of the fused storage."""
            if len(parts) == 1:
                return parts[0].weight, parts[0].bias
            key = tuple(id(m) for m in parts)
            if key in fused_before:
                w, bias = fused_before[key]
                off, same = 0, True
                for m in parts:      # still the views made below (nobody loaded or moved the weights since)?
                    same = same and m.weight.data_ptr() == w[off:].data_ptr() and m.weight.dtype == w.dtype
                    off += m.weight.shape[0]
                if same and off == w.shape[0]:
                    return w, bias
            w = torch.cat([m.weight for m in parts], 0).contiguous()
            bias = None
            if any(m.bias is not None for m in parts):
                bias = torch.cat([m.bias if m.bias is not None else m.weight.new_zeros(m.weight.shape[0])
                                  for m in parts]).contiguous()
            off = 0
            for m in parts:
                n = m.weight.shape[0]
                m.weight.data = w[off:off + n]
                if m.bias is not None:
                    m.bias.data = bias[off:off + n]
                off += n
            fused_before[key] = (w, bias)
            return w, bias

        with torch.no_grad():
            for layer in model.model.layers[: cfg.num_hidden_layers]:
                at, mlp = layer.self_attn, layer.mlp
                # Phi-3 ships q|k|v and gate|up already fused (modeling_trimkv_phi3.py:98,338); Qwen3 and Llama do not.
                qkv = [at.qkv_proj] if hasattr(at, "qkv_proj") else [at.q_proj, at.k_proj, at.v_proj]
                w, bias = fuse(qkv + [at.retention_gate.linear1])
                gu, gu_bias = fuse([mlp.gate_up_proj] if hasattr(mlp, "gate_up_proj") else [mlp.gate_proj, mlp.up_proj])
                self.layers.append((layer, w, bias, gu, gu_bias))
        self.hq, self.hkv, self.eps = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.rms_norm_eps
        # tc_gemm: tkv_skinny_gemm for the four per-layer projections instead of the library GEMMs (True, or the subset
        # of {"qkvg", "o", "gu", "down"} to switch).  Off by default: at 32
        # rows these GEMMs are bound by launch and pipeline-fill latency, and the tensor-core kernel only matches cuBLAS
        # (5-12 us per call either way on B200) while its fp32 partials make the consumers slower.
        # fused_down: the MLP's activation and down projection as one kernel (tkv_skinny_gemm_swiglu) instead of
        # tkv_silu_mul + a library GEMM.  Off by default: measured 4.47 ms per decode step against 4.11 ms (Qwen3-1.7B
        # shape, batch 32): converting the activation tiles inside the GEMM's pipeline costs more than the launch it saves.
        self.use_tc_gemm, self.fused_down = tc_gemm, fused_down
        self._partials = {}

    @property
    def cache(self) -> TrimKVCache:
        cache = self._cache()
        if cache is None:
            raise RuntimeError("the cache this decode step was built for no longer exists")
        return cache

    def _gemm(self, x, w, tag):
        """x [B, K] @ w [N, K].T through the weight-streaming tensor-core kernel; returns (partials, splits), or
        (None, 0) when the shape is outside its envelope (then the caller uses the library GEMM)."""
        m, k = x.shape
        n = w.shape[0]
        use = self.use_tc_gemm if isinstance(self.use_tc_gemm, bool) else tag in self.use_tc_gemm
        splits = ops.skinny_gemm_splits(m, n, k) if use else 0
        if splits == 0:
            return None, 0
        buf = self._partials.get((tag, m))
        if buf is None:
            buf = torch.empty(splits, m, n, dtype=torch.float32, device=x.device)
            self._partials[(tag, m)] = buf
        ops.skinny_gemm(x, w, buf, self.cache._status)
        return buf, splits

    def __call__(self, ids: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        """ids [B,1] int64, pos [1] int64 (device) -> logits [B, vocab]."""
        import torch.nn.functional as F
        from .attn import tkv_attention_forward
        m, cache = self.model.model, self.cache
        bsz = ids.shape[0]
        x = F.embedding(ids.view(bsz), m.embed_tokens.weight)          # residual stream, updated in place
        cos, sin = m.rotary_emb(x, pos.view(1, 1))
        cos, sin = cos.reshape(-1), sin.reshape(-1)
        h = torch.empty_like(x)
        q_out = torch.empty(bsz, self.hq, 1, 128, dtype=x.dtype, device=x.device)
        delta, d_splits = None, 0
        d_bias = None
        for l, (layer, w_qkvg, b_qkvg, w_gu, b_gu) in enumerate(self.layers):
            at = layer.self_attn
            ops.add_rmsnorm(x, delta, layer.input_layernorm.weight, h, self.eps, d_splits, d_bias if d_splits else None)
            qkvg, s1 = self._gemm(h, w_qkvg, "qkvg")
            if s1 == 0:
                qkvg = F.linear(h, w_qkvg, b_qkvg)
            qn, kn = getattr(at, "q_norm", None), getattr(at, "k_norm", None)
            k, v, kw = cache.decode_prep(l, qkvg, qn.weight if qn is not None else None,
                                         kn.weight if kn is not None else None, self.eps, cos, sin,
                                         at.retention_gate.linear2.weight, at.retention_gate.bias, pos, q_out, self.hq,
                                         s1, b_qkvg if s1 else None)
            o, _, _ = tkv_attention_forward(at, q_out, k, v, None, scaling=at.scaling, flash_attn_kwargs=kw)
            a, s2 = self._gemm(o.view(bsz, -1), at.o_proj.weight, "o")
            if s2 == 0:
                a = F.linear(o.view(bsz, -1), at.o_proj.weight, at.o_proj.bias)
            ops.add_rmsnorm(x, a, layer.post_attention_layernorm.weight, h, self.eps, s2, at.o_proj.bias if s2 else None)
            gu, s3 = self._gemm(h, w_gu, "gu")
            if s3 == 0:
                gu = F.linear(h, w_gu, b_gu)
            d_bias = layer.mlp.down_proj.bias
            w_down = layer.mlp.down_proj.weight
            d_splits = ops.skinny_gemm_splits(bsz, w_down.shape[0], w_down.shape[1]) if (self.fused_down and s3 == 0) else 0
            if d_splits:
                delta = self._partials.get(("down_swiglu", bsz))
                if delta is None:
                    delta = torch.empty(d_splits, bsz, w_down.shape[0], dtype=torch.float32, device=x.device)
                    self._partials[("down_swiglu", bsz)] = delta
                ops.skinny_gemm_swiglu(gu, w_down, delta, self.cache._status)
                continue
            act = torch.empty(bsz, w_gu.shape[0] // 2, dtype=x.dtype, device=x.device)
            ops.silu_mul(gu, act, s3, b_gu if s3 else None)
            delta, d_splits = self._gemm(act, w_down, "down")
            if d_splits == 0:
                delta = F.linear(act, w_down, d_bias)
        ops.add_rmsnorm(x, delta, m.norm.weight, h, self.eps, d_splits, d_bias if d_splits else None)
        return F.linear(h, self.model.lm_head.weight)


class GraphedForwardStep:
    """The fused decode step behind ``TrimKVForCausalLM.forward`` (``config.fused_decode_step``): static input buffers, two
    plain calls that size the workspaces, then one CUDA graph replayed per call.  Lives on the cache it serves and refers
    to it weakly; the caller passes the cache to every call.  The graph is dropped and recorded again when the cache's
    slabs were re-homed (growth without eviction) and is not used for a step that would exceed the capacity (that step
    runs plainly, which grows the slabs)."""

    EAGER_CALLS = 2

    def __init__(self, model, cache: TrimKVCache, use_graph: bool = True):
        self.step = FusedDecodeStep(model, cache)
        self.model, self.use_graph = model, use_graph
        dev = model.device
        self.ids = torch.zeros(cache._batch, 1, dtype=torch.int64, device=dev)
        self.pos = torch.zeros(1, dtype=torch.int64, device=dev)
        self.calls, self.graph, self.logits, self.key, self.launches_per_replay = 0, None, None, None, 0

    def _slab_key(self, cache):
        return (cache._slab["k"].data_ptr(), cache._cap, cache._batch) if cache._slab is not None else None

    def release_graph(self) -> None:
        if self.graph is not None:
            torch.cuda.synchronize()
            self.graph.reset()
            self.graph, self.logits = None, None

    def __call__(self, cache: TrimKVCache, input_ids: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        """input_ids [B,1], pos int64[1] (device) -> logits [B, vocab] (a tensor of the caller's own)."""
        self.ids.copy_(input_ids)
        self.pos.copy_(pos)
        fits = cache._slab is not None and max(cache._cache_len) + 1 <= cache._cap
        if self.graph is not None and (self.key != self._slab_key(cache) or not fits):
            self.release_graph()
            self.calls, cache.static_views = 0, False
        if (not self.use_graph or not fits or self.calls < self.EAGER_CALLS or torch.cuda.is_current_stream_capturing()):
            self.calls += 1
            return self.step(self.ids, self.pos)
        if self.graph is None:
            cache.static_views = True        # views of the whole capacity: the recorded launches stay valid as lengths grow
            snap = cache.snapshot_counters()
            self.graph = torch.cuda.CUDAGraph()
            before = ops.launch_count
            with torch.cuda.graph(self.graph):
                self.logits = self.step(self.ids, self.pos)
            self.launches_per_replay = ops.launch_count - before
            ops.launch_count = before
            cache.restore_counters(snap)
            self.key = self._slab_key(cache)
        self.graph.replay()
        ops.launch_count += self.launches_per_replay
        cache.advance(1)
        return self.logits.clone()


class GreedyDecoder:
    """Steps a prefilled (model, cache) pair one token at a time.

    ``step(ids)``: ``ids`` is ``[B,1]`` int64 on the host (pinned) or device, or None to feed back the
    previous step's argmax without leaving the device.  Returns the device tensor holding the new ids.
    """

    def __init__(self, model, cache: TrimKVCache, use_graph: bool = True, fused: bool = True, head_shard_group=None,
                 fused_gather: bool = False, tc_gemm: bool = False, fused_down: bool = False):
        self.model, self.cache, self.cfg = model, cache, model.config
        self.fused = None
        if head_shard_group is not None:
            self.fused = HeadShardedDecodeStep(model, cache, head_shard_group, fused_gather=fused_gather)
        elif fused and FusedDecodeStep.supports(model) and model.lm_head.weight.dtype in (torch.bfloat16, torch.float16):
            self.fused = FusedDecodeStep(model, cache, tc_gemm=tc_gemm, fused_down=fused_down)
        dev = model.device
        self.batch = cache._batch
        self.ids = torch.zeros(self.batch, 1, dtype=torch.int64, device=dev)
        self.next_ids = torch.zeros(self.batch, 1, dtype=torch.int64, device=dev)
        self.pos = torch.full((1,), cache.get_seq_length(), dtype=torch.int64, device=dev)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.use_graph = use_graph

    def _forward(self):
        cfg = self.cfg
        if self.fused is not None:
            self.logits = self.fused(self.ids, self.pos)
        else:
            compress, cfg.compress_memory = cfg.compress_memory, False  # eviction is driven from step()
            auto, cfg.fused_decode_step = getattr(cfg, "fused_decode_step", False), False   # this branch is the module path
            try:
                out = self.model(input_ids=self.ids, past_key_values=self.cache, cache_position=self.pos,
                                 logits_to_keep=1)
            finally:
                cfg.compress_memory, cfg.fused_decode_step = compress, auto
            self.logits = out.logits[:, -1]
        self.next_ids.copy_(self.logits.argmax(-1, keepdim=True))
        self.ids.copy_(self.next_ids)
        self.pos.add_(1)

    def capture(self):
        """Records one decode step.  Views handed to attention span the full capacity so the recorded
        launch geometry is valid for every later length; the kernels read the live lengths on the device."""
        self.cache.static_views = True
        snap = self.cache.snapshot_counters()
        self.graph = torch.cuda.CUDAGraph()
        before = ops.launch_count
        with torch.cuda.graph(self.graph):
            self._forward()
        self.launches_per_replay = ops.launch_count - before
        ops.launch_count = before
        self.cache.restore_counters(snap)

    def release_graph(self) -> None:
        """Destroys the captured decode graph (the next ``step`` captures again).  Needed before a process group whose
        collectives the graph recorded is destroyed: the communicator's destruction waits for every graph that
        captured its work."""
        if self.graph is not None:
            torch.cuda.synchronize()
            self.graph.reset()
            self.graph = None

    def close(self) -> None:
        """Releases what ties this decoder to other ranks: the captured graph and, in the head-sharded mode that
        pushes over NVLink, the mappings of the peers' exchange blocks (collective: every rank calls it)."""
        self.release_graph()
        if hasattr(self.fused, "close"):
            self.fused.close()

    def step(self, ids: Optional[torch.Tensor] = None, eager: bool = False) -> torch.Tensor:
        if ids is not None:
            self.ids.copy_(ids, non_blocking=True)
        if self.use_graph and not eager:
            if self.graph is None:
                self.capture()
            self.graph.replay()
            ops.launch_count += self.launches_per_replay
            self.cache.advance(1)
        else:
            self._forward()
        self.model.model.compress_after_forward(self.cache)     # the eviction check that ends the model's forward pass
        return self.next_ids


class HeadShardedDecodeStep(FusedDecodeStep):
    """Decode step with the KV heads (and their query heads, cache segments and attention) split across ranks.

    Rank r of N owns KV heads ``[r*Hkv/N, (r+1)*Hkv/N)``: its slice of the q/k/v projections and of the gate's second
    layer, the cache segments of those heads for every request, and their attention.  After attention one all-gather
    of ``[B, Hq/N * D]`` per layer (NCCL over NVLink) rebuilds ``[B, Hq * D]``; o_proj, the MLP and the LM head are
    replicated, so every rank ends the step with the same logits.  Nothing on the cache path is exchanged: a segment
    is appended to, evicted and attended on the rank that owns it.  The reference has no counterpart (it is single
    process); per head the arithmetic is that of the unsharded step.
    """

    def __init__(self, model, cache: TrimKVCache, group=None, fused_gather: bool = False):
        import torch.distributed as dist
        super().__init__(model, cache)
        self.group = group
        # fused_gather: the attention merge stores into every rank's gathered buffer over NVLink and raises a flag
        # (PeerExchange) instead of a separate all-gather; set up lazily, when the batch size is known.
        self.fused_gather, self._xchg = fused_gather, None
        if fused_gather and model.config.num_hidden_layers < 2:
            # The buffer rotation relies on a second exchange between two uses of a buffer (it is what proves that the
            # peers have read it); a one-layer model has none.
            raise ValueError("fused_gather needs a model of at least two layers")
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        cfg = model.config
        if cfg.num_key_value_heads % self.world:
            raise ValueError(f"{cfg.num_key_value_heads} KV heads cannot be split over {self.world} ranks")
        self.hkv_l = cfg.num_key_value_heads // self.world
        self.hq_l = cfg.num_attention_heads // self.world
        if cache._hkv != self.hkv_l:
            raise ValueError("the cache must hold this rank's KV heads only (see TrimKVCache.head_shard)")
        d, hq, hkv = 128, cfg.num_attention_heads, cfg.num_key_value_heads
        q0, k0 = self.rank * self.hq_l * d, self.rank * self.hkv_l * d
        self.local = []
        with torch.no_grad():
            for layer, w, bias, _, _ in self.layers:
                rows = torch.cat([torch.arange(q0, q0 + self.hq_l * d), hq * d + torch.arange(k0, k0 + self.hkv_l * d),
                                  (hq + hkv) * d + torch.arange(k0, k0 + self.hkv_l * d),
                                  torch.arange((hq + 2 * hkv) * d, w.shape[0])]).to(w.device)
                g = layer.self_attn.retention_gate
                h0 = self.rank * self.hkv_l
                self.local.append((w[rows].contiguous(), None if bias is None else bias[rows].contiguous(),
                                   g.linear2.weight[h0:h0 + self.hkv_l].contiguous(), g.bias[h0:h0 + self.hkv_l].contiguous()))

    def close(self) -> None:
        if self._xchg is not None:
            self._xchg.close()
            self._xchg = None

    def _attend_and_push(self, l, q_out, k, v, kw, scaling):
        """Attention of this rank's heads, merged straight into every rank's gathered buffer; returns the local one
        once all ranks' blocks have arrived (stream-ordered)."""
        from .attn import _workspace
        from .parallel import PeerExchange
        bsz, dim = q_out.shape[0], q_out.shape[-1]
        width = self.hq_l * self.world * dim
        if self._xchg is None:
            self._xchg = PeerExchange(bsz, width, q_out.dtype, q_out.device, nbuf=3, group=self.group)
            self._local_out = torch.empty(bsz, self.hq_l, dim, dtype=q_out.dtype, device=q_out.device)
        x = self._xchg
        # Layer 0 has a buffer of its own and the others alternate, so that a buffer is never rewritten before
        # every rank has read its previous content (see tkv_decode_attn_push in the header).
        i = 2 if l == 0 else (l & 1)
        max_len, cap = k.shape[2], k.stride(1) // dim
        ws = _workspace(q_out.device, ops.decode_attn_workspace_bytes(bsz, self.hq_l, self.hkv_l, dim, max_len))
        ops.decode_attn_push(q_out[:, :, 0, :], k, v, kw["head_lens"], cap, self._local_out, ws, self.hkv_l, scaling,
                             max_len, x.out_ptrs[i], x.flag_ptrs, self.world, self.rank, width,
                             self.rank * self.hq_l * dim, x.sync, kw.get("status"))
        ops.peer_wait(x.flags, x.sync, self.world, self.rank, kw.get("status"))
        return x.buffer(i)

    def __call__(self, ids: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist
        import torch.nn.functional as F
        from .attn import tkv_attention_forward
        m, cache = self.model.model, self.cache
        bsz = ids.shape[0]
        x = F.embedding(ids.view(bsz), m.embed_tokens.weight)
        cos, sin = m.rotary_emb(x, pos.view(1, 1))
        cos, sin = cos.reshape(-1), sin.reshape(-1)
        h = torch.empty_like(x)
        q_out = torch.empty(bsz, self.hq_l, 1, 128, dtype=x.dtype, device=x.device)
        gathered = torch.empty(self.world, bsz, self.hq_l * 128, dtype=x.dtype, device=x.device)
        delta = None
        for l, (layer, _, _, w_gu, b_gu) in enumerate(self.layers):
            at = layer.self_attn
            w_l, b_l, g2_l, gb_l = self.local[l]
            ops.add_rmsnorm(x, delta, layer.input_layernorm.weight, h, self.eps)
            qkvg = F.linear(h, w_l, b_l)
            qn, kn = getattr(at, "q_norm", None), getattr(at, "k_norm", None)
            k, v, kw = cache.decode_prep(l, qkvg, qn.weight if qn is not None else None,
                                         kn.weight if kn is not None else None, self.eps, cos, sin, g2_l, gb_l,
                                         pos, q_out, self.hq_l)
            if self.fused_gather:
                full = self._attend_and_push(l, q_out, k, v, kw, at.scaling)
            else:
                o, _, _ = tkv_attention_forward(at, q_out, k, v, None, scaling=at.scaling, flash_attn_kwargs=kw)
                dist.all_gather_into_tensor(gathered, o.view(bsz, -1), group=self.group)
                full = gathered.permute(1, 0, 2).reshape(bsz, -1)      # rank-major head blocks = head order
            a = F.linear(full, at.o_proj.weight, at.o_proj.bias)
            ops.add_rmsnorm(x, a, layer.post_attention_layernorm.weight, h, self.eps)
            gu = F.linear(h, w_gu, b_gu)
            act = torch.empty(bsz, w_gu.shape[0] // 2, dtype=x.dtype, device=x.device)
            ops.silu_mul(gu, act)
            delta = F.linear(act, layer.mlp.down_proj.weight, layer.mlp.down_proj.bias)
        ops.add_rmsnorm(x, delta, m.norm.weight, h, self.eps)
        return F.linear(h, self.model.lm_head.weight)
