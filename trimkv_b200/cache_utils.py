"""`TrimKVCache` on the B200 kernels: same surface as the reference class, different storage.

Mirrors ``TrimKVCache`` of the reference (src/trimkv/cache_utils.py:11-223): ``update`` returns the
5-tuple ``(K, V, log beta, positions, flash_attn_kwargs)``, ``compress`` applies the per-head
keep-top-M policy once a layer holds ``M + B`` tokens, and the bookkeeping methods keep their names
and meaning.  Storage differs: after the prompt all layers live in one *capacity-strided flat cache*
(one slab per tensor kind, ``[layers, B*Hkv, cap, ...]``), appended to and compacted in place by the
CUDA kernels, instead of per-layer tensors re-allocated by ``torch.cat``/``gather`` every step.

What a caller sees:
  * ``key_cache[l]`` / ``value_cache[l]``: ``[B, Hkv, n, D]`` views (strided by ``cap``) — same shape as
    the reference's tensors; ``retention_weights[l]`` ``[B, Hkv, n]`` is held in fp32 (the exact upcast
    the reference applies before scoring, :172) and ``kv_positions[l]`` in int32 (``log()`` returns int64).
  * ``flash_attn_kwargs`` carries ``head_lens`` / ``cu_seqlens_k`` (int32, per segment ``b*Hkv + h``) like
    the reference's flat caches (:682-687).
There is no CPU path: tensors must live on a CUDA device.
"""
from __future__ import annotations

import weakref
from typing import Any, Dict, Iterable, List, Optional, Tuple

import torch

from . import ops

__all__ = ["TrimKVCache", "DynamicBudgetTrimKVCache", "BatchedDynamicBudgetTrimKVCache"]

# Longest segment tkv_evict_select / tkv_evict accept (kMaxSelectLen in csrc/tkv_evict.cu).
MAX_ONE_PIECE_PROMPT = 57000


class _LayerViews:
    """List-like accessor (``cache.key_cache[layer]``) that builds views of the slabs on demand."""

    def __init__(self, cache: "TrimKVCache", kind: str):
        # Weak: the cache owns these accessors, and a reference back would make every cache (gigabytes of slabs) wait
        # for the cycle collector instead of being freed when its last user drops it.
        self._ref, self._kind = weakref.ref(cache), kind

    @property
    def _cache(self) -> "TrimKVCache":
        cache = self._ref()
        if cache is None:
            raise ReferenceError("the cache this accessor belongs to no longer exists")
        return cache

    def __len__(self):
        return len(self._cache)

    def __getitem__(self, layer_idx: int) -> torch.Tensor:
        if isinstance(layer_idx, slice):
            return [self[i] for i in range(*layer_idx.indices(len(self)))]
        if layer_idx < 0:
            layer_idx += len(self)
        return self._cache._view(self._kind, layer_idx)

    def __iter__(self):
        for i in range(len(self)):
            yield self[i]


class TrimKVCache:
    def __init__(
        self,
        max_seq_len: int = 20480,
        _distributed_cache_data: Iterable = None,
        device: str = "cuda",
        memory_size: Optional[int] = None,
        buffer_size: Optional[int] = None,
        num_layers: Optional[int] = None,
    ) -> None:
        # Same first three arguments as the reference (cache_utils.py:12-33).  memory_size/buffer_size are
        # optional hints: when given, the slabs are sized M+B at the first decode step even if compress()
        # has not been called yet.
        if _distributed_cache_data is not None:
            raise NotImplementedError("Distributed cache data is not supported for TrimKVCache")
        self.max_seq_len = max_seq_len
        self.device = device
        self._seen_tokens = 0
        self.n_seen_tokens: List[int] = []
        self.offset = torch.tensor(0, dtype=torch.int64)
        self.block_mask = None
        self.sliding_window_size = 0
        self._hint_m, self._hint_b = memory_size, buffer_size
        # With memory_size, buffer_size and num_layers all known up front, each layer's prompt K/V is reduced to its
        # top-M rows as soon as that layer's update() is called (the caller still attends over its own dense tensors),
        # instead of keeping the prompt K/V of every layer alive until compress().  Same survivors either way.
        self._hint_layers = num_layers
        self.defer_handoff = False   # set when compress() will be called with a strategy that needs the keys (knorm_alpha)

        self._pending: List[Optional[Tuple[torch.Tensor, ...]]] = []  # per layer: dense prompt (K, V, beta, pos)
        self._cache_len: List[int] = []                               # per layer: live rows per segment
        self._slab = None  # dict(k, v, beta, pos, len, cu) once materialised
        self._cap = 0
        self._batch = self._hkv = self._dim = None
        self._status = None
        self._evict_ws = None        # scratch of the several-CTAs-per-segment eviction, sized on first use
        self.last_kept_idx: Optional[torch.Tensor] = None  # filled when record_kept is set (tests, log)
        self.record_kept = False
        # When set, K/V views span the whole capacity (shape independent of the live length), which a
        # captured CUDA graph of the decode step needs; lengths are then read from head_lens only.
        self.static_views = False

        self.key_cache = _LayerViews(self, "k")
        self.value_cache = _LayerViews(self, "v")
        self.retention_weights = _LayerViews(self, "beta")
        self.kv_positions = _LayerViews(self, "pos")
        self.head_lens = _LayerViews(self, "len")
        self.cu_seqlens_k = _LayerViews(self, "cu")

    # ------------------------------------------------------------------ container protocol
    def __len__(self):
        return len(self._cache_len)

    def __getitem__(self, layer_idx: int):
        if layer_idx < len(self):
            return (self.key_cache[layer_idx], self.value_cache[layer_idx],
                    self.retention_weights[layer_idx], self.kv_positions[layer_idx])
        raise KeyError(f"Cache only has {len(self)} layers, attempted to access layer with index {layer_idx}")

    def __iter__(self):
        for layer_idx in range(len(self)):
            yield self[layer_idx]

    # ------------------------------------------------------------------ bookkeeping (cache_utils.py:48-60,134-138)
    def get_seq_length(self, layer_idx: Optional[int] = None) -> int:
        if layer_idx is None:
            return self._seen_tokens
        return self.n_seen_tokens[layer_idx] if layer_idx < len(self.n_seen_tokens) else 0

    def get_cache_length(self, layer_idx: int = 0) -> int:
        return self._cache_len[layer_idx] if layer_idx < len(self._cache_len) else 0

    def get_total_cached_tokens(self, num_key_value_heads: Optional[int] = None) -> int:
        if num_key_value_heads is None:
            num_key_value_heads = self._hkv or 0
        return sum(self.get_cache_length(l) * num_key_value_heads for l in range(len(self)))

    # HF generate() probes these on any cache object.
    is_compileable = False
    is_sliding = [False]

    def get_mask_sizes(self, cache_position: torch.Tensor, layer_idx: int = 0) -> Tuple[int, int]:
        return self.get_cache_length(layer_idx) + cache_position.shape[0], 0

    def advance(self, num_tokens: int = 1) -> None:
        """Host-side counters of one ``update`` per layer, for callers that replay a captured CUDA graph
        of the decode step (the kernels bump the device-side lengths themselves)."""
        self._seen_tokens += num_tokens
        for l in range(len(self)):
            self.n_seen_tokens[l] += num_tokens
            self._cache_len[l] += num_tokens

    def snapshot_counters(self):
        """The host-side counters that ``update`` / ``decode_prep`` / ``advance`` move, for ``restore_counters``: a CUDA
        graph capture of a decode step runs the host side of the step without running its kernels."""
        return (self._seen_tokens, list(self.n_seen_tokens), list(self._cache_len))

    def restore_counters(self, snap) -> None:
        self._seen_tokens, self.n_seen_tokens, self._cache_len = snap[0], list(snap[1]), list(snap[2])

    # ------------------------------------------------------------------ views
    def _view(self, kind: str, l: int):
        if l >= len(self):
            raise IndexError(l)
        if self._pending[l] is not None:
            k, v, beta, pos = self._pending[l]
            if kind in ("len", "cu"):
                b, h, s, _ = k.shape
                if kind == "len":
                    return torch.full((b * h,), s, dtype=torch.int32, device=k.device)
                return torch.arange(0, b * h * s + 1, s, dtype=torch.int32, device=k.device)
            return {"k": k, "v": v, "beta": beta, "pos": pos}[kind]
        if self._slab is None:  # skipped layer that never received data (cache_utils.py:82-88)
            return torch.tensor([])
        n, s = self._cache_len[l], self._slab
        if self.static_views:
            n = self._cap
        if kind == "k" or kind == "v":
            return s[kind][l].view(self._batch, self._hkv, self._cap, self._dim)[:, :, :n]
        if kind == "beta" or kind == "pos":
            return s[kind][l].view(self._batch, self._hkv, self._cap)[:, :, :n]
        return s[kind][l]

    # ------------------------------------------------------------------ update (cache_utils.py:62-110)
    def update(
        self,
        key_states: torch.Tensor,
        value_states: torch.Tensor,
        retention_weights: torch.Tensor,
        cache_positions: torch.Tensor,
        layer_idx: int,
        cache_kwargs: Optional[Dict[str, Any]] = None,
    ):
        if key_states is not None:
            bsz, num_heads, seq_len, dim = key_states.shape
            if not key_states.is_cuda:
                raise ops._lib.TrimKVNativeError("TrimKVCache (B200) holds CUDA tensors only; there is no CPU path")
            if layer_idx == 0:
                self._seen_tokens += seq_len
            while len(self._cache_len) <= layer_idx:  # includes skipped layers
                self._pending.append(None)
                self._cache_len.append(0)
                self.n_seen_tokens.append(0)
            if self._cache_len[layer_idx] == 0 and self._eager_handoff(layer_idx):
                if cache_positions.dim() == 1:
                    cache_positions = cache_positions[None, None, :].expand_as(retention_weights)
                self._batch, self._hkv, self._dim = bsz, num_heads, dim
                self._pending[layer_idx] = (key_states, value_states, retention_weights, cache_positions)
                self._cache_len[layer_idx] = seq_len
                self.n_seen_tokens[layer_idx] = seq_len
                self._materialise(only_layer=layer_idx)
                # the prompt pass attends over the caller's dense tensors, exactly as with the deferred hand-off
                return key_states, value_states, retention_weights, cache_positions, {}
            elif self._cache_len[layer_idx] == 0 and self._slab is None:
                # First tokens of this layer: keep the caller's tensors, as the reference does (:90-94).
                if cache_positions.dim() == 1:
                    cache_positions = cache_positions[None, None, :].expand_as(retention_weights)
                self._pending[layer_idx] = (key_states, value_states, retention_weights, cache_positions)
                self._cache_len[layer_idx] = seq_len
                self.n_seen_tokens[layer_idx] = seq_len
                self._batch, self._hkv, self._dim = bsz, num_heads, dim
            else:
                if self._slab is None or self._pending[layer_idx] is not None:
                    self._materialise(extra=seq_len)
                if layer_idx >= self._slab["k"].shape[0]:
                    raise NotImplementedError("a layer that first receives tokens after the prompt hand-off")
                if (bsz, num_heads, dim) != (self._batch, self._hkv, self._dim):
                    raise ValueError("batch size / KV heads / head_dim changed between updates")
                if self._cache_len[layer_idx] + seq_len > self._cap:
                    if torch.cuda.is_current_stream_capturing():
                        raise RuntimeError("cache capacity exhausted during CUDA graph capture")
                    self._grow(self._cache_len[layer_idx] + seq_len)
                s = self._slab
                ops.append(s["k"][layer_idx], s["v"][layer_idx], s["beta"][layer_idx], s["pos"][layer_idx],
                           s["len"][layer_idx], s["cu"][layer_idx], key_states, value_states, retention_weights,
                           cache_positions, self._cap, self._status)
                self._cache_len[layer_idx] += seq_len
                self.n_seen_tokens[layer_idx] += seq_len
        return (self.key_cache[layer_idx], self.value_cache[layer_idx], self.retention_weights[layer_idx],
                self.kv_positions[layer_idx], self._attn_kwargs(layer_idx))

    def decode_prep(self, layer_idx: int, qkvg, q_norm_w, k_norm_w, eps, cos, sin, gate_w2, gate_bias, pos, q_out,
                    num_q_heads: int, in_splits: int = 0, in_bias=None):
        """Fused form of ``update`` for one new token per request: the kernel normalises and rotates q and k,
        finishes the retention gate and appends K, V, log beta and the position in one launch.  Same counter
        updates as ``update``; returns ``(K view, V view, flash_attn_kwargs)``."""
        if self._slab is None or self._pending[layer_idx] is not None:
            self._materialise(extra=1)
        if self._cache_len[layer_idx] + 1 > self._cap:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("cache capacity exhausted during CUDA graph capture")
            self._grow(self._cache_len[layer_idx] + 1)
        if layer_idx == 0:
            self._seen_tokens += 1
        s = self._slab
        ops.decode_prep(qkvg, q_norm_w, k_norm_w, eps, cos, sin, gate_w2, gate_bias, pos, q_out,
                        s["k"][layer_idx], s["v"][layer_idx], s["beta"][layer_idx], s["pos"][layer_idx],
                        s["len"][layer_idx], s["cu"][layer_idx], self._cap, num_q_heads, self._hkv, self._status,
                        in_splits, in_bias)
        self._cache_len[layer_idx] += 1
        self.n_seen_tokens[layer_idx] += 1
        return self.key_cache[layer_idx], self.value_cache[layer_idx], self._attn_kwargs(layer_idx)

    def _eager_handoff(self, layer_idx: int) -> bool:
        return (type(self) is TrimKVCache and not self.defer_handoff and self._hint_m is not None and self._hint_b is not None
                and self._hint_layers is not None and layer_idx < self._hint_layers and not self.sliding_window_size
                and all(p is None for p in self._pending))

    def _attn_kwargs(self, l: int) -> Dict[str, Any]:
        if self._slab is None or self._pending[l] is not None:
            return {}
        return {"head_lens": self._slab["len"][l], "cu_seqlens_k": self._slab["cu"][l],
                "batch_size": self._batch, "num_kv_heads": self._hkv, "status": self._status,
                "uniform_lengths": True}   # every segment of a layer has the same length in this class

    # ------------------------------------------------------------------ storage
    def _alloc(self, cap: int):
        dev, nseg = self._any_pending_or_slab_device(), self._batch * self._hkv
        nl = max(len(self), self._hint_layers or 0)
        dt = self._kv_dtype
        slab = {
            "k": torch.empty(nl, nseg * cap, self._dim, dtype=dt, device=dev),
            "v": torch.empty(nl, nseg * cap, self._dim, dtype=dt, device=dev),
            "beta": torch.empty(nl, nseg * cap, dtype=torch.float32, device=dev),
            "pos": torch.empty(nl, nseg * cap, dtype=torch.int32, device=dev),
            "len": torch.zeros(nl, nseg, dtype=torch.int32, device=dev),
            "cu": torch.zeros(nl, nseg + 1, dtype=torch.int32, device=dev),
        }
        return slab

    def _any_pending_or_slab_device(self):
        if self._slab is not None:
            return self._slab["k"].device
        return next(p[0].device for p in self._pending if p is not None)

    def _materialise(self, extra: int = 0, memory_size: Optional[int] = None, buffer_size: Optional[int] = None,
                     only_layer: Optional[int] = None):
        """Moves the dense prompt tensors of every layer (or of ``only_layer``) into the slabs (the prefill hand-off)."""
        pend = [p for p in self._pending if p is not None]
        if not pend:
            return
        # Rows are only evicted here when compress() asked for it (or in the per-layer hand-off, which stands for it);
        # the constructor hints alone just size the slabs.
        do_select = memory_size is not None or only_layer is not None
        m = memory_size if memory_size is not None else self._hint_m
        bsz = buffer_size if buffer_size is not None else self._hint_b
        self._kv_dtype = pend[0][0].dtype
        dev = pend[0][0].device
        if self._status is None:
            self._status = ops.new_status(dev)
        longest = max(self._cache_len)
        if m is not None and bsz is not None:
            kept_longest = max((m if (do_select and n >= m + bsz) else n) for n in self._cache_len)
            cap = max(m + bsz, kept_longest + extra)
        else:
            cap = (longest + extra + 63) // 64 * 64 if extra >= 64 else 1 << max(8, (longest + extra + 255).bit_length())
        first = self._slab is None
        if first:
            self._cap = cap
            self._slab = self._alloc(cap)
        nseg = self._batch * self._hkv
        s = self._slab
        kept_all = []
        for l, p in enumerate(self._pending):
            if p is None:
                continue
            k, v, beta, pos = p
            n = k.shape[2]
            beta32 = beta.to(torch.float32).reshape(nseg, n).contiguous()
            pos32 = pos.to(torch.int32).reshape(nseg, n).contiguous()
            kept_idx = kept_cnt = None
            if do_select and m is not None and bsz is not None and n >= m + bsz:
                if n > MAX_ONE_PIECE_PROMPT:
                    raise ValueError(
                        f"a prompt of {n} tokens cannot be reduced to memory_size in one piece (the selection kernel "
                        f"holds one score per token in shared memory, at most {MAX_ONE_PIECE_PROMPT}); feed it in pieces: "
                        "model.generate(..., prefill_chunk_size=N) or several forward calls of at most that many tokens")
                kept_idx = torch.empty(nseg, m, dtype=torch.int32, device=dev)
                kept_cnt = torch.empty(nseg, dtype=torch.int32, device=dev)
                ops.evict_select(beta32, pos32, None, n, nseg, self.n_seen_tokens[l] + 1, m, m + bsz, n,
                                 kept_idx, kept_cnt, self._status)
                self._cache_len[l] = m
                if self.record_kept:
                    kept_all.append(kept_idx.view(self._batch, self._hkv, m))
            ops.compact(s["k"][l], s["v"][l], s["beta"][l], s["pos"][l], self._cap, k, v, beta32, pos32,
                        kept_idx, kept_cnt, s["len"][l], s["cu"][l], nseg, self._status)
            self._pending[l] = None
        if kept_all:
            self.last_kept_idx = torch.stack(kept_all)  # [layers, B, Hkv, M]

    def _grow(self, need: int):
        """Re-homes every layer in slabs of at least ``need`` rows per segment (rare: no eviction or a large chunk)."""
        self._rehome(max(need, 2 * self._cap))

    def _rehome(self, new_cap: int):
        old, old_cap = self._slab, self._cap
        self._slab, self._cap = self._alloc(new_cap), new_cap
        nseg = self._batch * self._hkv
        for l in range(len(self)):
            n = min(self._cache_len[l], new_cap)
            if n == 0:
                continue
            k = old["k"][l].view(self._batch, self._hkv, old_cap, self._dim)[:, :, :n]
            v = old["v"][l].view(self._batch, self._hkv, old_cap, self._dim)[:, :, :n]
            ops.compact(self._slab["k"][l], self._slab["v"][l], self._slab["beta"][l], self._slab["pos"][l], new_cap,
                        k, v, old["beta"][l].view(nseg, old_cap), old["pos"][l].view(nseg, old_cap),
                        None, old["len"][l], self._slab["len"][l], self._slab["cu"][l], nseg, self._status)

    # ------------------------------------------------------------------ compress (cache_utils.py:140-198)
    def compress(
        self,
        strategy: str = "alpha",
        memory_size: int = 2048,
        buffer_size: int = 512,
        floor_budget_ratio: float = 0.0,   # accepted and unused, as in the reference (:145-146)
        alpha_threshold: float = 0.0,
        num_layers: Optional[int] = None,
        num_key_value_heads: Optional[int] = None,
        skip_layers: int = 0,
    ):
        if strategy not in ("alpha", "knorm_alpha"):
            raise ValueError(f"Unknown compression strategy: {strategy}")
        knorm = strategy == "knorm_alpha"
        if (knorm and type(self) is TrimKVCache and not self.defer_handoff and self._hint_m is not None
                and self._hint_b is not None and self._hint_layers is not None and not self.sliding_window_size):
            # With these constructor hints update() has already reduced each layer's prompt to its top rows, by the
            # "alpha" score: the key norms would come too late.
            raise ValueError("memory_size / buffer_size / num_layers given to the constructor select the prompt's rows with "
                             "strategy 'alpha' inside update(); leave them out (or set defer_handoff) to compress with "
                             "'knorm_alpha'")
        num_layers = len(self) if num_layers is None else num_layers
        if num_layers == 0:
            return
        if any(p is not None for p in self._pending):
            if skip_layers:
                raise NotImplementedError("skip_layers with a pending prompt")
            if not self.sliding_window_size and not knorm:
                self._materialise(memory_size=memory_size, buffer_size=buffer_size)
                return
            # A protected tail and the key norms are only known to the in-place kernel: home the whole prompt, then
            # evict below.
            self._hint_m = self._hint_b = None
            self._materialise(extra=max(64, buffer_size))
        w = int(self.sliding_window_size)
        if w >= memory_size and w > 0:
            raise ValueError("sliding_window_size must be smaller than memory_size")
        trigger = memory_size + buffer_size
        fire = [l for l in range(skip_layers, num_layers) if trigger <= self._cache_len[l]]
        if not fire:
            return
        s, nseg = self._slab, self._batch * self._hkv
        all_same = (len(fire) == len(self) and len({self.n_seen_tokens[l] for l in fire}) == 1
                    and len({self._cache_len[l] for l in fire}) == 1)
        kept = None
        if all_same:
            # Every layer fires in the same forward (same lengths): one launch over the whole slab.
            nl, n = len(self), self._cache_len[0]
            if self.record_kept:
                kept = torch.empty(nl * nseg, memory_size, dtype=torch.int32, device=s["k"].device)
            self._evict(s["k"], s["v"], s["beta"], s["pos"], s["len"], s["cu"], nseg, nl * nseg,
                        self.n_seen_tokens[0] + 1, n, w, memory_size, trigger, kept, knorm)
            if kept is not None:
                self.last_kept_idx = kept.view(nl, self._batch, self._hkv, memory_size)
        else:
            for l in fire:
                if self.record_kept:
                    kept = torch.empty(nseg, memory_size, dtype=torch.int32, device=s["k"].device)
                self._evict(s["k"][l], s["v"][l], s["beta"][l], s["pos"][l], s["len"][l], s["cu"][l], nseg, nseg,
                            self.n_seen_tokens[l] + 1, self._cache_len[l], w, memory_size, trigger, kept, knorm)
                if kept is not None:
                    self.last_kept_idx = kept.view(self._batch, self._hkv, memory_size)
        for l in fire:
            self._cache_len[l] = memory_size

    def _evict(self, k, v, beta, pos, ln, cu, group, nseg, q_idx, n, w, memory_size, trigger, kept, knorm):
        """One eviction launch over ``nseg`` segments of length ``n``.  With few segments (one layer of a small batch)
        the rows of each segment are shared by several CTAs so that more of the GPU moves them; measured on B200 this
        pays up to about 64 segments, beyond that one CTA per segment is as fast or faster."""
        ctas = min(32, 1024 // nseg) if 0 < nseg <= 64 else 1
        row_pair = 2 * k.shape[-1] * k.element_size() + 8
        if ctas >= 2 and 0 < n - memory_size and (n - memory_size) * row_pair <= 200 * 1024:
            need = (nseg, memory_size, ctas)
            if self._evict_ws is None or self._evict_ws[0] != need:
                self._evict_ws = (need, ops.evict_multi_workspace(nseg, memory_size, ctas, k.device))
            ops.evict_multi(k, v, beta, pos, ln, cu, group, nseg, self._cap, q_idx, memory_size, trigger, n, ctas,
                            self._evict_ws[1], protect_last=w, knorm=knorm, kept_idx_out=kept, status=self._status)
        else:
            ops.evict_ex(k, v, beta, pos, ln, cu, group, nseg, self._cap, q_idx, n, None, w, memory_size, trigger,
                         kept, 0, self._status, knorm)

    # ------------------------------------------------------------------ misc API (cache_utils.py:112-132,200-223)
    def check_status(self) -> None:
        """Synchronises and raises if a kernel reported a device-side problem."""
        if self._status is not None:
            code = ops.read_status(self._status)
            if code:
                names = {1: "segment capacity exceeded", 2: "segment longer than the stated bound", 3: "bad kept index"}
                raise ops._lib.TrimKVNativeError(f"device status {code}: {names.get(code, 'unknown')}")

    def log(self, layer_idx: int = None):
        logs = {}
        if layer_idx is None:
            for l in range(len(self)):
                logs[l] = {"seen_tokens": self.get_seq_length(l),
                           "kv_positions": self.kv_positions[l].detach().to(torch.int64).cpu()}
        else:
            logs["seen_tokens"] = self.get_seq_length(layer_idx)
            logs["kv_positions"] = self.kv_positions[layer_idx].detach().to(torch.int64).cpu()
        return logs

    def _clone_from_dense(self, layers, device=None) -> "TrimKVCache":
        new = TrimKVCache(max_seq_len=self.max_seq_len, device=device or self.device,
                          memory_size=self._hint_m, buffer_size=self._hint_b)
        new._seen_tokens = self._seen_tokens
        for l, (k, v, b, p) in enumerate(layers):
            new._pending.append((k, v, b, p))
            new._cache_len.append(k.shape[2])
            new.n_seen_tokens.append(self.n_seen_tokens[l])
            new._batch, new._hkv, new._dim = k.shape[0], k.shape[1], k.shape[3]
        return new

    def head_shard(self, rank: int, world_size: int) -> "TrimKVCache":
        """A cache holding only KV heads ``[rank*Hkv/world, (rank+1)*Hkv/world)`` of every layer and request: the
        per-rank cache of the KV-head-sharded decode (segments are independent, so nothing else changes)."""
        if self._hkv % world_size:
            raise ValueError(f"{self._hkv} KV heads cannot be split over {world_size} ranks")
        hl = self._hkv // world_size
        lo, hi = rank * hl, (rank + 1) * hl
        n = None
        dense = []
        for l, (k, v, b, p) in enumerate(self):
            n = self._cache_len[l]
            dense.append((k[:, lo:hi, :n].contiguous(), v[:, lo:hi, :n].contiguous(), b[:, lo:hi, :n].contiguous(),
                          p[:, lo:hi, :n].contiguous()))
        return self._clone_from_dense(dense)

    def batch_select_indices(self, indices: torch.Tensor):
        dense = [(k[indices, ...].contiguous(), v[indices, ...].contiguous(), b[indices, ...].contiguous(),
                  p[indices, ...].contiguous()) for (k, v, b, p) in self]
        other = self._clone_from_dense(dense)
        self.__dict__.update({k: v for k, v in other.__dict__.items()
                              if k not in ("key_cache", "value_cache", "retention_weights", "kv_positions",
                                           "head_lens", "cu_seqlens_k")})

    def batch_split(self, full_batch_size: int, split_size: int) -> List["TrimKVCache"]:
        out = []
        for i in range(0, full_batch_size, split_size):
            dense = [(k[i:i + split_size].contiguous(), v[i:i + split_size].contiguous(),
                      b[i:i + split_size].contiguous(), p[i:i + split_size].contiguous()) for (k, v, b, p) in self]
            out.append(self._clone_from_dense(dense))
        return out

    def copy_to_device(self, device: str) -> "TrimKVCache":
        dense = [(k.to(device).contiguous(), v.to(device).contiguous(), b.to(device).contiguous(),
                  p.to(device).contiguous()) for (k, v, b, p) in self]
        return self._clone_from_dense(dense, device=device)


class BatchedDynamicBudgetTrimKVCache(TrimKVCache):
    """Flat varlen cache whose token budget is shared between heads (and optionally layers) of a request.

    Mirrors ``BatchedDynamicBudgetTrimKVCache`` of the reference (src/trimkv/cache_utils.py:563-971): segments are
    ordered ``b*Hkv + h``; ``update`` returns ``flash_attn_kwargs`` with ``head_lens`` / ``cu_seqlens_k`` /
    ``batch_size`` / ``num_kv_heads`` (:682-687); ``compress`` implements ``alpha``, ``layer_wise_alpha``,
    ``alpha_threshold`` with ``floor_budget_ratio`` exactly as :697-945 decide which rows survive.  The rows stay
    in the capacity-strided slabs: the top-k over a request's concatenated scores becomes a keep count per segment
    (``tkv_group_budget``) followed by the in-place per-segment eviction (``tkv_evict_ex``).  Scores are computed in
    the dtype log beta arrives in, as the reference does (:755; bf16 models score in bf16).  Differences: log beta is
    held as fp32 (exact), ties go to the lower concatenated index, and
    K/V are handed out as strided ``[B, Hkv, n_max, D]`` views (``packed(layer)`` builds the reference's
    ``[sum n, D]`` tensors on demand).
    """

    _batched = True

    def __init__(self, max_seq_len: int = 20480, _distributed_cache_data: Iterable = None, device: str = "cuda") -> None:
        if _distributed_cache_data is not None:
            raise NotImplementedError("Distributed cache data is not supported for " + type(self).__name__)
        super().__init__(max_seq_len=max_seq_len, device=device)
        self._rows: List[int] = []   # per layer: total live rows (host copy, refreshed after every eviction)
        self._beta_dtype = torch.float32  # dtype log beta arrives in: the dtype the reference scores in
        self._knorm = False               # set by compress() for the "knorm_*" strategies
        self.batch_size: Optional[int] = None
        self.num_kv_heads: Optional[int] = None

    # ---- update ---------------------------------------------------------------------------------------
    def update(self, key_states, value_states, retention_weights, cache_positions, layer_idx, cache_kwargs=None):
        if key_states is not None:
            bsz, h, s, _ = key_states.shape
            if not self._batched:
                assert bsz == 1, "Batch size greater than 1 is not supported for DynamicBudgetTrimKVCache"
            if self.batch_size is None:
                self.batch_size, self.num_kv_heads = bsz, h
            else:
                assert bsz == self.batch_size, f"Batch size changed: {self.batch_size} -> {bsz}"
                assert h == self.num_kv_heads, f"Num KV heads changed: {self.num_kv_heads} -> {h}"
            self._beta_dtype = retention_weights.dtype
            while len(self._rows) <= layer_idx:
                self._rows.append(0)
            self._rows[layer_idx] += bsz * h * s
        out = super().update(key_states, value_states, retention_weights, cache_positions, layer_idx, cache_kwargs)
        return out

    def decode_prep(self, layer_idx: int, *args, **kwargs):
        # One new row per segment: keep the host-side row total in step (compress() triggers on it and the attention
        # grid is sized by it) before the kwargs of this step are built.
        while len(self._rows) <= layer_idx:
            self._rows.append(0)
        self._rows[layer_idx] += self._batch * self._hkv
        return super().decode_prep(layer_idx, *args, **kwargs)

    def advance(self, num_tokens: int = 1) -> None:
        super().advance(num_tokens)
        for l in range(len(self._rows)):
            self._rows[l] += self._batch * self._hkv * num_tokens

    def snapshot_counters(self):
        return super().snapshot_counters() + (list(self._rows),)

    def restore_counters(self, snap) -> None:
        super().restore_counters(snap)
        self._rows = list(snap[3])     # compress() triggers on these totals: a captured, unexecuted step must not count

    def _attn_kwargs(self, l: int) -> Dict[str, Any]:
        kw = super()._attn_kwargs(l)
        if kw:
            kw = dict(kw, batch_size=self._batch, num_kv_heads=self._hkv, uniform_lengths=False)
            if l < len(self._rows) and not self.static_views:
                # Head lengths differ under a shared budget; their sum is known here without a device read, which
                # lets the attention size its grid by tokens instead of by the longest head.  (Not for views of the
                # whole capacity: a captured step is replayed with growing lengths, which a captured total would
                # under-state.)
                kw["total_len_bound"] = self._rows[l]
        return kw

    # ---- bookkeeping ----------------------------------------------------------------------------------
    def get_total_cached_tokens(self, num_key_value_heads: Optional[int] = None) -> int:
        return sum(self._rows)

    def get_cache_length(self, layer_idx: int = 0, batch_idx: int = 0, head_idx: int = 0) -> int:
        if layer_idx >= len(self):
            return 0
        if self._pending[layer_idx] is not None or self._slab is None:
            return self._cache_len[layer_idx]
        return int(self._slab["len"][layer_idx][batch_idx * self._hkv + head_idx].item())

    def packed(self, layer_idx: int):
        """``(K [sum n, D], V, log beta [sum n, 1], positions [sum n, 1])`` in the reference's packed order."""
        k, v, b, p = self[layer_idx]
        if self._pending[layer_idx] is not None:
            d = k.shape[-1]
            return k.reshape(-1, d), v.reshape(-1, d), b.reshape(-1, 1), p.reshape(-1, 1)
        lens = self._slab["len"][layer_idx].view(self._batch, self._hkv, 1)
        mask = torch.arange(k.shape[2], device=k.device).view(1, 1, -1) < lens
        return k[mask], v[mask], b[mask].unsqueeze(-1), p[mask].unsqueeze(-1)

    def log(self):
        pos = []
        for l in range(len(self)):
            p = self.kv_positions[l].to(torch.int64).cpu()
            lens = self.head_lens[l].cpu().view(self._batch, self._hkv)
            for b in range(self._batch):
                for h in range(self._hkv):
                    pos.append(p[b, h, : int(lens[b, h])])
        return {"batch_size": self._batch, "num_kv_heads": self._hkv, "head_wise_kv_positions": pos,
                "flat_head_lens": torch.cat([self.head_lens[l].view(-1) for l in range(len(self))]).cpu().numpy()}

    def copy_to_device(self, device):
        raise NotImplementedError("copy_to_device not implemented for " + type(self).__name__)

    # ---- compress -------------------------------------------------------------------------------------
    def _after_eviction(self, memory_hint: int):
        """One read-back per eviction: true per-layer maxima and totals; shrinks over-sized slabs."""
        lens = self._slab["len"].to(torch.int64)
        mx = lens.max(dim=1).values.cpu().tolist()
        tot = lens.sum(dim=1).cpu().tolist()
        for l in range(len(self)):
            self._cache_len[l], self._rows[l] = int(mx[l]), int(tot[l])
        want = max(self._cache_len) + memory_hint
        if self._cap > 2 * want and not torch.cuda.is_current_stream_capturing():
            self._rehome(want)

    def _budget_and_evict(self, layers, groups_per_layer, inner, n_outer, k_total, threshold, floor_mode, floor_cnt,
                          buffer_size):
        s, nseg, nl = self._slab, self._batch * self._hkv, len(self)
        q_idx = self.get_seq_length() + 1
        # The reference multiplies (q_idx - pos) * log beta in the dtype log beta arrived in (src/trimkv/cache_utils.py:
        # 386, 441, 755, 882) and compares with a threshold of that dtype (:462, :893).
        sd = {torch.bfloat16: 1, torch.float16: 2}.get(self._beta_dtype, 0)
        if threshold is not None and sd:
            threshold = float(torch.tensor(threshold, dtype=torch.float32).to(self._beta_dtype))
        scores = None
        if self._knorm:
            # log_alpha + log ||k||: written once for all rows, so that the budget kernel's five passes and the
            # eviction read 4 bytes per row instead of the K rows.
            scores = torch.empty(nl, nseg * self._cap, dtype=torch.float32, device=s["k"].device)
            ops.flat_scores(s["k"], s["beta"], s["pos"], s["len"], nl * nseg, self._cap, q_idx, max(self._cache_len),
                            scores, knorm=True, score_dtype=sd)
        keep = torch.empty(nl, nseg, dtype=torch.int32, device=s["k"].device)
        keep.copy_(s["len"])  # layers that do not fire keep everything
        if n_outer > 1:       # one group per request spans all layers
            ops.group_budget(s["beta"], s["pos"], s["len"], self._cap, groups_per_layer, inner, n_outer, nseg, q_idx,
                             k_total, keep, threshold, floor_mode, floor_cnt, self._status, sd, scores)
        else:
            for l in layers:
                ops.group_budget(s["beta"][l], s["pos"][l], s["len"][l], self._cap, groups_per_layer, inner, 1, nseg,
                                 q_idx, k_total, keep[l], threshold, floor_mode, floor_cnt, self._status, sd,
                                 None if scores is None else scores[l])
        kept = None
        if self.record_kept:
            kept = torch.full((nl * nseg, self._cap), -1, dtype=torch.int32, device=s["k"].device)
        ops.evict_ex(s["k"], s["v"], s["beta"], s["pos"], s["len"], s["cu"], nseg, nl * nseg, self._cap, q_idx,
                     max(self._cache_len), keep, 0, kept_idx_out=kept, kept_stride=self._cap, status=self._status,
                     score_dtype=sd, scores=scores)
        if kept is not None:
            self.last_kept_idx = kept.view(nl, self._batch, self._hkv, self._cap)
        self._after_eviction(buffer_size)

    def compress(self, strategy: str = "alpha", memory_size: int = 2048, buffer_size: int = 512,
                 floor_budget_ratio: float = 0.0, alpha_threshold: float = 0.0, num_layers: Optional[int] = None,
                 num_key_value_heads: Optional[int] = None, skip_layers: int = 0):
        base = strategy.replace("layer_wise_", "")
        if base not in ("alpha", "alpha_threshold", "knorm_alpha", "knorm_alpha_threshold") or \
                ("layer_wise" in strategy and "threshold" in base):
            raise ValueError(f"Unknown compression strategy: {strategy}")
        self._knorm = base.startswith("knorm")
        L = len(self) if num_layers is None else num_layers
        if L == 0 or self.batch_size is None:
            return
        if L != len(self):
            raise NotImplementedError("compress over a subset of the layers")
        B, H, M, Bf = self._batch, self._hkv, memory_size, buffer_size
        thr = "threshold" in strategy
        total = sum(self._rows)
        import math
        log_thr = (math.log(alpha_threshold) if alpha_threshold > 0 else float("-inf")) if thr else None
        if self._batched:
            # src/trimkv/cache_utils.py:714-738
            if total <= B * H * (M + Bf) * L and not thr:
                return
            if "layer_wise" in strategy:
                fire = [l for l in range(L) if self._rows[l] > B * H * (M + Bf)]
                if not fire:
                    return
                self._ensure_slab()
                k = M * H if floor_budget_ratio <= 0 else int(M * H * (1 - floor_budget_ratio))
                self._budget_and_evict(fire, B, H, 1, k, None, 2 if floor_budget_ratio > 0 else 0,
                                       int(M * floor_budget_ratio), Bf)
            else:
                if total // B <= L * H * (M + Bf) and not thr:
                    return
                self._ensure_slab()
                self._budget_and_evict(range(L), B, H, L, L * H * M, log_thr, 0, 0, Bf)
        else:
            # src/trimkv/cache_utils.py:346-369, 418-536 (batch size 1)
            if "layer_wise" in strategy:
                fire = [l for l in range(L) if H * (M + Bf) < self._rows[l]]
                if not fire:
                    return
                self._ensure_slab()
                self._budget_and_evict(fire, 1, H, 1, H * M, None, 0, 0, Bf)
            else:
                if L * H * (M + Bf) > total and not thr:
                    return
                self._ensure_slab()
                if floor_budget_ratio == 0:
                    self._budget_and_evict(range(L), 1, H, L, L * H * M, log_thr, 0, 0, Bf)
                else:
                    assert not thr, "Thresholding strategy is not compatible with floor_budget_ratio > 0"
                    self._budget_and_evict(range(L), 1, H, L, int(L * H * M * (1 - floor_budget_ratio)), None, 1,
                                           int(M * floor_budget_ratio), Bf)

    def _ensure_slab(self):
        """Moves a pending prompt into the slabs without evicting (the shared budget is applied afterwards)."""
        if any(p is not None for p in self._pending):
            self._hint_m = self._hint_b = None
            self._materialise(extra=64)


class DynamicBudgetTrimKVCache(BatchedDynamicBudgetTrimKVCache):
    """Batch-size-1 flat cache with a budget shared across heads / layers.

    Mirrors ``DynamicBudgetTrimKVCache`` (src/trimkv/cache_utils.py:226-560): same storage and kernels as the batched
    class, with the reference's batch-1 trigger rules and its per-head floor arithmetic (:486-536).
    """

    _batched = False

    def get_cache_length(self, layer_idx: int = 0, head_idx: int = 0) -> int:
        return super().get_cache_length(layer_idx, 0, head_idx)
