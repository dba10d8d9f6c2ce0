"""CPU restatement of the TRIM-KV cache hot path (numpy).  TEST INFRASTRUCTURE ONLY.

This module is the checker the CUDA path is compared against.  Nothing in the
product package imports it; only the tests, the smoke check and the
``cpu_baseline`` / ``--impl reference`` legs of the benchmark do.

Every function restates one piece of the reference (yejun-yun/trimkv) and
cites the file:line it follows.  Pinning: the functions here are compared
against the reference's own Python, imported on CPU, by
``tests/golden/make_golden.py``; the resulting vectors are committed under
``tests/golden/`` and re-checked by ``tests/test_oracle.py``.  The attention
arithmetic of the reference lives in the third-party flash-attn wheel
(flash_attn==2.7.2.post1, call sites src/trimkv/attn/flash_attn.py:61-71 and
:135-145); no reference test pins results there, so for attention the oracle
restates the published softmax(q K^T / sqrt(D)) V per segment following
src/trimkv/attn/eager_attn.py:48-73 and is pinned against that eager function.

Tie rule.  The reference keeps ``torch.topk(scores, M)`` whose order among
equal scores is unspecified.  The canonical rule used here (and by the CUDA
kernels) is: larger score first; among equal scores the lower index (= lower
position, positions are ascending inside a segment) wins; -0.0 == +0.0; NaN
ranks above +inf (torch.topk treats NaN as the largest value).
"""
from __future__ import annotations

import numpy as np

__all__ = [
    "retention_scores",
    "round_to_dtype",
    "canonical_topm",
    "compress_rows",
    "OracleTrimKVCache",
    "flat_append",
    "OracleBatchedFlatCache",
    "varlen_gqa_attention",
    "dense_gqa_attention",
]


# --------------------------------------------------------------------------
# eviction arithmetic
# --------------------------------------------------------------------------
def round_to_dtype(x: np.ndarray, dtype: str) -> np.ndarray:
    """fp32 values rounded (nearest even) to ``dtype`` ("float32", "bfloat16", "float16"), returned as fp32."""
    x = np.asarray(x, dtype=np.float32)
    if dtype == "float32":
        return x
    if dtype == "float16":
        with np.errstate(over="ignore"):
            return x.astype(np.float16).astype(np.float32)
    if dtype != "bfloat16":
        raise ValueError(dtype)
    u = x.view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32).view(np.float32)
    return np.where(np.isfinite(x), r, x).astype(np.float32)


def retention_scores(log_beta: np.ndarray, kv_positions: np.ndarray, q_idx: int, score_dtype: str = "float32") -> np.ndarray:
    """fp32 score = fp32(log beta) * fp32(q_idx - pos), one rounding.

    src/trimkv/cache_utils.py:172-174: ``log_beta = rw.to(float32)``;
    ``q_idx = seen + 1``; ``log_alpha = log_beta * (q_idx - kv_positions)``.
    torch promotes the int64 age to fp32 and multiplies once.

    ``score_dtype`` other than fp32 restates the flat classes, which skip the upcast (:386, :441, :755, :882:
    ``(q_idx - kv_pos) * rw`` with ``rw`` in the model dtype): torch casts the int64 age to that dtype, multiplies in
    fp32 and rounds the product to it.  ``log_beta`` must then hold values representable in that dtype.
    """
    lb = np.asarray(log_beta).astype(np.float32)
    age = (np.int64(q_idx) - np.asarray(kv_positions).astype(np.int64)).astype(np.float32)
    if score_dtype != "float32":
        return round_to_dtype(lb * round_to_dtype(age, score_dtype), score_dtype)
    return (lb * age).astype(np.float32)


def canonical_topm(scores: np.ndarray, m: int) -> np.ndarray:
    """Indices of the ``m`` largest scores along the last axis, ascending.

    src/trimkv/cache_utils.py:190-192 (``topk`` then ``sort`` of the indices)
    with the canonical tie rule of this module's docstring.
    """
    s = np.asarray(scores, dtype=np.float32)
    n = s.shape[-1]
    if m > n:
        raise ValueError(f"cannot keep {m} of {n}")
    flat = s.reshape(-1, n)
    nan = np.isnan(flat)
    clean = np.where(nan, np.float32(0), flat) + np.float32(0)  # -0.0 -> +0.0
    idx = np.broadcast_to(np.arange(n), flat.shape)
    # lexsort: the last key is the primary one.
    order = np.lexsort((idx, -clean.astype(np.float64), ~nan), axis=-1)
    out = np.sort(order[:, :m], axis=-1).astype(np.int64)
    return out.reshape(s.shape[:-1] + (m,))


def compress_rows(key, value, log_beta, kv_positions, q_idx: int, m: int, sliding_window_size: int = 0,
                  strategy: str = "alpha", score_dtype: str = "float32"):
    """One ``compress_layer`` on dense ``[..., n, D]`` / ``[..., n]`` arrays.

    src/trimkv/cache_utils.py:167-198, strategy "alpha"; the newest ``sliding_window_size`` rows score +inf (:186-187).
    Returns (key, value, log_beta, kv_positions, kept_idx).
    """
    sc = retention_scores(log_beta, kv_positions, q_idx, score_dtype)
    if strategy == "knorm_alpha":
        # :176-180: scores = log_alpha + log(||k||_2); fp32 keys only here (16-bit keys round norm and log to that dtype)
        kn = np.sqrt(np.sum(np.asarray(key, np.float32) ** 2, axis=-1, dtype=np.float32))
        sc = (sc + np.log(kn).astype(np.float32)).astype(np.float32)
    elif strategy != "alpha":
        raise ValueError(f"Unknown compression strategy: {strategy}")
    if sliding_window_size > 0:
        sc = sc.copy()
        sc[..., -sliding_window_size:] = np.inf
    keep = canonical_topm(sc, m)
    k2 = np.take_along_axis(key, keep[..., None], axis=-2)
    v2 = np.take_along_axis(value, keep[..., None], axis=-2)
    b2 = np.take_along_axis(log_beta, keep, axis=-1)
    p2 = np.take_along_axis(kv_positions, keep, axis=-1)
    return k2, v2, b2, p2, keep


class OracleTrimKVCache:
    """Dense per-layer cache, restating ``TrimKVCache``.

    src/trimkv/cache_utils.py:11-223.  Arrays per layer: key/value
    ``[B,H,n,D]``, retention_weights (log beta) ``[B,H,n]``, kv_positions
    ``[B,H,n]`` int64, ``n_seen_tokens`` per layer.
    """

    def __init__(self):
        self._seen_tokens = 0
        self.key_cache = []
        self.value_cache = []
        self.retention_weights = []
        self.kv_positions = []
        self.n_seen_tokens = []
        self.last_kept = {}
        self.sliding_window_size = 0

    def __len__(self):
        return len(self.key_cache)

    def get_seq_length(self, layer_idx=None):
        # cache_utils.py:48-54
        if layer_idx is None:
            return self._seen_tokens
        return self.n_seen_tokens[layer_idx] if layer_idx < len(self.n_seen_tokens) else 0

    def get_cache_length(self, layer_idx=0):
        # cache_utils.py:134-138
        if layer_idx >= len(self.key_cache):
            return 0
        return self.key_cache[layer_idx].shape[-2]

    def update(self, key_states, value_states, retention_weights, cache_positions, layer_idx):
        # cache_utils.py:62-110
        s = key_states.shape[-2]
        if layer_idx == 0:
            self._seen_tokens += s
        pos = np.asarray(cache_positions, dtype=np.int64)
        if pos.ndim == 1:
            pos = np.broadcast_to(pos[None, None, :], retention_weights.shape)
        if len(self.key_cache) <= layer_idx:
            while len(self.key_cache) < layer_idx:  # skipped layers
                self.key_cache.append(np.zeros((0,)))
                self.value_cache.append(np.zeros((0,)))
                self.retention_weights.append(np.zeros((0,)))
                self.kv_positions.append(np.zeros((0,), dtype=np.int64))
                self.n_seen_tokens.append(0)
            self.key_cache.append(np.array(key_states))
            self.value_cache.append(np.array(value_states))
            self.retention_weights.append(np.array(retention_weights))
            self.kv_positions.append(np.array(pos))
            self.n_seen_tokens.append(s)
        elif self.key_cache[layer_idx].size == 0:
            self.key_cache[layer_idx] = np.array(key_states)
            self.value_cache[layer_idx] = np.array(value_states)
            self.retention_weights[layer_idx] = np.array(retention_weights)
            self.kv_positions[layer_idx] = np.array(pos)
            self.n_seen_tokens[layer_idx] = s
        else:
            self.key_cache[layer_idx] = np.concatenate([self.key_cache[layer_idx], key_states], axis=-2)
            self.value_cache[layer_idx] = np.concatenate([self.value_cache[layer_idx], value_states], axis=-2)
            self.retention_weights[layer_idx] = np.concatenate(
                [self.retention_weights[layer_idx], retention_weights], axis=-1)
            self.kv_positions[layer_idx] = np.concatenate([self.kv_positions[layer_idx], pos], axis=-1)
            self.n_seen_tokens[layer_idx] += s
        return (self.key_cache[layer_idx], self.value_cache[layer_idx],
                self.retention_weights[layer_idx], self.kv_positions[layer_idx], {})

    def compress(self, strategy="alpha", memory_size=2048, buffer_size=512, skip_layers=0, **_ignored):
        # cache_utils.py:140-158: trigger is evaluated per layer, after the forward.
        if strategy not in ("alpha", "knorm_alpha"):
            raise ValueError(f"Unknown compression strategy: {strategy}")
        for layer_idx in range(skip_layers, len(self.key_cache)):
            if memory_size + buffer_size <= self.get_cache_length(layer_idx):
                self.compress_layer(layer_idx, memory_size, strategy)

    def compress_layer(self, layer_idx, memory_size, strategy="alpha"):
        # cache_utils.py:160-198
        q_idx = self.get_seq_length(layer_idx) + 1
        k, v, b, p, keep = compress_rows(
            self.key_cache[layer_idx], self.value_cache[layer_idx],
            self.retention_weights[layer_idx], self.kv_positions[layer_idx], q_idx, memory_size,
            self.sliding_window_size, strategy)
        self.key_cache[layer_idx] = k
        self.value_cache[layer_idx] = v
        self.retention_weights[layer_idx] = b
        self.kv_positions[layer_idx] = p
        self.last_kept[layer_idx] = keep


# --------------------------------------------------------------------------
# flat (varlen) layout
# --------------------------------------------------------------------------
def flat_append(cache: np.ndarray, state: np.ndarray, headlens: np.ndarray, cu_headlens: np.ndarray) -> np.ndarray:
    """Functional flat append: ``[sum n_h, D]`` + ``[1,H,S,D]`` -> ``[sum n_h + H*S, D]``.

    src/trimkv/triton/db_cache_utils.py:86-186: segment h of the output starts at
    ``cu[h] + h*S``; its old rows come first (:6-38), its S new rows follow (:41-83).
    """
    _, h_, s_, d_ = state.shape
    out = np.empty((cache.shape[0] + h_ * s_, d_), dtype=cache.dtype)
    for h in range(h_):
        n = int(headlens[h])
        src = int(cu_headlens[h])
        dst = src + h * s_
        out[dst:dst + n] = cache[src:src + n]
        out[dst + n:dst + n + s_] = state[0, h]
    return out


class OracleBatchedFlatCache:
    """Flat varlen cache with ``B*H`` segments ordered ``b*H + h``; per-head top-M eviction.

    Layout and append follow ``BatchedDynamicBudgetTrimKVCache.update``
    (src/trimkv/cache_utils.py:596-689); the eviction policy is the per-head
    one of ``TrimKVCache.compress_layer`` (:160-198) applied segment by segment,
    then ``head_lens``/``cu_seqlens_k`` are rebuilt as at :829-834.
    """

    def __init__(self):
        self._seen_tokens = 0
        self.key_cache, self.value_cache = [], []
        self.retention_weights, self.kv_positions = [], []
        self.head_lens, self.cu_seqlens_k = [], []
        self.batch_size = None
        self.num_kv_heads = None

    def get_seq_length(self):
        return self._seen_tokens

    def update(self, key_states, value_states, retention_weights, cache_positions, layer_idx):
        b_, h_, s_, d_ = key_states.shape
        self.batch_size, self.num_kv_heads = b_, h_
        if layer_idx == 0:
            self._seen_tokens += s_
        pos = np.asarray(cache_positions, dtype=np.int64)
        if pos.ndim == 1:
            pos = np.broadcast_to(pos[None, None, :], (b_, h_, s_))
        nseq = b_ * h_
        if len(self.key_cache) <= layer_idx:
            self.key_cache.append(np.ascontiguousarray(key_states).reshape(-1, d_))
            self.value_cache.append(np.ascontiguousarray(value_states).reshape(-1, d_))
            self.retention_weights.append(np.ascontiguousarray(retention_weights).reshape(-1, 1))
            self.kv_positions.append(np.ascontiguousarray(pos).reshape(-1, 1))
            self.head_lens.append(np.full((nseq,), s_, dtype=np.int32))
            self.cu_seqlens_k.append(np.arange(0, nseq * s_ + 1, s_, dtype=np.int32))
        else:
            hl, cu = self.head_lens[layer_idx], self.cu_seqlens_k[layer_idx]
            self.key_cache[layer_idx] = flat_append(
                self.key_cache[layer_idx], np.ascontiguousarray(key_states).reshape(1, nseq, s_, d_), hl, cu)
            self.value_cache[layer_idx] = flat_append(
                self.value_cache[layer_idx], np.ascontiguousarray(value_states).reshape(1, nseq, s_, d_), hl, cu)
            self.retention_weights[layer_idx] = flat_append(
                self.retention_weights[layer_idx],
                np.ascontiguousarray(retention_weights).reshape(1, nseq, s_, 1), hl, cu)
            self.kv_positions[layer_idx] = flat_append(
                self.kv_positions[layer_idx], np.ascontiguousarray(pos).reshape(1, nseq, s_, 1), hl, cu)
            self.head_lens[layer_idx] = hl + np.int32(s_)
            self.cu_seqlens_k[layer_idx] = cu + np.arange(0, nseq * s_ + 1, s_, dtype=np.int32)
        return (self.key_cache[layer_idx], self.value_cache[layer_idx], self.retention_weights[layer_idx],
                self.kv_positions[layer_idx],
                {"head_lens": self.head_lens[layer_idx], "cu_seqlens_k": self.cu_seqlens_k[layer_idx],
                 "batch_size": self.batch_size, "num_kv_heads": self.num_kv_heads})

    def compress(self, memory_size, buffer_size):
        q_idx = self._seen_tokens + 1
        for l in range(len(self.key_cache)):
            hl, cu = self.head_lens[l], self.cu_seqlens_k[l]
            ks, vs, bs, ps, nl = [], [], [], [], []
            for s in range(hl.shape[0]):
                a, n = int(cu[s]), int(hl[s])
                k, v = self.key_cache[l][a:a + n], self.value_cache[l][a:a + n]
                b, p = self.retention_weights[l][a:a + n, 0], self.kv_positions[l][a:a + n, 0]
                if n >= memory_size + buffer_size:
                    k, v, b, p, _ = compress_rows(k, v, b, p, q_idx, memory_size)
                ks.append(k); vs.append(v); bs.append(b[:, None]); ps.append(p[:, None]); nl.append(k.shape[0])
            self.key_cache[l] = np.concatenate(ks, 0)
            self.value_cache[l] = np.concatenate(vs, 0)
            self.retention_weights[l] = np.concatenate(bs, 0)
            self.kv_positions[l] = np.concatenate(ps, 0)
            self.head_lens[l] = np.asarray(nl, dtype=np.int32)
            self.cu_seqlens_k[l] = np.concatenate([[0], np.cumsum(nl)]).astype(np.int32)


# --------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------
def _softmax_av(q, k, v, scale, n_visible):
    """q [G,Q,D], k/v [n,D] fp32; query row i sees keys j < n_visible[i]."""
    s = np.einsum("gqd,nd->gqn", q, k) * np.float32(scale)
    n = k.shape[0]
    mask = np.arange(n)[None, :] < np.asarray(n_visible)[:, None]  # [Q,n]
    s = np.where(mask[None], s, -np.inf)
    m = s.max(axis=-1, keepdims=True)
    m = np.where(np.isfinite(m), m, 0.0)
    p = np.exp(s - m)
    den = p.sum(axis=-1, keepdims=True)
    p = np.where(den > 0, p / np.where(den > 0, den, 1.0), 0.0)
    return np.einsum("gqn,nd->gqd", p, v)


def varlen_gqa_attention(query, key_flat, value_flat, cu_seqlens_k, batch_size, num_kv_heads, scale=None):
    """Per-segment GQA attention over a packed varlen cache, fp32.

    Restates ``batched_dynamic_kv_budget_attention_forward``
    (src/trimkv/attn/flash_attn.py:79-151): segment ``b*Hkv + h`` holds the keys
    of KV head h of request b; the G = Hq/Hkv query heads ``h*G .. h*G+G-1``
    attend to it; causal with bottom-right alignment (query row i of Q sees keys
    ``j <= n - Q + i``, flash-attn's ``causal=True`` convention); softmax scale
    defaults to D^-1/2 (:85 accepts ``scaling`` but does not forward it).
    query [B,Hq,Q,D] -> output [B,Q,Hq,D] (:147-149).
    """
    q = np.asarray(query, dtype=np.float32)
    b_, hq, ql, d_ = q.shape
    g = hq // num_kv_heads
    scale = d_ ** -0.5 if scale is None else scale
    kf = np.asarray(key_flat, dtype=np.float32)
    vf = np.asarray(value_flat, dtype=np.float32)
    out = np.zeros((b_, ql, hq, d_), dtype=np.float32)
    for b in range(b_):
        for h in range(num_kv_heads):
            s = b * num_kv_heads + h
            a, e = int(cu_seqlens_k[s]), int(cu_seqlens_k[s + 1])
            n = e - a
            if n == 0:
                continue
            vis = n - ql + np.arange(ql) + 1
            o = _softmax_av(q[b, h * g:(h + 1) * g], kf[a:e], vf[a:e], scale, vis)  # [G,Q,D]
            out[b, :, h * g:(h + 1) * g, :] = o.transpose(1, 0, 2)
    return out


def dense_gqa_attention(query, key, value, scale=None, causal=True):
    """Dense ``[B,Hkv,n,D]`` keys; same arithmetic (src/trimkv/attn/eager_attn.py:48-73)."""
    b_, hkv, n, d_ = key.shape
    kf = np.ascontiguousarray(key).reshape(-1, d_)
    vf = np.ascontiguousarray(value).reshape(-1, d_)
    cu = np.arange(0, b_ * hkv * n + 1, n, dtype=np.int64)
    if not causal:
        raise NotImplementedError
    return varlen_gqa_attention(query, kf, vf, cu, b_, hkv, scale)


# --------------------------------------------------------------------------
# budget-sharing eviction of the flat caches
# --------------------------------------------------------------------------
def _group_keep_counts(scores, k_total=None, threshold=None, bucketize_attribution=False):
    """scores: list of 1-D fp32 arrays (the group's segments in concatenated order).  Returns how many rows of
    each segment are among the group's k_total best (canonical ties: lower concatenated index first), or
    score >= threshold.

    bucketize_attribution restates src/trimkv/cache_utils.py:495-498: the selected flat indices are attributed to
    heads with ``torch.bucketize(idx, cumsum(head_lens))`` (right=False), which files an index equal to a boundary
    -- the first row of the next head -- under the previous head."""
    lens = [len(s) for s in scores]
    flat = np.concatenate(scores) if scores else np.zeros((0,), np.float32)
    if threshold is not None:
        keep = flat >= np.float32(threshold)
    else:
        k = min(int(k_total), flat.shape[0])
        keep = np.zeros(flat.shape[0], bool)
        if k > 0:
            keep[canonical_topm(flat[None], k)[0]] = True
    out, a = [], 0
    if bucketize_attribution:
        bounds = np.cumsum(lens)
        which = np.searchsorted(bounds, np.nonzero(keep)[0], side="left")
        return [int((which == j).sum()) for j in range(len(lens))]
    for n in lens:
        out.append(int(keep[a:a + n].sum())); a += n
    return out


class OracleFlatBudgetCache(OracleBatchedFlatCache):
    """``compress`` of the reference's flat caches, with canonical ties; scores in ``score_dtype`` (the dtype the
    reference's tensors hold log beta in: it multiplies without an upcast).

    ``batched=True`` restates BatchedDynamicBudgetTrimKVCache.compress (src/trimkv/cache_utils.py:697-945),
    ``batched=False`` DynamicBudgetTrimKVCache.compress (:334-536, batch size 1).  Keeping a group's top-k equals
    keeping each segment's own top-c rows for the per-segment counts c, so every variant reduces to counts.
    """

    def __init__(self, batched=True, score_dtype="float32", key_dtype="float32"):
        super().__init__()
        self.batched = batched
        self.score_dtype = score_dtype
        self.key_dtype = key_dtype      # dtype the reference's key tensors would have (norm and log are rounded to it)
        self._knorm = False

    def _scores(self, l, seg):
        a, n = int(self.cu_seqlens_k[l][seg]), int(self.head_lens[l][seg])
        sc = retention_scores(self.retention_weights[l][a:a + n, 0], self.kv_positions[l][a:a + n, 0],
                              self._seen_tokens + 1, self.score_dtype)
        if self._knorm:
            # :388-390, :443-450, :757-759, :876-878: scores = log_alpha + log(key.norm(dim=-1).clamp_min(1e-12)); the
            # norm (fp32 accumulation), the clamp constant and the log are rounded to the keys' dtype, the sum to the
            # promoted dtype (16-bit only if both operands are).
            k = np.asarray(self.key_cache[l][a:a + n], np.float32)
            nrm = round_to_dtype(np.sqrt(np.sum(k * k, axis=-1, dtype=np.float32)), self.key_dtype)
            nrm = np.maximum(nrm, round_to_dtype(np.float32(1e-12), self.key_dtype))
            lg = round_to_dtype(np.log(nrm).astype(np.float32), self.key_dtype)
            sc = (sc + lg).astype(np.float32)
            if self.score_dtype != "float32" and self.key_dtype == self.score_dtype:
                sc = round_to_dtype(sc, self.score_dtype)
        return sc

    def _apply(self, counts):
        """counts[l][seg] rows kept (canonical top-c inside the segment)."""
        q_idx = self._seen_tokens + 1
        for l, cl in counts.items():
            ks, vs, bs, ps, nl = [], [], [], [], []
            for seg in range(self.head_lens[l].shape[0]):
                a, n = int(self.cu_seqlens_k[l][seg]), int(self.head_lens[l][seg])
                k, v = self.key_cache[l][a:a + n], self.value_cache[l][a:a + n]
                b, p = self.retention_weights[l][a:a + n, 0], self.kv_positions[l][a:a + n, 0]
                c = min(cl[seg], n)
                if c < n:
                    if c == 0:
                        k, v, b, p = k[:0], v[:0], b[:0], p[:0]
                    else:
                        keep = canonical_topm(self._scores(l, seg)[None], c)[0]
                        k, v, b, p = k[keep], v[keep], b[keep], p[keep]
                ks.append(k); vs.append(v); bs.append(b[:, None]); ps.append(p[:, None]); nl.append(k.shape[0])
            self.key_cache[l] = np.concatenate(ks, 0); self.value_cache[l] = np.concatenate(vs, 0)
            self.retention_weights[l] = np.concatenate(bs, 0); self.kv_positions[l] = np.concatenate(ps, 0)
            self.head_lens[l] = np.asarray(nl, dtype=np.int32)
            self.cu_seqlens_k[l] = np.concatenate([[0], np.cumsum(nl)]).astype(np.int32)

    def compress(self, strategy="alpha", memory_size=2048, buffer_size=512, floor_budget_ratio=0.0,
                 alpha_threshold=0.0):
        L = len(self.key_cache)
        B = self.batch_size if self.batched else 1
        H = self.num_kv_heads if self.batched else self.head_lens[0].shape[0]
        M, Bf = memory_size, buffer_size
        rows = [self.key_cache[l].shape[0] for l in range(L)]
        total = sum(rows)
        thr = "threshold" in strategy
        self._knorm = "knorm" in strategy
        # :462, :893 compare with a 0-dim fp32 tensor, which torch casts to the dtype of the scores
        log_thr = round_to_dtype(np.log(np.float32(alpha_threshold)), self.score_dtype) if thr else None
        counts = {}
        if self.batched:
            if total <= B * H * (M + Bf) * L and not thr:          # :714-717
                return
            if "layer_wise" in strategy:                            # :719-729
                for l in range(L):
                    if rows[l] <= B * H * (M + Bf):
                        continue
                    cl = []
                    for b in range(B):
                        sc = [self._scores(l, b * H + h) for h in range(H)]
                        k = M * H if floor_budget_ratio <= 0 else int(M * H * (1 - floor_budget_ratio))   # :781-783
                        s = _group_keep_counts(sc, k_total=k)
                        if floor_budget_ratio > 0:                  # :789-806
                            fl = int(M * floor_budget_ratio)
                            s = [max(si, min(fl, len(x))) for si, x in zip(s, sc)]
                        cl += s
                    counts[l] = cl
            else:                                                   # :836-945
                if total // B <= L * H * (M + Bf) and not thr:
                    return
                per = {l: [0] * (B * H) for l in range(L)}
                for b in range(B):
                    sc = [self._scores(l, b * H + h) for l in range(L) for h in range(H)]
                    s = _group_keep_counts(sc, k_total=L * H * M, threshold=log_thr)
                    for i, c in enumerate(s):
                        per[i // H][b * H + i % H] = c
                counts = per
        else:
            if "layer_wise" in strategy:                            # :356-369
                for l in range(L):
                    if H * (M + Bf) >= rows[l]:
                        continue
                    counts[l] = _group_keep_counts([self._scores(l, h) for h in range(H)], k_total=H * M)  # :396-397
            else:                                                   # :418-536
                if L * H * (M + Bf) > total and not thr:
                    return
                sc = [self._scores(l, h) for l in range(L) for h in range(H)]
                if floor_budget_ratio == 0:
                    s = _group_keep_counts(sc, k_total=L * H * M, threshold=log_thr)
                else:
                    s = _group_keep_counts(sc, k_total=int(L * H * M * (1 - floor_budget_ratio)),
                                           bucketize_attribution=True)                                     # :491-498
                    fl = int(M * floor_budget_ratio)                                                       # :499
                    s = [min(len(x), si + fl) for si, x in zip(s, sc)]
                counts = {l: s[l * H:(l + 1) * H] for l in range(L)}
        self._apply(counts)
