/*
 * trimkv_b200 — C ABI of the B200 (sm_100a) TRIM-KV cache hot path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream and
 * returns an int: 0 = launched, negative = argument error detected on the host
 * before any launch (tkv_last_error() describes it).  Problems that only the
 * device can see (a segment that would overflow its capacity, a length beyond
 * the stated bound) are reported through the caller-provided `status` word: the
 * kernel records the code with atomicMax and skips the offending segment; it
 * never traps and never waits without a bound.  The library allocates no device
 * memory and keeps no state besides the per-thread error string.
 *
 * Cache layout ("capacity-strided flat cache").  A cache holds `nseg` segments,
 * one per (request b, KV head h), segment index b*Hkv + h — the order of the
 * reference's flat cache (src/trimkv/cache_utils.py:621,632-643).  Segment s
 * owns rows [s*cap, s*cap + len[s]) of
 *     k_cache, v_cache : [nseg*cap, D]   bf16 / f16 / f32
 *     beta_cache       : [nseg*cap]      f32   (log beta, the retention gate output)
 *     pos_cache        : [nseg*cap]      i32   (original token position)
 *     seg_len          : [nseg]          i32
 *     cu_seqlens       : [nseg+1]        i32   exclusive prefix sum of seg_len
 *                        (what the reference hands to flash-attn as cu_seqlens_k,
 *                        src/trimkv/cache_utils.py:682-687)
 * Rows of a segment are in ascending position order.
 */
#ifndef TRIMKV_B200_H_
#define TRIMKV_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* tkv_stream_t; /* == cudaStream_t */

/* element types of K/V rows and of incoming log beta */
enum { TKV_BF16 = 0, TKV_F16 = 1, TKV_F32 = 2 };

/* host-side return codes */
enum {
  TKV_OK = 0,
  TKV_ERR_ARG = -1,       /* bad pointer / size / dtype / alignment */
  TKV_ERR_UNSUPPORTED = -2,
  TKV_ERR_LAUNCH = -3     /* cudaGetLastError() after the launch was not cudaSuccess */
};

/* device-side codes written to *status (atomicMax; 0 = clean) */
enum {
  TKV_DEV_OK = 0,
  TKV_DEV_CAPACITY = 1,   /* len + s_new > cap: segment skipped */
  TKV_DEV_LEN_BOUND = 2,  /* len > max_len given by the host: segment skipped */
  TKV_DEV_BAD_INDEX = 3,  /* a kept index outside [0, n): row skipped */
  TKV_DEV_TIMEOUT = 4     /* a bounded wait inside a kernel ran out: that work item produced no output */
};

int tkv_version(void);

/* Text of the last host-side error on the calling thread ("" if none). */
const char* tkv_last_error(void);

/*
 * Append s_new tokens to every segment, in place.
 * Replaces TrimKVCache.update's torch.cat x4 (src/trimkv/cache_utils.py:104-108) and
 * update_flatten_view_triton x4 + the head_lens / cu_seqlens_k bumps
 * (src/trimkv/triton/db_cache_utils.py:86-186, src/trimkv/cache_utils.py:649-680).
 *
 * k_new/v_new : [batch, hkv, s_new, D] with element strides (k_sb, k_sh, k_ss), rows contiguous.
 * beta_new    : [batch, hkv, s_new] of beta_dtype, element strides (b_sb, b_sh, b_ss); stored as f32.
 * pos_new     : int64, element strides (p_sb, p_sh, p_ss); a 1-D [s_new] position vector is
 *               passed with p_sb = p_sh = 0 (src/trimkv/cache_utils.py:79).
 * seg_len[s] += s_new; cu_seqlens[i] += i*s_new (cu_seqlens may be NULL).
 */
int tkv_append(void* k_cache, void* v_cache, float* beta_cache, int32_t* pos_cache,
               int32_t* seg_len, int32_t* cu_seqlens,
               const void* k_new, const void* v_new, int64_t k_sb, int64_t k_sh, int64_t k_ss,
               const void* beta_new, int beta_dtype, int64_t b_sb, int64_t b_sh, int64_t b_ss,
               const int64_t* pos_new, int64_t p_sb, int64_t p_sh, int64_t p_ss,
               int batch, int hkv, int s_new, int head_dim, int64_t cap, int kv_dtype,
               int32_t* status, tkv_stream_t stream);

/*
 * Retention-score top-M selection only (no data movement).
 * Replaces the score + topk + sort of TrimKVCache.compress_layer
 * (src/trimkv/cache_utils.py:172-192): score = f32(log beta) * f32(q_idx - pos), one
 * rounding; keep the `memory_size` largest; equal scores: lower index first; -0 == +0; NaN
 * largest.  For every segment with n = seg_len[s] (or n_uniform if seg_len is NULL):
 *   n >= trigger_len and n > memory_size : kept_idx[s, 0..M) = ascending kept indices, kept_cnt[s] = M
 *   otherwise                            : kept_cnt[s] = n (kept_idx untouched: nothing is evicted)
 * beta: f32 [nseg, beta_stride]; pos: i32 [nseg, pos_stride] (pos_stride 0 = shared by all segments).
 * max_len: host-known upper bound of n (sizes shared memory; <= 57000).
 */
int tkv_evict_select(const float* beta, int64_t beta_stride, const int32_t* pos, int64_t pos_stride,
                     const int32_t* seg_len, int n_uniform, int nseg, int64_t q_idx,
                     int memory_size, int trigger_len, int max_len,
                     int32_t* kept_idx, int32_t* kept_cnt, int32_t* status, tkv_stream_t stream);

/*
 * Gather kept rows from a source into a (different) capacity-strided cache:
 * dst row j of segment s <- src row kept_idx[s, j], j < kept_cnt[s] (kept_idx NULL or
 * kept_cnt[s] == n means identity: copy the first kept_cnt[s] rows).
 * Replaces the four gathers of TrimKVCache.compress_layer (src/trimkv/cache_utils.py:195-198)
 * for the prefill hand-off, where the source is the dense prompt K/V [batch, hkv, n, D]
 * (element strides k_sb, k_sh, k_ss).  src and dst must not overlap.
 * Sets seg_len[s] = kept_cnt[s] and rebuilds cu_seqlens (if not NULL) per group of
 * `group` segments (cu_seqlens: [nseg/group, group+1]).
 */
int tkv_compact(void* k_dst, void* v_dst, float* beta_dst, int32_t* pos_dst, int64_t cap,
                const void* k_src, const void* v_src, int64_t k_sb, int64_t k_sh, int64_t k_ss,
                const float* beta_src, int64_t beta_stride, const int32_t* pos_src, int64_t pos_stride,
                const int32_t* kept_idx, int64_t kept_stride, const int32_t* kept_cnt,
                int32_t* seg_len, int32_t* cu_seqlens, int group,
                int batch, int hkv, int n_src, int head_dim, int kv_dtype,
                int32_t* status, tkv_stream_t stream);

/*
 * Fused eviction, in place: select (as tkv_evict_select) then stable stream compaction of
 * K, V, log beta and position rows of every segment with seg_len >= trigger_len down to
 * memory_size rows, then seg_len = memory_size and cu_seqlens rebuilt per group.
 * Replaces TrimKVCache.compress / compress_layer (src/trimkv/cache_utils.py:140-198) and the
 * head_lens / cu_seqlens_k rebuild of the flat caches (:406-416, :829-834).
 * kept_idx_out (nullable, [nseg, memory_size]) receives the kept indices of evicted segments.
 */
int tkv_evict(void* k_cache, void* v_cache, float* beta_cache, int32_t* pos_cache,
              int32_t* seg_len, int32_t* cu_seqlens, int group,
              int nseg, int64_t cap, int head_dim, int kv_dtype, int64_t q_idx,
              int memory_size, int trigger_len, int max_len,
              int32_t* kept_idx_out, int32_t* status, tkv_stream_t stream);

/*
 * tkv_evict with a keep count per segment and a protected tail.
 * keep_cnt (nullable, [nseg]): segment s keeps its keep_cnt[s] best rows (untouched if keep_cnt[s] >= its
 * length); with keep_cnt == NULL it behaves as tkv_evict.  protect_last: the newest rows always score +inf
 * (TrimKVCache.sliding_window_size, src/trimkv/cache_utils.py:186-187).  kept_stride: row stride of
 * kept_idx_out when keep counts vary.  strategy: TKV_STRATEGY_ALPHA, or TKV_STRATEGY_KNORM_ALPHA to add log ||k|| to
 * the score (src/trimkv/cache_utils.py:176-180; norm and log rounded to K's dtype as torch does).
 * Used after tkv_group_budget for the budget-sharing strategies.
 */
enum { TKV_STRATEGY_ALPHA = 0, TKV_STRATEGY_KNORM_ALPHA = 1,
       TKV_STRATEGY_KNORM_ALPHA_CLAMPED = 2 /* the flat classes' form: log(max(||k||, 1e-12)), :390 */ };
/* OR-ed into `strategy`: dtype the retention score log beta * (q_idx - pos) is computed in.  TrimKVCache upcasts to
 * fp32 (src/trimkv/cache_utils.py:172); the flat budget-sharing caches multiply in the stored dtype
 * (:386, :441, :755, :882), i.e. the age is rounded to that dtype and so is the product. */
enum { TKV_SCORE_F32 = 0, TKV_SCORE_BF16 = 1 << 8, TKV_SCORE_F16 = 2 << 8 };
int tkv_evict_ex(void* k_cache, void* v_cache, float* beta_cache, int32_t* pos_cache,
                 int32_t* seg_len, int32_t* cu_seqlens, int group,
                 int nseg, int64_t cap, int head_dim, int kv_dtype, int64_t q_idx,
                 int memory_size, int trigger_len, int max_len,
                 const int32_t* keep_cnt, int protect_last, int kept_stride, int strategy,
                 const float* scores /* nullable: precomputed by tkv_flat_scores, [nseg*cap] */,
                 int32_t* kept_idx_out, int32_t* status, tkv_stream_t stream);

/*
 * tkv_evict with ctas_per_segment CTAs sharing the rows of each evicting segment (same result, bit for bit).
 * For calls in which few segments evict at once (one request, or a steady state in which each segment fires once
 * every buffer_size steps), where one CTA per segment would leave most SMs idle; same reference code as tkv_evict
 * (src/trimkv/cache_utils.py:140-198).  Requires max_len - memory_size rows of K+V to fit in shared memory
 * (<= 200 KB) and ctas_per_segment <= 32.  workspace: device scratch of tkv_evict_multi_workspace_bytes() bytes,
 * contents irrelevant before and after the call; one workspace serves one stream at a time.
 * ctas_per_segment == 1 is tkv_evict_ex without keep counts.
 */
int64_t tkv_evict_multi_workspace_bytes(int nseg, int memory_size, int ctas_per_segment);
int tkv_evict_multi(void* k_cache, void* v_cache, float* beta_cache, int32_t* pos_cache,
                    int32_t* seg_len, int32_t* cu_seqlens, int group,
                    int nseg, int64_t cap, int head_dim, int kv_dtype, int64_t q_idx,
                    int memory_size, int trigger_len, int max_len, int protect_last, int strategy,
                    int ctas_per_segment, void* workspace, int64_t workspace_bytes,
                    int32_t* kept_idx_out, int32_t* status, tkv_stream_t stream);

/*
 * Keep counts under a shared token budget.  Group g consists of the segments
 * {g*inner + o*outer_stride + i : o < n_outer, i < inner}; among all rows of a group the k_total best scores are
 * kept (ties: lower index in that concatenated order), or, with use_threshold, every row whose score is
 * >= threshold.  Per segment the number of kept rows s becomes keep_cnt = s (floor_mode 0),
 * min(len, s' + floor_cnt) (1) or max(s, min(floor_cnt, len)) (2); in mode 1, s' is s after the reference's
 * attribution (src/trimkv/cache_utils.py:495-498: a kept row that is the first of its head is counted for the
 * preceding head of the group).
 * Replaces the top-k + mask + per-head .item() loops of _compress_layer, _compress_all_layers,
 * _compress_layer_batched and _compress_all_layers_batched
 * (src/trimkv/cache_utils.py:371-416, 418-536, 740-834, 836-945); scores in fp32 or in the stored dtype.
 */
int tkv_group_budget(const float* beta_cache, const int32_t* pos_cache, const int32_t* seg_len, int64_t cap,
                     int groups, int inner, int n_outer, int64_t outer_stride, int64_t q_idx,
                     int64_t k_total, int use_threshold, float threshold, int floor_mode, int floor_cnt,
                     int score_dtype /* 0 fp32, 1 bf16, 2 f16: as TKV_SCORE_* >> 8 */,
                     const float* scores /* nullable: precomputed by tkv_flat_scores */,
                     int32_t* keep_cnt, int32_t* status, tkv_stream_t stream);

/*
 * Scores of every live row, once, into scores_out [nseg*cap] (fp32 holding values of the score dtype), for the
 * strategies that read the K rows: "knorm_alpha" / "knorm_alpha_threshold" of the flat caches
 * (src/trimkv/cache_utils.py:388-390, 443-450, 757-759, 876-878: log_alpha + log(max(||k||, 1e-12)), every step
 * rounded as torch rounds it for tensors of these dtypes).  strategy: TKV_STRATEGY_* | TKV_SCORE_*.
 * tkv_group_budget and tkv_evict_ex then take the array through their `scores` argument.
 */
int tkv_flat_scores(const void* k_cache, const float* beta_cache, const int32_t* pos_cache,
                    const int32_t* seg_len, int nseg, int64_t cap, int head_dim, int kv_dtype,
                    int64_t q_idx, int strategy, int max_len, float* scores_out, tkv_stream_t stream);

/*
 * Functional append on the reference's packed layout: out[origin_rows + heads*s_new, row] = for every head its
 * old rows followed by its s_new new rows.  cache: [origin_rows, row_bytes]; state: [heads*s_new, row_bytes];
 * cu_headlens: [heads+1] exclusive prefix sum of the old per-head lengths.  Any row size (K/V rows, 2-byte log
 * beta, 8-byte positions).  Same contract as update_flatten_view_triton
 * (src/trimkv/triton/db_cache_utils.py:86-186) without its host synchronisation.
 */
int tkv_flat_append_packed(const void* cache, const void* state, const int32_t* cu_headlens, void* out,
                           int heads, int s_new, int64_t origin_rows, int64_t row_bytes, tkv_stream_t stream);

/* Rebuild cu_seqlens[g, 0..group] = exclusive prefix sum of seg_len[g*group .. ] for each group. */
int tkv_rebuild_cu_seqlens(const int32_t* seg_len, int32_t* cu_seqlens, int nseg, int group,
                           tkv_stream_t stream);

/*
 * Split-KV varlen GQA decode attention, one query token per request.
 * Replaces batched_dynamic_kv_budget_attention_forward -> flash_attn_varlen_func
 * (src/trimkv/attn/flash_attn.py:79-151) and the dense path for TrimKVCache:
 * for segment s = b*hkv + h the G = hq/hkv query heads h*G..h*G+G-1 of request b attend to
 * rows [start(s), start(s)+seg_len[s]) of k_cache/v_cache, softmax in f32, scale applied to
 * q.k before the softmax.  start(s) = seg_start[s] if seg_start != NULL (packed layout,
 * cu_seqlens_k of the reference) else s*cap.  With seg_start, cap states the number of rows of the packed
 * k_cache / v_cache (sum of the lengths, at least seg_start[s] + seg_len[s] for every s): the tensor-core
 * kernel bounds its tile loads by it; cap = 0 (rows not stated) selects the CUDA-core kernel, which reads
 * row by row.
 * q   : [batch, hq, D] with element strides (q_sb, q_sh); same dtype as K/V (bf16 or f16).
 * out : [batch, hq, D] contiguous (the reference's [B, Q=1, Hq, D], flash_attn.py:147-149).
 * workspace: tkv_decode_attn_workspace_bytes(...) bytes of scratch, 256-byte aligned.
 * max_len: host-known upper bound of seg_len (sizes the grid).
 */
size_t tkv_decode_attn_workspace_bytes(int batch, int hq, int hkv, int head_dim, int max_len);

int tkv_decode_attn(const void* q, int64_t q_sb, int64_t q_sh,
                    const void* k_cache, const void* v_cache,
                    const int32_t* seg_len, const int32_t* seg_start, int64_t cap,
                    void* out, void* workspace, size_t workspace_bytes,
                    int batch, int hq, int hkv, int head_dim, int kv_dtype,
                    float scale, int max_len, int32_t* status, tkv_stream_t stream);

/*
 * tkv_decode_attn for ragged lengths.  total_len_bound: an upper bound on the sum of seg_len over all segments that
 * the host knows without reading device memory (the flat budget-sharing caches keep it: head_lens sums to at most
 * budget + buffer per layer, src/trimkv/cache_utils.py:346-369, 714-738).  The split kernel's grid is then sized
 * by total_len_bound / 256 + nseg work items instead of nseg * ceil(max_len / 256), most of which would find no
 * tokens; a one-CTA kernel builds the item list from seg_len first.  Same result as tkv_decode_attn.  If the true
 * total exceeds the bound the surplus chunks are skipped and the status word reports TKV_DEV_LEN_BOUND.
 * The workspace is larger by the item list: tkv_decode_attn_ragged_workspace_bytes().
 */
size_t tkv_decode_attn_ragged_workspace_bytes(int batch, int hq, int hkv, int head_dim, int max_len,
                                              int64_t total_len_bound);
int tkv_decode_attn_ragged(const void* q, int64_t q_sb, int64_t q_sh,
                           const void* k_cache, const void* v_cache,
                           const int32_t* seg_len, const int32_t* seg_start, int64_t cap,
                           void* out, void* workspace, size_t workspace_bytes,
                           int batch, int hq, int hkv, int head_dim, int kv_dtype,
                           float scale, int max_len, int64_t total_len_bound,
                           int32_t* status, tkv_stream_t stream);

/*
 * Several query tokens per request against the cache that already holds them (a later prompt, speculative or
 * multi-token decoding): what flash_attn_varlen_func(causal=True) computes for the reference when Q > 1
 * (src/trimkv/attn/flash_attn.py:118-145).  Segment s has seg_len[s] cached tokens INCLUDING the q_tokens new ones;
 * query token i of a request attends to the first seg_len - q_tokens + i + 1 tokens of each of its segments
 * (bottom-right aligned causal mask).  q: [batch, q_tokens, hq, D] with element strides (q_sb, q_st, q_sh);
 * out: [batch, q_tokens, hq, D] contiguous.  Same tensor-core kernel as tkv_decode_attn with the query rows
 * (token, head) on the MMA's N dimension, 16 rows per CTA; each further group of 16 rows re-reads the K/V chunk, so
 * this entry point is meant for a handful of tokens, not for whole prompts.  Requires bf16/f16, head_dim 128 and
 * the capacity-strided layout (TKV_ERR_UNSUPPORTED otherwise).
 */
size_t tkv_decode_attn_multi_workspace_bytes(int batch, int hq, int hkv, int head_dim, int max_len, int q_tokens);
int tkv_decode_attn_multi(const void* q, int64_t q_sb, int64_t q_st, int64_t q_sh,
                          const void* k_cache, const void* v_cache, const int32_t* seg_len, int64_t cap,
                          void* out, void* workspace, size_t workspace_bytes,
                          int batch, int hq, int hkv, int head_dim, int kv_dtype,
                          float scale, int max_len, int q_tokens, int32_t* status, tkv_stream_t stream);

/*
 * Head-sharded decode (each rank holds hkv of the KV heads and their hq query heads; no counterpart in the
 * single-process reference): tkv_decode_attn whose merge step stores the result straight into the gathered
 * [batch, out_row_stride] buffer of EVERY rank, at element column out_col_offset, and then raises this rank's flag
 * on every peer; it replaces "attention, then all-gather" by one pass.  peer_out[r] / peer_flags[r]: HOST arrays of
 * `world` device pointers (rank r's buffer and its int32[world] flag array, mapped into this process, e.g. through
 * CUDA IPC; entry `rank` is this rank's own memory).  Only plain stores go to peer memory; nothing is read from it.
 * sync_state: int32[3] in this rank's memory, zero before the first exchange, private to this (stream, group).
 * `out` is still required (scratch for single-chunk problems).  world <= 8.
 * tkv_peer_wait: to be enqueued before the first kernel that reads the gathered buffer; returns (on the stream)
 * once every peer's flag has reached this rank's exchange count.  The wait is bounded (about four seconds), after
 * which the status word reports TKV_DEV_TIMEOUT and the stream continues.
 * A buffer may be written again by the peers as soon as this rank has completed its NEXT exchange (raising its flag
 * for exchange e+1 is what tells the peers that it has consumed the buffer of exchange e), so consecutive exchanges
 * must use different buffers and a buffer's next use must lie at least two exchanges later: two buffers in
 * alternation for an even number of exchanges per step, three (one of them for the first exchange of a step) in
 * general; a single exchange per step is not supported.
 */
int tkv_decode_attn_push(const void* q, int64_t q_sb, int64_t q_sh,
                         const void* k_cache, const void* v_cache,
                         const int32_t* seg_len, const int32_t* seg_start, int64_t cap,
                         void* out, void* workspace, size_t workspace_bytes,
                         int batch, int hq, int hkv, int head_dim, int kv_dtype,
                         float scale, int max_len,
                         void* const* peer_out, int32_t* const* peer_flags, int world, int rank,
                         int64_t out_row_stride, int64_t out_col_offset, int32_t* sync_state,
                         int32_t* status, tkv_stream_t stream);
int tkv_peer_wait(const int32_t* flags, int32_t* sync_state, int world, int rank,
                  int max_polls /* polls of about 0.2 us each before giving up; <= 0: 2^24, about four seconds */,
                  int32_t* status, tkv_stream_t stream);
/* Lets kernels of the current device store to memory of peer_device (cudaDeviceEnablePeerAccess; a no-op if it is
 * already enabled or peer_device is the current device).  Needed once per peer before tkv_decode_attn_push. */
int tkv_enable_peer_access(int peer_device);
/*
 * Many query tokens per request (a prompt pass, a piece of a chunked prefill) against the cache that already
 * holds them: what flash_attn_varlen_func(causal=True) computes for the reference when Q > 1
 * (src/trimkv/attn/flash_attn.py:118-145; for the dense prompt pass, the causal attention of
 * src/trimkv/attn/__init__.py:15-26).  Same semantics as tkv_decode_attn_multi (segment s holds seg_len[s] tokens
 * including the q_tokens new ones; query token i sees the first seg_len - q_tokens + i + 1 of them), different
 * kernel: a block of 128 query rows (token, head) stays resident in shared memory and the segment's K/V are
 * streamed past it once with an online softmax, so the work per cached token does not grow with q_tokens / 128
 * re-reads and no workspace or merge step is needed.
 * q: [batch, q_tokens, hq, D] with element strides (q_sb, q_st, q_sh); out: [batch, q_tokens, hq, D] contiguous.
 * k_cache / v_cache: capacity-strided [batch*hkv, cap, D]; a dense prompt [batch, hkv, S, D] is the case cap = S.
 * seg_len: NULL = every segment holds max_len tokens.  Requires bf16/f16 and head_dim 128.
 */
int tkv_prefill_attn(const void* q, int64_t q_sb, int64_t q_st, int64_t q_sh,
                     const void* k_cache, const void* v_cache, const int32_t* seg_len, int64_t cap,
                     void* out, int batch, int hq, int hkv, int head_dim, int kv_dtype,
                     float scale, int max_len, int q_tokens, int32_t* status, tkv_stream_t stream);

/* Sharing a device allocation between the rank processes of one box (CUDA IPC; host-only calls, no kernel).
 * tkv_ipc_export: handle (TKV_IPC_HANDLE_BYTES bytes) of the allocation that contains ptr, and ptr's offset in it.
 * tkv_ipc_import: maps an exported allocation into this process with the CURRENT device (peer access to the owning
 * GPU is enabled by the mapping); *base_out + offset is the peer's ptr.  One import per handle and process.
 * tkv_ipc_close: unmaps. */
#define TKV_IPC_HANDLE_BYTES 64
int tkv_ipc_export(const void* ptr, void* handle_out, int64_t* offset_out);
int tkv_ipc_import(const void* handle, void** base_out);
int tkv_ipc_close(void* base);

/*
 * tkv_decode_attn for callers that cannot allocate device memory.  (No counterpart in the reference: its
 * attention always runs inside PyTorch, whose allocator provides flash-attn's temporaries.)
 * Meant for hosts that cannot hand the library a workspace: a server whose block arena already owns the whole
 * device, a plug-in slot without access to the host's allocator, or a loop that cannot afford the device-wide
 * synchronisation of cudaMalloc/cudaFree.  Same arguments and results as tkv_decode_attn without
 * `workspace`; the per-chunk partial results live in an array of TKV_STATIC_SCRATCH_BYTES that is part of
 * the library image, so every GPU that loads the library holds that much memory until the process exits.
 *  - Limit: problems whose per-chunk partials exceed TKV_STATIC_SCRATCH_BYTES (never more than
 *    tkv_decode_attn_workspace_bytes(...) of the same problem) are refused with TKV_ERR_UNSUPPORTED (nothing is
 *    launched); use tkv_decode_attn for those.
 *  - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that
 *    device current); make that first call outside any stream capture.  No call allocates or frees memory.
 *    The address is kept per device for the life of the process, so do not call this after cudaDeviceReset.
 *  - It runs the CUDA-core split kernel for every shape (head_dim 64 or 128, bf16 or f16, either layout; with
 *    seg_start, cap is not used).
 *  - All calls on a device share the one array, and it keeps whatever the previous call left there (no call
 *    relies on its initial content).  Two calls that can overlap on the GPU (different streams, or a second
 *    process thread) race on it: serialise them on one stream or order them with events.
 */
#define TKV_STATIC_SCRATCH_BYTES (32u << 20)
int tkv_decode_attn_static(const void* q, int64_t q_sb, int64_t q_sh,
                           const void* k_cache, const void* v_cache,
                           const int32_t* seg_len, const int32_t* seg_start, int64_t cap,
                           void* out, int batch, int hq, int hkv, int head_dim, int kv_dtype,
                           float scale, int max_len, int32_t* status, tkv_stream_t stream);

/*
 * Fused producer of one decode step (one new token per request), head_dim 128, bf16/f16.
 * Replaces, per layer, q_norm / k_norm, the retention-gate tail, RoPE, the transposes and
 * cache.update of TrimKVQwen3Attention.forward
 * (src/trimkv/models/qwen3/modeling_trimkv_qwen3.py:328-353, gate tail :174-178); with q_norm_w and
 * k_norm_w both NULL the per-head RMSNorm is skipped, which is the producer of the Llama and Phi-3 attention
 * (src/trimkv/models/llama/modeling_trimkv_llama.py:303-332, src/trimkv/models/phi3/modeling_trimkv_phi3.py:353-384;
 * Phi-3's fused qkv_proj already has the q | k | v row layout).
 * qkvg : [batch, row_stride] rows holding  q (hq*128) | k (hkv*128) | v (hkv*128) | gate hidden (gate_inter),
 *        i.e. the output of one GEMM over the concatenated q/k/v/linear1 weights (linear1 bias included).
 * cos/sin : [128] of the model dtype for this token's position; pos: int64[1], that position.
 * Writes q_out [batch, hq, 128] = RoPE(RMSNorm(q)) and appends RoPE(RMSNorm(k)), v,
 * log beta = logsigmoid(gate_w2 . SiLU(gate hidden) + gate_bias) and pos to every segment
 * (seg_len += 1, cu_seqlens[i] += i), rounding to the model dtype after every step the eager
 * PyTorch sequence rounds at.
 * in_splits / in_bias (also on tkv_add_rmsnorm's delta and tkv_silu_mul's gate_up): 0 = the input is in the model
 * dtype; s > 0 = the input is the fp32 output of tkv_skinny_gemm, s partial sums [s][rows][cols] that the kernel
 * adds in order, plus in_bias (model dtype, [cols], nullable), rounded once to the model dtype.
 */
int tkv_decode_prep(const void* qkvg, int64_t row_stride,
                    const void* q_norm_w, const void* k_norm_w, float eps,
                    const void* cos, const void* sin,
                    const void* gate_w2, const void* gate_bias, int gate_inter,
                    const int64_t* pos, void* q_out,
                    void* k_cache, void* v_cache, float* beta_cache, int32_t* pos_cache,
                    int32_t* seg_len, int32_t* cu_seqlens, int64_t cap,
                    int batch, int hq, int hkv, int head_dim, int dtype,
                    int in_splits, const void* in_bias,
                    int32_t* status, tkv_stream_t stream);

/*
 * residual[r, :] += delta[r, :] (skipped if delta is NULL); out[r, :] = weight * RMSNorm(residual[r, :]).
 * Replaces the residual add + Qwen3RMSNorm pairs of the decoder layer
 * (src/trimkv/models/qwen3/modeling_trimkv_qwen3.py:414-437).  cols % 8 == 0; out may not alias residual.
 */
int tkv_add_rmsnorm(void* residual, const void* delta, const void* weight, void* out,
                    int rows, int cols, float eps, int dtype, int in_splits, const void* in_bias,
                    tkv_stream_t stream);

/*
 * out[r, j] = SiLU(gate_up[r, j]) * gate_up[r, inter + j]: the activation of Qwen3MLP over the output of one
 * GEMM with the concatenated gate/up weights (src/trimkv/models/qwen3/modeling_trimkv_qwen3.py:436).
 */
int tkv_silu_mul(const void* gate_up, void* out, int rows, int inter, int dtype, int in_splits,
                 const void* in_bias, tkv_stream_t stream);

/*
 * Weight-streaming GEMM of the decode step on tcgen05 + TMA: partial[s][m][n] (fp32) such that
 * sum_s partial[s] = x[m, k] . w[n, k]^T, for m <= 32 rows, k a multiple of 64, x/w bf16 or f16, row-major.
 * Replaces the nn.Linear calls on one token per request (q/k/v/gate, o_proj, gate/up, down:
 * src/trimkv/models/qwen3/modeling_trimkv_qwen3.py:328-333,383,436).  s = tkv_skinny_gemm_splits(m, n, k) (0 if the
 * shape is unsupported); partial must hold s*m*n floats.  The consumers above add the partials.
 */
int tkv_skinny_gemm_splits(int m, int n, int k);
int tkv_skinny_gemm(const void* x, const void* w, float* partial, int m, int n, int k, int dtype,
                    int32_t* status, tkv_stream_t stream);

/*
 * tkv_skinny_gemm whose activation operand is computed instead of loaded: x[m, k] = SiLU(gate_up[m, :k]) *
 * gate_up[m, k:2k], i.e. tkv_silu_mul and the down projection of Qwen3MLP.forward in one kernel
 * (src/trimkv/models/qwen3/modeling_trimkv_qwen3.py:120-122; Phi-3's gate|up output has the same layout,
 * src/trimkv/models/phi3/modeling_trimkv_phi3.py:102-108).  gate_up: [m, 2k] row-major, model dtype, as one GEMM
 * over the concatenated gate/up weights produces it (bias already added).  Same partial-sum output and rounding
 * (SiLU rounded, product rounded) as the two separate calls.
 */
int tkv_skinny_gemm_swiglu(const void* gate_up, const void* w, float* partial, int m, int n, int k, int dtype,
                           int32_t* status, tkv_stream_t stream);

/* Blocks until `stream` is idle, then returns *status (a TKV_DEV_* code) and clears it. */
int tkv_read_status(int32_t* status, tkv_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* TRIMKV_B200_H_ */
