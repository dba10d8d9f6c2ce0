// Retention-score top-M eviction: selection, stable stream compaction, cu_seqlens rebuild.
//
// Replaces TrimKVCache.compress / compress_layer (src/trimkv/cache_utils.py:140-198): fp32 score,
// torch.topk, torch.sort and four gathers into fresh allocations.  Here one CTA owns one segment:
//   1. keys: score = f32(log beta) * f32(q_idx - pos) mapped to an order-preserving uint32, kept in
//      shared memory (4 bytes per live token);
//   2. 4-pass, 8-bit radix select of the M-th largest key, warp-aggregated histogram updates;
//   3. one ordered block scan turns "key > T, or key == T and among the first r equal keys" into the
//      ascending list of kept indices (written over the keys);
//   4. in-place stable compaction: tiles of kept rows are loaded into registers (16-byte vectors),
//      a barrier, then stored at their destination.  dst <= src for every row and tiles are handled
//      in ascending order, so a tile's stores can only land on rows whose content was already consumed.
// Algorithmic bytes per segment: 8n (scan) + 2*M*row_pair_bytes (move K,V) + 8M (metadata).
#include "tkv_common.cuh"

namespace tkv {

constexpr int kEvictThreads = 256;
constexpr int kEvictUnroll = 8;              // 16-byte vectors in flight per thread and tile
constexpr int kEvictMaxCtas = 32;            // CTAs sharing one segment's rows (tkv_evict_multi)
constexpr int kMaxSelectLen = 57000;         // keys must fit in 227 KB of shared memory

constexpr int kEvictThreadsWide = 512;       // for long segments, whose key array allows fewer CTAs per SM
constexpr int kMoveThreads = 256;            // evict_move_kernel: its staging area limits CTAs per SM, so each is wide
constexpr int kMoveGridCtas = 148 * 4;       // evict_move_kernel: blocks in its grid (they loop over the evicting segments)
constexpr int kEvictThreadsPlan = 1024;      // selection only (plan mode): few segments, so each gets a full CTA
struct SelectScratch {
  int hist[256];
  int warp_sums[kEvictThreadsPlan / 32 + 1];
  int sel_digit;
  int sel_k;
  int first_evicted;
};

// Finds T = key of the m-th largest element and r = how many elements equal to T are kept.
// All threads of the block call this; keys[0..n) are in shared memory.
template <int kThreads>
__device__ __forceinline__ void radix_select_mth(const uint32_t* keys, int n, int m, SelectScratch* sc,
                                                 uint32_t* thresh, int* n_eq_keep) {
  const int lane = threadIdx.x & 31;
  uint32_t prefix = 0, decided = 0;
  int k = m;
  const int n_round = (n + kThreads - 1) / kThreads * kThreads;
#pragma unroll 1
  for (int shift = 24; shift >= 0; shift -= 8) {
    if (threadIdx.x < 256) sc->hist[threadIdx.x] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n_round; i += kThreads) {
      uint32_t key = i < n ? keys[i] : 0u;
      const bool valid = i < n && (key & decided) == prefix;
      const int digit = valid ? (int)((key >> shift) & 255u) : 256 + lane;
      // Lanes with the same digit elect one leader that adds their count: the high digits of the
      // scores are nearly constant, which would serialise plain shared-memory atomics.
      const unsigned peers = __match_any_sync(0xffffffffu, digit);
      if (valid && lane == __ffs(peers) - 1) atomicAdd(&sc->hist[digit], __popc(peers));
    }
    __syncthreads();
    // Thread t looks at bin 255 - t: an exclusive scan in this order is the count of strictly larger digits.
    const int bin = 255 - (int)threadIdx.x;
    const int c = threadIdx.x < 256 ? sc->hist[bin] : 0;
    int total;
    const int above = block_exclusive_scan<kThreads>(c, sc->warp_sums, &total);
    if (threadIdx.x < 256 && above < k && k <= above + c) { sc->sel_digit = bin; sc->sel_k = k - above; }
    __syncthreads();
    prefix |= (uint32_t)sc->sel_digit << shift;
    decided |= 255u << shift;
    k = sc->sel_k;
    __syncthreads();
  }
  *thresh = prefix;
  *n_eq_keep = k;
}

// Overwrites keys[0..m) with the ascending indices of the kept elements; returns the first evicted index.
template <int kThreads>
__device__ __forceinline__ int build_kept_list(uint32_t* keys, int n, uint32_t thresh, int n_eq_keep,
                                               SelectScratch* sc) {
  constexpr int kItems = 4;
  constexpr int kChunk = kThreads * kItems;
  if (threadIdx.x == 0) sc->first_evicted = n;
  int eq_base = 0, gt_base = 0;
#pragma unroll 1
  for (int base = 0; base < n; base += kChunk) {
    uint32_t key[kItems];
    int packed = 0;  // low 16 bits: #equal, high 16 bits: #greater (n < 65536)
    const int i0 = base + threadIdx.x * kItems;
#pragma unroll
    for (int u = 0; u < kItems; ++u) {
      const int i = i0 + u;
      key[u] = i < n ? keys[i] : 0u;
      if (i < n) packed += (key[u] == thresh) ? 1 : (key[u] > thresh ? (1 << 16) : 0);
    }
    int total;
    const int excl = block_exclusive_scan<kThreads>(packed, sc->warp_sums, &total);  // syncs inside
    int eq = eq_base + (excl & 0xffff), gt = gt_base + (excl >> 16);
    int my_first_evicted = n;
#pragma unroll
    for (int u = 0; u < kItems; ++u) {
      const int i = i0 + u;
      if (i >= n) break;
      const bool is_eq = key[u] == thresh, is_gt = key[u] > thresh;
      const bool keep = is_gt || (is_eq && eq < n_eq_keep);
      if (keep) keys[gt + min(eq, n_eq_keep)] = (uint32_t)i;
      else my_first_evicted = min(my_first_evicted, i);
      eq += is_eq; gt += is_gt;
    }
    if (my_first_evicted < n) atomicMin(&sc->first_evicted, my_first_evicted);
    eq_base += total & 0xffff; gt_base += total >> 16;
  }
  __syncthreads();
  return sc->first_evicted;
}

// Which (row of the tile, 16-byte column of the K|V row pair) vector number u of this thread is.  Vector i = tid +
// u*kThreads of a tile is row i / nvec, column i % nvec; when nvec divides the block size the column is fixed per
// thread and the row advances by a constant, which saves two integer divisions per 16 bytes moved.
struct TileMap {
  int r0, col0, rstep, nvec, regular;
  const char* cbase;   // address of this thread's column in row 0 of the segment (regular case)
};
template <int kThreads>
__device__ __forceinline__ TileMap make_tile_map(int nvec, int row_vecs, const char* kbase, const char* vbase) {
  TileMap t;
  t.nvec = nvec; t.regular = (kThreads % nvec) == 0;
  t.r0 = threadIdx.x / nvec; t.col0 = threadIdx.x - t.r0 * nvec; t.rstep = kThreads / nvec;
  t.cbase = t.col0 < row_vecs ? kbase + (int64_t)t.col0 * 16 : vbase + (int64_t)(t.col0 - row_vecs) * 16;
  return t;
}
template <int kThreads>
__device__ __forceinline__ int tile_row(const TileMap& t, int u) {
  return t.regular ? t.r0 + u * t.rstep : (int)(threadIdx.x + u * kThreads) / t.nvec;
}
template <int kThreads>
__device__ __forceinline__ int tile_col(const TileMap& t, int u, int r) {
  return t.regular ? t.col0 : (int)(threadIdx.x + u * kThreads) - r * t.nvec;
}
template <int kThreads>
__device__ __forceinline__ char* tile_ptr(const TileMap& t, int u, int r, int row, int64_t row_bytes, int row_vecs,
                                          const char* kbase, const char* vbase) {
  if (t.regular) return const_cast<char*>(t.cbase) + (int64_t)row * row_bytes;
  const int col = (int)(threadIdx.x + u * kThreads) - r * t.nvec;
  return const_cast<char*>(col < row_vecs ? kbase + (int64_t)col * 16 : vbase + (int64_t)(col - row_vecs) * 16) +
         (int64_t)row * row_bytes;
}

// Destination rows [lo, hi) of CTA c when `ctas` CTAs share rows [j0, m) of a segment.  A range is a whole number of
// tiles and at least as long as the largest displacement (<= tail_max, which the host derives from max_len - M), so
// that no CTA reads beyond its right neighbour's range; short segments simply use fewer of the CTAs.
__device__ __forceinline__ void move_range(int m, int j0, int ctas, int tail_max, int tile_rows, int c, int* lo, int* hi,
                                           int* per_out) {
  const int total = max(m - j0, 0);
  const int per = max(((total + ctas - 1) / ctas + tile_rows - 1) / tile_rows, (tail_max + tile_rows - 1) / tile_rows) * tile_rows;
  *lo = min(m, j0 + c * per);
  *hi = min(m, *lo + per);
  *per_out = per;
}

// log ||k||_2 of one K row as torch computes it for a tensor of K's dtype (src/trimkv/cache_utils.py:176-180, 388-390):
// the norm accumulates in fp32 and is rounded to the dtype, and the log is rounded to it again.
// Called by a whole warp (lanes stride over the row's 16-byte vectors); every lane returns the value.
__device__ __forceinline__ float log_row_norm(const char* row, int row_vecs, int kv_dtype, int lane, bool clamp) {
  float ss = 0.f;
  for (int c = lane; c < row_vecs; c += 32) {
    const uint4 v = ld16(row + (int64_t)c * 16);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (kv_dtype == TKV_F32) { const float a = __uint_as_float(w[j]); ss = fmaf(a, a, ss); }
      else if (kv_dtype == TKV_BF16) {
        const float a = __uint_as_float(w[j] << 16), b = __uint_as_float(w[j] & 0xffff0000u);
        ss = fmaf(a, a, ss); ss = fmaf(b, b, ss);
      } else {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
        ss = fmaf(f.x, f.x, ss); ss = fmaf(f.y, f.y, ss);
      }
    }
  }
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  float nrm = sqrtf(ss);
  if (kv_dtype == TKV_BF16) nrm = __bfloat162float(__float2bfloat16_rn(nrm));
  else if (kv_dtype == TKV_F16) nrm = __half2float(__float2half_rn(nrm));
  if (clamp) {  // the flat classes clamp the norm at 1e-12 (a scalar torch rounds to the tensor's dtype); TrimKVCache does not
    float floor_ = 1e-12f;
    if (kv_dtype == TKV_BF16) floor_ = __bfloat162float(__float2bfloat16_rn(floor_));
    else if (kv_dtype == TKV_F16) floor_ = __half2float(__float2half_rn(floor_));
    nrm = fmaxf(nrm, floor_);
  }
  float lg = logf(nrm);
  if (kv_dtype == TKV_BF16) lg = __bfloat162float(__float2bfloat16_rn(lg));
  else if (kv_dtype == TKV_F16) lg = __half2float(__float2half_rn(lg));
  return lg;
}

// log_alpha + log ||k||: torch adds in fp32 and rounds to the promoted dtype, which is 16-bit only if both the
// stored log beta (score_dtype) and K are 16-bit.
__device__ __forceinline__ float knorm_score(float log_alpha, float log_norm, int score_dtype, int kv_dtype) {
  const float s = __fadd_rn(log_alpha, log_norm);
  if (score_dtype == 1 && kv_dtype == TKV_BF16) return __bfloat162float(__float2bfloat16_rn(s));
  if (score_dtype == 2 && kv_dtype == TKV_F16) return __half2float(__float2half_rn(s));
  return s;
}

struct EvictParams {
  char* k; char* v; float* beta; int32_t* pos;
  int32_t* seg_len;
  int nseg; int64_t cap; int row_vecs; int64_t q_idx;
  int m, trigger_len, max_len;
  const int32_t* keep_cnt;   // per-segment number of rows to keep (NULL: m for every segment at or above trigger_len)
  int protect_last;          // the newest `protect_last` rows always score +inf (sliding window)
  int knorm, kv_dtype;       // knorm: score += log ||k||  (strategy "knorm_alpha")
  int score_dtype;           // dtype the retention score is computed in (retention_score_as)
  const float* scores;       // precomputed scores [nseg*cap] (tkv_flat_scores), or NULL: computed here
  int32_t* kept_idx_out; int32_t* status;
  // Plan mode (several CTAs per segment move the rows afterwards): the kept list and {rows kept, first row that
  // moves} go to global memory and nothing is moved here.
  int32_t* plan; int32_t* plan_kept; int64_t plan_stride;
  int32_t* plan_tail; int ctas, tail_max;   // plan_tail[seg, c]: first row of CTA c's range that it must stage
  int32_t* fired_count; int32_t* fired;     // segments that evict, in the order they finished selecting; *fired_count
                                            // holds their number minus one (the workspace is preset to 0xFF bytes)
};

template <int kThreads>
__global__ void __launch_bounds__(kThreads, 1024 / kThreads) evict_inplace_kernel(EvictParams p) {
  extern __shared__ __align__(16) uint32_t keys[];
  __shared__ SelectScratch sc;
  const int seg = blockIdx.x;
  const int n = p.seg_len[seg];
  const int m = p.keep_cnt != nullptr ? p.keep_cnt[seg] : p.m;
  if (p.keep_cnt == nullptr ? (n < p.trigger_len || n <= m) : (m >= n || m < 0)) return;
  if (n > p.max_len || n > p.cap) {
    if (threadIdx.x == 0) report(p.status, TKV_DEV_LEN_BOUND);
    return;
  }
  if (m == 0) {
    if (threadIdx.x == 0) p.seg_len[seg] = 0;
    return;
  }
  const int64_t row0 = (int64_t)seg * p.cap;
  if (p.scores != nullptr) {
    for (int i = threadIdx.x; i < n; i += kThreads)
      keys[i] = i >= n - p.protect_last ? score_key(INFINITY) : score_key(p.scores[row0 + i]);
  } else if (p.knorm) {
    // strategy "knorm_alpha" (src/trimkv/cache_utils.py:176-180): score = log_alpha + log(||k||).  A warp per row.
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const char* kb = p.k + row0 * (int64_t)p.row_vecs * 16;
    for (int i = warp; i < n; i += kThreads / 32) {
      const float lg = log_row_norm(kb + (int64_t)i * p.row_vecs * 16, p.row_vecs, p.kv_dtype, lane, p.knorm == 2);
      if (lane == 0) {
        const float sc_ = knorm_score(retention_score_as(p.beta[row0 + i], p.pos[row0 + i], p.q_idx, p.score_dtype), lg,
                                      p.score_dtype, p.kv_dtype);
        keys[i] = i >= n - p.protect_last ? score_key(INFINITY) : score_key(sc_);
      }
    }
  } else {
    for (int i = threadIdx.x; i < n; i += kThreads)
      keys[i] = i >= n - p.protect_last ? score_key(INFINITY)
                                        : score_key(retention_score_as(p.beta[row0 + i], p.pos[row0 + i], p.q_idx, p.score_dtype));
  }
  __syncthreads();
  uint32_t thresh; int n_eq_keep;
  radix_select_mth<kThreads>(keys, n, m, &sc, &thresh, &n_eq_keep);
  const int j0 = build_kept_list<kThreads>(keys, n, thresh, n_eq_keep, &sc);
  const int32_t* kept = reinterpret_cast<const int32_t*>(keys);
  if (p.kept_idx_out != nullptr)
    for (int j = threadIdx.x; j < m; j += kThreads) p.kept_idx_out[(int64_t)seg * p.m + j] = kept[j];
  if (p.plan != nullptr) {
    for (int j = j0 + threadIdx.x; j < m; j += kThreads) p.plan_kept[(int64_t)seg * p.plan_stride + j] = kept[j];
    if (threadIdx.x == 0) {
      p.plan[2 * seg] = m; p.plan[2 * seg + 1] = min(j0, m);
      p.fired[atomicAdd(p.fired_count, 1) + 1] = seg;
    }
    if ((int)threadIdx.x < p.ctas) {
      // First row of the range whose source the right neighbour may overwrite (kept is ascending).  The last CTA
      // with rows has no such neighbour: sources at or beyond m are written by nobody.
      const int nvec2 = 2 * p.row_vecs;
      int lo, hi, per;
      move_range(m, min(j0, m), p.ctas, p.tail_max, min(kMoveThreads, (kMoveThreads * kEvictUnroll) / nvec2),
                 threadIdx.x, &lo, &hi, &per);
      int a = lo, b = hi;
      if (hi < m) while (a < b) { const int mid = (a + b) >> 1; if (kept[mid] >= hi) b = mid; else a = mid + 1; }
      else a = hi;
      p.plan_tail[(int64_t)seg * p.ctas + threadIdx.x] = a;
    }
    return;
  }

  // Stable in-place compaction of rows j0..m (rows before the first evicted one stay where they are).
  const int nvec = 2 * p.row_vecs;                       // K vectors then V vectors of one token
  const int tile_rows = min(kThreads, (kThreads * kEvictUnroll) / nvec);
  const int64_t row_bytes = (int64_t)p.row_vecs * 16;
  char* kbase = p.k + row0 * row_bytes;
  char* vbase = p.v + row0 * row_bytes;
  const TileMap tm = make_tile_map<kThreads>(nvec, p.row_vecs, kbase, vbase);
#pragma unroll 1
  for (int jb = j0; jb < m; jb += tile_rows) {
    const int rows = min(tile_rows, m - jb);
    uint4 reg[kEvictUnroll];
#pragma unroll
    for (int u = 0; u < kEvictUnroll; ++u) {
      const int r = tile_row<kThreads>(tm, u);
      if (r < rows) reg[u] = ld16(tile_ptr<kThreads>(tm, u, r, kept[jb + r], row_bytes, p.row_vecs, kbase, vbase));
    }
    float bt = 0.f; int32_t ps = 0;
    if (threadIdx.x < rows) {
      const int src = kept[jb + threadIdx.x];
      bt = p.beta[row0 + src];
      ps = p.pos[row0 + src];
    }
    __syncthreads();  // every load of this tile is performed before any of its stores
#pragma unroll
    for (int u = 0; u < kEvictUnroll; ++u) {
      const int r = tile_row<kThreads>(tm, u);
      if (r < rows) st16(tile_ptr<kThreads>(tm, u, r, jb + r, row_bytes, p.row_vecs, kbase, vbase), reg[u]);
    }
    if (threadIdx.x < rows) {
      p.beta[row0 + jb + threadIdx.x] = bt;
      p.pos[row0 + jb + threadIdx.x] = ps;
    }
  }
  if (threadIdx.x == 0) p.seg_len[seg] = m;
}

// ---- Several CTAs per segment -------------------------------------------------------------------------------------
// When few segments evict at once (one request, or the steady state where a segment fires every B steps), one CTA
// per segment leaves most SMs idle while each firing segment moves megabytes alone.  Here the selection runs first
// (evict_inplace_kernel in plan mode) and `ctas` CTAs then share the rows of one segment: CTA c owns destination
// rows [lo_c, hi_c).  Row j comes from kept[j] >= j, and kept[j] - j never exceeds the rows evicted, so CTA c reads
// rows in [lo_c, hi_c + E) and writes [lo_c, hi_c): the only conflict is with its right neighbour, whose
// destinations cover the last sources of CTA c.  Order of work in each CTA:
//   1. stage the "tail" (rows whose source lies at or beyond hi_c; at most E of them) in shared memory;
//   2. raise flag[c] (release): the neighbour may now overwrite those sources;
//   3. wait for flag[c-1] (acquire, bounded);
//   4. move the remaining rows tile by tile exactly as the one-CTA kernel does, then store the tail.
// A CTA only waits for a lower-numbered one that raises its flag before waiting itself, so the chain cannot
// dead-lock as long as blocks are dispatched in index order; the wait is bounded anyway and reports a timeout.
struct MoveParams {
  char* k; char* v; float* beta; int32_t* pos; int32_t* seg_len;
  int64_t cap; int row_vecs; int ctas; int tail_max;
  const int32_t* plan; const int32_t* plan_tail; const int32_t* kept; int64_t kept_stride;
  int32_t* flags; int32_t* status;
  const int32_t* fired_count; const int32_t* fired;
};

__device__ __forceinline__ int ld_acquire(const int32_t* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.b32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release(int32_t* p, int v) {
  asm volatile("st.release.gpu.global.b32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// CTA c's share of one evicting segment.  Every return is taken by the whole CTA.
__device__ __forceinline__ void move_segment_part(const MoveParams& p, const int seg, const int c, uint4* tail_kv, int& s_ok) {
  constexpr int kThreads = kMoveThreads;
  const int m = p.plan[2 * seg];
  if (m < 0) return;                                  // this segment keeps everything
  const int j0 = p.plan[2 * seg + 1];
  const int nvec = 2 * p.row_vecs;
  const int tile_rows = min(kThreads, (kThreads * kEvictUnroll) / nvec);
  int lo, hi, per;
  move_range(m, j0, p.ctas, p.tail_max, tile_rows, c, &lo, &hi, &per);
  int32_t* flag = p.flags + (int64_t)seg * p.ctas + c;
  if (lo >= hi) {
    if (threadIdx.x == 0) { st_release(flag, 1); if (c == 0) p.seg_len[seg] = m; }
    return;
  }
  const int32_t* kept = p.kept + (int64_t)seg * p.kept_stride;
  const int64_t row0 = (int64_t)seg * p.cap;
  const int64_t row_bytes = (int64_t)p.row_vecs * 16;
  char* kbase = p.k + row0 * row_bytes;
  char* vbase = p.v + row0 * row_bytes;
  const TileMap tm = make_tile_map<kThreads>(nvec, p.row_vecs, kbase, vbase);
  const int jt = min(max(p.plan_tail[(int64_t)seg * p.ctas + c], lo), hi);   // first row to stage (selection kernel)
  const int ntail = hi - jt;
  float* tail_beta = reinterpret_cast<float*>(tail_kv + (int64_t)p.tail_max * nvec);
  int32_t* tail_pos = reinterpret_cast<int32_t*>(tail_beta + p.tail_max);
  const bool tail_fits = ntail <= p.tail_max && kept[hi - 1] - (hi - 1) <= per;
  if (tail_fits) {
    // A tile at a time: all index loads, then all row loads, then the shared-memory stores.
#pragma unroll 1
    for (int rb = 0; rb < ntail; rb += tile_rows) {
      int src[kEvictUnroll]; uint4 val[kEvictUnroll];
#pragma unroll
      for (int u = 0; u < kEvictUnroll; ++u) {
        const int r = rb + tile_row<kThreads>(tm, u);
        src[u] = r < ntail ? kept[jt + r] : 0;   // (rows past the tile are fetched again by the next round: harmless)
      }
#pragma unroll
      for (int u = 0; u < kEvictUnroll; ++u) {
        const int r = tile_row<kThreads>(tm, u);
        if (rb + r < ntail) val[u] = ld16(tile_ptr<kThreads>(tm, u, r, src[u], row_bytes, p.row_vecs, kbase, vbase));
      }
#pragma unroll
      for (int u = 0; u < kEvictUnroll; ++u) {
        const int r = tile_row<kThreads>(tm, u);
        if (rb + r < ntail) tail_kv[(rb + r) * nvec + tile_col<kThreads>(tm, u, r)] = val[u];
      }
    }
    for (int r = threadIdx.x; r < ntail; r += kThreads) {
      const int src = kept[jt + r];
      tail_beta[r] = p.beta[row0 + src]; tail_pos[r] = p.pos[row0 + src];
    }
  }
  __syncthreads();                                    // the staged values have arrived: the loads are performed
  if (threadIdx.x == 0) {
    st_release(flag, 1);
    int ok = tail_fits ? 1 : 0;
    if (!tail_fits) report(p.status, TKV_DEV_CAPACITY);
    if (ok && c > 0) {
      int spins = 0;
      while (ld_acquire(flag - 1) != 1) {
        if (++spins > (1 << 21)) { ok = 0; report(p.status, TKV_DEV_TIMEOUT); break; }
        __nanosleep(100);
      }
    }
    s_ok = ok;
  }
  __syncthreads();
  if (!s_ok) return;                                  // nothing of this range was written

  // Source rows of the next tile are fetched while this tile's rows are in flight, so that the dependent
  // index -> row loads do not add up.
  int src_row[kEvictUnroll], src_meta = 0;
  auto fetch_indices = [&](int jb) {
    const int rows = min(tile_rows, jt - jb);
#pragma unroll
    for (int u = 0; u < kEvictUnroll; ++u) {
      const int r = tile_row<kThreads>(tm, u);
      src_row[u] = r < rows ? kept[jb + r] : 0;
    }
    src_meta = (int)threadIdx.x < rows ? kept[jb + threadIdx.x] : 0;
  };
  if (lo < jt) fetch_indices(lo);
#pragma unroll 1
  for (int jb = lo; jb < jt; jb += tile_rows) {
    const int rows = min(tile_rows, jt - jb);
    uint4 reg[kEvictUnroll];
#pragma unroll
    for (int u = 0; u < kEvictUnroll; ++u) {
      const int r = tile_row<kThreads>(tm, u);
      if (r < rows) reg[u] = ld16(tile_ptr<kThreads>(tm, u, r, src_row[u], row_bytes, p.row_vecs, kbase, vbase));
    }
    float bt = 0.f; int32_t ps = 0;
    if (threadIdx.x < rows) { bt = p.beta[row0 + src_meta]; ps = p.pos[row0 + src_meta]; }
    if (jb + tile_rows < jt) fetch_indices(jb + tile_rows);
    __syncthreads();  // every load of this tile is performed before any of its stores
#pragma unroll
    for (int u = 0; u < kEvictUnroll; ++u) {
      const int r = tile_row<kThreads>(tm, u);
      if (r < rows) st16(tile_ptr<kThreads>(tm, u, r, jb + r, row_bytes, p.row_vecs, kbase, vbase), reg[u]);
    }
    if (threadIdx.x < rows) { p.beta[row0 + jb + threadIdx.x] = bt; p.pos[row0 + jb + threadIdx.x] = ps; }
  }
  __syncthreads();    // the last tile's loads may have read rows of the tail's destination
#pragma unroll 1
  for (int rb = 0; rb < ntail; rb += tile_rows) {
#pragma unroll
    for (int u = 0; u < kEvictUnroll; ++u) {
      const int r = tile_row<kThreads>(tm, u);
      if (rb + r < ntail)
        st16(tile_ptr<kThreads>(tm, u, r, jt + rb + r, row_bytes, p.row_vecs, kbase, vbase),
             tail_kv[(rb + r) * nvec + tile_col<kThreads>(tm, u, r)]);
    }
  }
  for (int r = threadIdx.x; r < ntail; r += kThreads) {
    p.beta[row0 + jt + r] = tail_beta[r]; p.pos[row0 + jt + r] = tail_pos[r];
  }
  if (c == 0 && threadIdx.x == 0) p.seg_len[seg] = m;
}

// Grid (ctas, Y): the CTAs with blockIdx.y = y take the evicting segments fired[y], fired[y + Y], ... in turn, so the
// grid is sized by the SMs and not by the segments: when one segment in a hundred evicts (the steady state), a grid of
// ctas x nseg blocks would spend its time launching blocks that find nothing to do.  CTA (c, y) still waits only for
// CTA (c-1, y) working on the same segment, which has a lower block index and handles its segments in the same order.
__global__ void __launch_bounds__(kMoveThreads) evict_move_kernel(MoveParams p) {
  extern __shared__ __align__(16) uint4 tail_kv[];   // [tail_max][2 * row_vecs], then beta[tail_max], pos[tail_max]
  __shared__ int s_ok;
  const int count = *p.fired_count + 1;
  for (int i = blockIdx.y; i < count; i += gridDim.y) {
    move_segment_part(p, p.fired[i], blockIdx.x, tail_kv, s_ok);
    __syncthreads();   // the staging area and s_ok are reused by the next segment
  }
}

struct SelectParams {
  const float* beta; int64_t beta_stride; const int32_t* pos; int64_t pos_stride;
  const int32_t* seg_len; int n_uniform; int nseg; int64_t q_idx;
  int m, trigger_len, max_len;
  int32_t* kept_idx; int32_t* kept_cnt; int32_t* status;
};

__global__ void __launch_bounds__(kEvictThreads) evict_select_kernel(SelectParams p) {
  extern __shared__ __align__(16) uint32_t keys[];
  __shared__ SelectScratch sc;
  const int seg = blockIdx.x;
  const int n = p.seg_len != nullptr ? p.seg_len[seg] : p.n_uniform;
  if (n < p.trigger_len || n <= p.m) {
    if (threadIdx.x == 0) p.kept_cnt[seg] = max(n, 0);
    return;
  }
  if (n > p.max_len) {
    if (threadIdx.x == 0) { report(p.status, TKV_DEV_LEN_BOUND); p.kept_cnt[seg] = n; }
    return;
  }
  const float* beta = p.beta + (int64_t)seg * p.beta_stride;
  const int32_t* pos = p.pos + (int64_t)seg * p.pos_stride;
  for (int i = threadIdx.x; i < n; i += kEvictThreads)
    keys[i] = score_key(retention_score(beta[i], pos[i], p.q_idx));
  __syncthreads();
  uint32_t thresh; int n_eq_keep;
  radix_select_mth<kEvictThreads>(keys, n, p.m, &sc, &thresh, &n_eq_keep);
  build_kept_list<kEvictThreads>(keys, n, thresh, n_eq_keep, &sc);
  const int32_t* kept = reinterpret_cast<const int32_t*>(keys);
  for (int j = threadIdx.x; j < p.m; j += kEvictThreads) p.kept_idx[(int64_t)seg * p.m + j] = kept[j];
  if (threadIdx.x == 0) p.kept_cnt[seg] = p.m;
}

struct CompactParams {
  char* k_dst; char* v_dst; float* beta_dst; int32_t* pos_dst; int64_t cap;
  const char* k_src; const char* v_src; int64_t k_sb, k_sh, k_ss;  // byte strides
  const float* beta_src; int64_t beta_stride; const int32_t* pos_src; int64_t pos_stride;
  const int32_t* kept_idx; int64_t kept_stride; const int32_t* kept_cnt;
  int32_t* seg_len; int hkv, n_src, row_vecs;
  int32_t* status;
};

constexpr int kCompactRows = 32;
// Out-of-place gather: any number of CTAs per segment, no ordering hazards.
__global__ void __launch_bounds__(256) compact_gather_kernel(CompactParams p) {
  const int seg = blockIdx.y;
  const int cnt = p.kept_cnt != nullptr ? p.kept_cnt[seg] : p.n_src;
  const int jb = blockIdx.x * kCompactRows;
  if (blockIdx.x == 0 && threadIdx.x == 0) p.seg_len[seg] = min(cnt, (int)min((int64_t)INT32_MAX, p.cap));
  if (jb >= cnt) return;
  if (cnt > p.cap) {
    if (threadIdx.x == 0) report(p.status, TKV_DEV_CAPACITY);
    return;
  }
  const bool identity = p.kept_idx == nullptr || cnt == p.n_src;
  const int32_t* kept = identity ? nullptr : p.kept_idx + (int64_t)seg * p.kept_stride;
  const int b = seg / p.hkv, h = seg - b * p.hkv;
  const int rows = min(kCompactRows, cnt - jb);
  const int nvec = 2 * p.row_vecs;
  const int64_t row_bytes = (int64_t)p.row_vecs * 16;
  const int64_t dst_row0 = (int64_t)seg * p.cap;
  const char* ksrc = p.k_src + b * p.k_sb + h * p.k_sh;
  const char* vsrc = p.v_src + b * p.k_sb + h * p.k_sh;
  for (int i = threadIdx.x; i < rows * nvec; i += blockDim.x) {
    const int r = i / nvec, c = i - r * nvec;
    const int src = identity ? jb + r : kept[jb + r];
    if ((unsigned)src >= (unsigned)p.n_src) { report(p.status, TKV_DEV_BAD_INDEX); continue; }
    const bool is_v = c >= p.row_vecs;
    const int cc = is_v ? c - p.row_vecs : c;
    const char* sp = (is_v ? vsrc : ksrc) + (int64_t)src * p.k_ss + (int64_t)cc * 16;
    char* dp = (is_v ? p.v_dst : p.k_dst) + (dst_row0 + jb + r) * row_bytes + (int64_t)cc * 16;
    st16(dp, ld16_stream(sp));
  }
  for (int r = threadIdx.x; r < rows; r += blockDim.x) {
    const int src = identity ? jb + r : kept[jb + r];
    if ((unsigned)src >= (unsigned)p.n_src) continue;
    p.beta_dst[dst_row0 + jb + r] = p.beta_src[(int64_t)seg * p.beta_stride + src];
    p.pos_dst[dst_row0 + jb + r] = p.pos_src[(int64_t)seg * p.pos_stride + src];
  }
}

// cu_seqlens[g, 0..group] = exclusive prefix sum of seg_len[g*group ..]; one CTA per group.
// Four consecutive lengths per thread, so that a group of up to 1024 segments (4096 with the wide block) takes one scan.
template <int kThreads>
__global__ void __launch_bounds__(kThreads) rebuild_cu_kernel(const int32_t* seg_len, int32_t* cu, int group) {
  __shared__ int warp_sums[kThreads / 32 + 1];
  const int g = blockIdx.x;
  const int32_t* len = seg_len + (int64_t)g * group;
  int32_t* out = cu + (int64_t)g * (group + 1);
  int running = 0;
  for (int base = 0; base < group; base += 4 * kThreads) {
    const int i0 = base + 4 * (int)threadIdx.x;
    int v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = i0 + u < group ? len[i0 + u] : 0;
    int total;
    int at = running + block_exclusive_scan<kThreads>(v[0] + v[1] + v[2] + v[3], warp_sums, &total);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (i0 + u < group) out[i0 + u] = at;
      at += v[u];
    }
    running += total;
  }
  if (threadIdx.x == 0) out[group] = running;
}

static int launch_rebuild(const int32_t* seg_len, int32_t* cu, int nseg, int group, cudaStream_t st) {
  if (cu == nullptr || nseg == 0) return TKV_OK;
  if (group <= 0 || nseg % group != 0)
    return fail(TKV_ERR_ARG, "cu_seqlens rebuild: nseg=%d is not a multiple of group=%d", nseg, group);
  if (group > 1024) rebuild_cu_kernel<1024><<<nseg / group, 1024, 0, st>>>(seg_len, cu, group);
  else rebuild_cu_kernel<256><<<nseg / group, 256, 0, st>>>(seg_len, cu, group);
  return check_launch("tkv_rebuild_cu_seqlens");
}

template <typename K>
static int set_smem(K kernel, size_t bytes, const char* what) {
  if (bytes > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return fail(TKV_ERR_LAUNCH, "%s: shared memory %zu: %s", what, bytes, cudaGetErrorString(e));
  }
  return TKV_OK;
}

}  // namespace tkv

extern "C" int tkv_rebuild_cu_seqlens(const int32_t* seg_len, int32_t* cu_seqlens, int nseg, int group,
                                      tkv_stream_t stream) {
  if (!seg_len || !cu_seqlens) return tkv::fail(TKV_ERR_ARG, "tkv_rebuild_cu_seqlens: NULL pointer argument");
  if (nseg < 0) return tkv::fail(TKV_ERR_ARG, "tkv_rebuild_cu_seqlens: nseg=%d", nseg);
  return tkv::launch_rebuild(seg_len, cu_seqlens, nseg, group, (cudaStream_t)stream);
}

static int evict_impl(void* k_cache, void* v_cache, float* beta_cache, int32_t* pos_cache,
                      int32_t* seg_len, int32_t* cu_seqlens, int group,
                      int nseg, int64_t cap, int head_dim, int kv_dtype, int64_t q_idx,
                      int memory_size, int trigger_len, int max_len, const int32_t* keep_cnt, int protect_last,
                      int strategy, int32_t* kept_idx_out, int32_t* status, tkv_stream_t stream,
                      int ctas = 1, void* workspace = nullptr, int64_t workspace_bytes = 0, const float* scores = nullptr) {
  using namespace tkv;
  const int es = elem_size(kv_dtype);
  if (es == 0) return fail(TKV_ERR_ARG, "tkv_evict: unknown kv_dtype %d", kv_dtype);
  if (!k_cache || !v_cache || !beta_cache || !pos_cache || !seg_len)
    return fail(TKV_ERR_ARG, "tkv_evict: NULL pointer argument");
  const int score_dtype = (strategy >> 8) & 3;
  strategy &= 0xff;
  if (strategy < 0 || strategy > 2 || score_dtype > 2) return fail(TKV_ERR_ARG, "tkv_evict: unknown strategy %d", strategy);
  if (nseg < 0 || cap <= 0 || head_dim <= 0 || memory_size <= 0 || max_len <= 0 || protect_last < 0)
    return fail(TKV_ERR_ARG, "tkv_evict: bad sizes nseg=%d cap=%lld head_dim=%d M=%d max_len=%d", nseg,
                (long long)cap, head_dim, memory_size, max_len);
  if (max_len > kMaxSelectLen)
    return fail(TKV_ERR_UNSUPPORTED, "tkv_evict: max_len=%d exceeds %d", max_len, kMaxSelectLen);
  const int64_t row_bytes = (int64_t)head_dim * es;
  if (row_bytes % 16 != 0 || 2 * (row_bytes / 16) > kEvictThreads * kEvictUnroll)  // one token must fit a tile
    return fail(TKV_ERR_ARG, "tkv_evict: unsupported row of %lld bytes", (long long)row_bytes);
  if (!aligned16(k_cache) || !aligned16(v_cache)) return fail(TKV_ERR_ARG, "tkv_evict: K/V must be 16-byte aligned");
  if (nseg == 0) return TKV_OK;
  EvictParams p;
  p.k = (char*)k_cache; p.v = (char*)v_cache; p.beta = beta_cache; p.pos = pos_cache; p.seg_len = seg_len;
  p.nseg = nseg; p.cap = cap; p.row_vecs = (int)(row_bytes / 16); p.q_idx = q_idx;
  p.m = memory_size; p.trigger_len = trigger_len; p.max_len = max_len;
  p.keep_cnt = keep_cnt; p.protect_last = protect_last; p.knorm = strategy; p.kv_dtype = kv_dtype;
  p.score_dtype = score_dtype; p.scores = scores;
  p.kept_idx_out = kept_idx_out; p.status = status;
  p.plan = nullptr; p.plan_kept = nullptr; p.plan_stride = 0; p.plan_tail = nullptr; p.ctas = 1; p.tail_max = 0;
  p.fired_count = nullptr; p.fired = nullptr;
  MoveParams mp;
  size_t move_smem = 0;
  if (ctas > 1) {
    // Workspace: flags [nseg, ctas] | plan [nseg, 2] | fired count [1] | fired [nseg] | plan_tail [nseg, ctas] |
    // kept [nseg, memory_size], all int32.
    if (keep_cnt != nullptr) return fail(TKV_ERR_UNSUPPORTED, "tkv_evict_multi: per-segment keep counts are not supported");
    if (ctas > kEvictMaxCtas || nseg > 65535)
      return fail(TKV_ERR_UNSUPPORTED, "tkv_evict_multi: ctas_per_segment=%d (limit %d), nseg=%d (limit 65535)", ctas, kEvictMaxCtas, nseg);
    const int64_t need = tkv_evict_multi_workspace_bytes(nseg, memory_size, ctas);
    if (workspace == nullptr || workspace_bytes < need || ((uintptr_t)workspace & 3))
      return fail(TKV_ERR_ARG, "tkv_evict_multi: workspace of %lld bytes, %lld needed", (long long)workspace_bytes, (long long)need);
    mp.tail_max = max_len - memory_size;               // no row moves further than the rows evicted before it
    move_smem = (size_t)mp.tail_max * (2 * row_bytes + 8);
    if (mp.tail_max <= 0 || move_smem > 200 * 1024)
      return fail(TKV_ERR_UNSUPPORTED, "tkv_evict_multi: max_len - memory_size = %d rows do not fit the staging area", mp.tail_max);
    int32_t* w = (int32_t*)workspace;
    mp.flags = w; p.plan = w + (int64_t)nseg * ctas; p.fired_count = p.plan + 2 * (int64_t)nseg; p.fired = p.fired_count + 1;
    p.plan_tail = p.fired + nseg; mp.fired_count = p.fired_count; mp.fired = p.fired;
    p.plan_kept = p.plan_tail + (int64_t)nseg * ctas; p.plan_stride = memory_size;
    p.ctas = ctas; p.tail_max = mp.tail_max; mp.plan_tail = p.plan_tail;
    mp.k = p.k; mp.v = p.v; mp.beta = p.beta; mp.pos = p.pos; mp.seg_len = seg_len; mp.cap = cap; mp.row_vecs = p.row_vecs;
    mp.ctas = ctas; mp.plan = p.plan; mp.kept = p.plan_kept; mp.kept_stride = memory_size; mp.status = status;
    // flags = -1 (not raised), plan = -1 (segment keeps everything), fired count = -1 (none) until the selection says
    // otherwise
    cudaError_t e = cudaMemsetAsync(workspace, 0xFF, ((size_t)nseg * ctas + 2 * (size_t)nseg + 1) * 4, (cudaStream_t)stream);
    if (e != cudaSuccess) return fail(TKV_ERR_LAUNCH, "tkv_evict_multi: memset: %s", cudaGetErrorString(e));
  }
  const size_t smem = (size_t)max_len * 4;
  // Long segments: the key array leaves room for at most 3 CTAs per SM, so each CTA gets twice the threads (and
  // twice the rows in flight per tile) to keep the memory system as busy as 4 narrow CTAs do.
  const bool wide = smem > 56 * 1024;
  int rc = wide ? set_smem(evict_inplace_kernel<kEvictThreadsWide>, smem, "tkv_evict")
                : set_smem(evict_inplace_kernel<kEvictThreads>, smem, "tkv_evict");
  if (rc != TKV_OK) return rc;
  if (ctas > 1) {
    rc = set_smem(evict_inplace_kernel<kEvictThreadsPlan>, smem, "tkv_evict_multi");
    if (rc != TKV_OK) return rc;
    evict_inplace_kernel<kEvictThreadsPlan><<<nseg, kEvictThreadsPlan, smem, (cudaStream_t)stream>>>(p);
  } else if (wide) evict_inplace_kernel<kEvictThreadsWide><<<nseg, kEvictThreadsWide, smem, (cudaStream_t)stream>>>(p);
  else evict_inplace_kernel<kEvictThreads><<<nseg, kEvictThreads, smem, (cudaStream_t)stream>>>(p);
  rc = check_launch("tkv_evict");
  if (rc != TKV_OK) return rc;
  if (ctas > 1) {
    rc = set_smem(evict_move_kernel, move_smem, "tkv_evict_multi");
    if (rc != TKV_OK) return rc;
    const int rows_y = nseg < kMoveGridCtas / ctas ? nseg : kMoveGridCtas / ctas;
    evict_move_kernel<<<dim3((unsigned)ctas, (unsigned)rows_y), kMoveThreads, move_smem, (cudaStream_t)stream>>>(mp);
    rc = check_launch("tkv_evict_multi");
    if (rc != TKV_OK) return rc;
  }
  return launch_rebuild(seg_len, cu_seqlens, nseg, group, (cudaStream_t)stream);
}

extern "C" int64_t tkv_evict_multi_workspace_bytes(int nseg, int memory_size, int ctas_per_segment) {
  if (nseg < 0 || memory_size <= 0 || ctas_per_segment <= 0) return 0;
  return (2 * (int64_t)nseg * ctas_per_segment + 3 * (int64_t)nseg + 1 + (int64_t)nseg * memory_size) * 4;
}

extern "C" int tkv_evict_multi(void* k_cache, void* v_cache, float* beta_cache, int32_t* pos_cache,
                               int32_t* seg_len, int32_t* cu_seqlens, int group,
                               int nseg, int64_t cap, int head_dim, int kv_dtype, int64_t q_idx,
                               int memory_size, int trigger_len, int max_len, int protect_last, int strategy,
                               int ctas_per_segment, void* workspace, int64_t workspace_bytes,
                               int32_t* kept_idx_out, int32_t* status, tkv_stream_t stream) {
  if (ctas_per_segment < 1) return tkv::fail(TKV_ERR_ARG, "tkv_evict_multi: ctas_per_segment=%d", ctas_per_segment);
  return evict_impl(k_cache, v_cache, beta_cache, pos_cache, seg_len, cu_seqlens, group, nseg, cap, head_dim, kv_dtype,
                    q_idx, memory_size, trigger_len, max_len, nullptr, protect_last, strategy, kept_idx_out, status, stream,
                    ctas_per_segment, workspace, workspace_bytes);
}

extern "C" int tkv_evict(void* k_cache, void* v_cache, float* beta_cache, int32_t* pos_cache,
                         int32_t* seg_len, int32_t* cu_seqlens, int group,
                         int nseg, int64_t cap, int head_dim, int kv_dtype, int64_t q_idx,
                         int memory_size, int trigger_len, int max_len,
                         int32_t* kept_idx_out, int32_t* status, tkv_stream_t stream) {
  return evict_impl(k_cache, v_cache, beta_cache, pos_cache, seg_len, cu_seqlens, group, nseg, cap, head_dim, kv_dtype,
                    q_idx, memory_size, trigger_len, max_len, nullptr, 0, 0, kept_idx_out, status, stream);
}

extern "C" int tkv_evict_ex(void* k_cache, void* v_cache, float* beta_cache, int32_t* pos_cache,
                            int32_t* seg_len, int32_t* cu_seqlens, int group,
                            int nseg, int64_t cap, int head_dim, int kv_dtype, int64_t q_idx,
                            int memory_size, int trigger_len, int max_len,
                            const int32_t* keep_cnt, int protect_last, int kept_stride, int strategy,
                            const float* scores, int32_t* kept_idx_out, int32_t* status, tkv_stream_t stream) {
  // kept_stride doubles as the row stride of kept_idx_out when keep counts vary per segment.
  return evict_impl(k_cache, v_cache, beta_cache, pos_cache, seg_len, cu_seqlens, group, nseg, cap, head_dim, kv_dtype,
                    q_idx, keep_cnt != nullptr ? (kept_stride > 0 ? kept_stride : 1) : memory_size, trigger_len, max_len,
                    keep_cnt, protect_last, strategy, kept_idx_out, status, stream, 1, nullptr, 0, scores);
}

extern "C" int tkv_evict_select(const float* beta, int64_t beta_stride, const int32_t* pos, int64_t pos_stride,
                                const int32_t* seg_len, int n_uniform, int nseg, int64_t q_idx,
                                int memory_size, int trigger_len, int max_len,
                                int32_t* kept_idx, int32_t* kept_cnt, int32_t* status, tkv_stream_t stream) {
  using namespace tkv;
  if (!beta || !pos || !kept_idx || !kept_cnt) return fail(TKV_ERR_ARG, "tkv_evict_select: NULL pointer argument");
  if (nseg < 0 || memory_size <= 0 || max_len <= 0 || (seg_len == nullptr && n_uniform < 0))
    return fail(TKV_ERR_ARG, "tkv_evict_select: bad sizes nseg=%d M=%d max_len=%d", nseg, memory_size, max_len);
  if (seg_len == nullptr && n_uniform > max_len)
    return fail(TKV_ERR_ARG, "tkv_evict_select: n_uniform=%d > max_len=%d", n_uniform, max_len);
  if (max_len > kMaxSelectLen)
    return fail(TKV_ERR_UNSUPPORTED, "tkv_evict_select: max_len=%d exceeds %d", max_len, kMaxSelectLen);
  if (nseg == 0) return TKV_OK;
  SelectParams p;
  p.beta = beta; p.beta_stride = beta_stride; p.pos = pos; p.pos_stride = pos_stride;
  p.seg_len = seg_len; p.n_uniform = n_uniform; p.nseg = nseg; p.q_idx = q_idx;
  p.m = memory_size; p.trigger_len = trigger_len; p.max_len = max_len;
  p.kept_idx = kept_idx; p.kept_cnt = kept_cnt; p.status = status;
  const size_t smem = (size_t)max_len * 4;
  int rc = set_smem(evict_select_kernel, smem, "tkv_evict_select");
  if (rc != TKV_OK) return rc;
  evict_select_kernel<<<nseg, kEvictThreads, smem, (cudaStream_t)stream>>>(p);
  return check_launch("tkv_evict_select");
}

extern "C" int tkv_compact(void* k_dst, void* v_dst, float* beta_dst, int32_t* pos_dst, int64_t cap,
                           const void* k_src, const void* v_src, int64_t k_sb, int64_t k_sh, int64_t k_ss,
                           const float* beta_src, int64_t beta_stride, const int32_t* pos_src, int64_t pos_stride,
                           const int32_t* kept_idx, int64_t kept_stride, const int32_t* kept_cnt,
                           int32_t* seg_len, int32_t* cu_seqlens, int group,
                           int batch, int hkv, int n_src, int head_dim, int kv_dtype,
                           int32_t* status, tkv_stream_t stream) {
  using namespace tkv;
  const int es = elem_size(kv_dtype);
  if (es == 0) return fail(TKV_ERR_ARG, "tkv_compact: unknown kv_dtype %d", kv_dtype);
  if (!k_dst || !v_dst || !beta_dst || !pos_dst || !k_src || !v_src || !beta_src || !pos_src || !seg_len)
    return fail(TKV_ERR_ARG, "tkv_compact: NULL pointer argument");
  if (batch < 0 || hkv <= 0 || n_src < 0 || head_dim <= 0 || cap <= 0)
    return fail(TKV_ERR_ARG, "tkv_compact: bad sizes");
  const int64_t row_bytes = (int64_t)head_dim * es;
  if (row_bytes % 16 != 0) return fail(TKV_ERR_ARG, "tkv_compact: row of %lld bytes is not a multiple of 16", (long long)row_bytes);
  if (!aligned16(k_dst) || !aligned16(v_dst) || !aligned16(k_src) || !aligned16(v_src))
    return fail(TKV_ERR_ARG, "tkv_compact: K/V pointers must be 16-byte aligned");
  if ((k_sb * es) % 16 || (k_sh * es) % 16 || (k_ss * es) % 16)
    return fail(TKV_ERR_ARG, "tkv_compact: K/V strides must be multiples of 16 bytes");
  const int64_t nseg = (int64_t)batch * hkv;
  if (nseg > 65535) return fail(TKV_ERR_UNSUPPORTED, "tkv_compact: more than 65535 segments per call");
  if (nseg == 0) return TKV_OK;
  CompactParams p;
  p.k_dst = (char*)k_dst; p.v_dst = (char*)v_dst; p.beta_dst = beta_dst; p.pos_dst = pos_dst; p.cap = cap;
  p.k_src = (const char*)k_src; p.v_src = (const char*)v_src;
  p.k_sb = k_sb * es; p.k_sh = k_sh * es; p.k_ss = k_ss * es;
  p.beta_src = beta_src; p.beta_stride = beta_stride; p.pos_src = pos_src; p.pos_stride = pos_stride;
  p.kept_idx = kept_idx; p.kept_stride = kept_stride; p.kept_cnt = kept_cnt;
  p.seg_len = seg_len; p.hkv = hkv; p.n_src = n_src; p.row_vecs = (int)(row_bytes / 16); p.status = status;
  const int max_rows = (int)(n_src < cap ? n_src : cap);
  dim3 grid((max_rows + kCompactRows - 1) / kCompactRows > 0 ? (max_rows + kCompactRows - 1) / kCompactRows : 1, (unsigned)nseg);
  compact_gather_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(p);
  int rc = check_launch("tkv_compact");
  if (rc != TKV_OK) return rc;
  return launch_rebuild(seg_len, cu_seqlens, (int)nseg, group, (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------------------------------------
// Budget sharing: how many rows each segment keeps when a token budget is shared by a group of segments.
//
// Replaces the global / layer-wise top-k of the reference's flat caches (src/trimkv/cache_utils.py:371-416
// _compress_layer, :418-536 _compress_all_layers, :740-834 _compress_layer_batched, :836-945
// _compress_all_layers_batched): there the scores of a whole layer (or of all layers) of one request are
// concatenated, torch.topk picks the budget, and Python loops with .item() rebuild the per-head lengths.
// Here one CTA per group streams the scores of its segments, radix-selects the group's threshold, then
// counts per segment how many rows clear it (ties go to the lower concatenated index, i.e. to earlier
// segments first).  Keeping a group's top-k is the same as keeping, in every segment, its own top-c rows for
// these counts c, which is what tkv_evict_ex then does in place.
namespace tkv {

constexpr int kBudgetThreads = 1024;
constexpr int kBudgetMaxSegs = 2048;

struct BudgetParams {
  const float* beta; const int32_t* pos; const int32_t* seg_len; int64_t cap;
  int inner, n_outer; int64_t outer_stride;     // group g = segments {g*inner + o*outer_stride + i}
  int64_t q_idx; int64_t k_total;
  int use_threshold; float threshold;           // keep score >= threshold instead of the k_total best
  int score_dtype;                              // see retention_score_as
  const float* scores;                          // precomputed scores [rows] (tkv_flat_scores) or NULL
  int floor_mode, floor_cnt;                    // 0: none, 1: c = min(n, s' + floor) with the reference's boundary
                                                // attribution for s', 2: c = max(s, min(floor, n))
  int32_t* keep_cnt; int32_t* status;
};

__global__ void __launch_bounds__(kBudgetThreads) group_budget_kernel(BudgetParams p) {
  __shared__ int s_len[kBudgetMaxSegs];
  __shared__ int s_gt[kBudgetMaxSegs];
  __shared__ int s_eq[kBudgetMaxSegs];
  __shared__ int hist[256];
  __shared__ int warp_sums[kBudgetThreads / 32 + 1];
  __shared__ int sel_digit, sel_k;
  __shared__ long long s_total;
  const int tid = threadIdx.x, lane = tid & 31;
  const int nsegs = p.inner * p.n_outer;
  const int64_t base = (int64_t)blockIdx.x * p.inner;
  auto seg_of = [&](int j) { return base + (int64_t)(j / p.inner) * p.outer_stride + (j % p.inner); };
  if (tid == 0) s_total = 0;
  __syncthreads();
  for (int j = tid; j < nsegs; j += kBudgetThreads) {
    const int n = max(p.seg_len[seg_of(j)], 0);
    s_len[j] = n; s_gt[j] = 0; s_eq[j] = 0;
    atomicAdd((unsigned long long*)&s_total, (unsigned long long)n);
  }
  __syncthreads();
  const long long total = s_total;
  uint32_t thresh = 0; long long n_eq_keep = 0;
  bool keep_all = false;
  if (p.use_threshold) {
    thresh = score_key(p.threshold);
    n_eq_keep = total;  // every row equal to the threshold is kept
  } else if (p.k_total >= total) {
    keep_all = true;
  } else if (p.k_total <= 0) {
    thresh = 0xFFFFFFFFu; n_eq_keep = 0;
  } else {
    // 4-pass radix select of the k_total-th largest key over all rows of the group.
    uint32_t prefix = 0, decided = 0;
    long long k = p.k_total;
#pragma unroll 1
    for (int shift = 24; shift >= 0; shift -= 8) {
      if (tid < 256) hist[tid] = 0;
      __syncthreads();
      for (int j = 0; j < nsegs; ++j) {
        const int n = s_len[j];
        const int64_t row0 = seg_of(j) * p.cap;
        const int n_round = (n + kBudgetThreads - 1) / kBudgetThreads * kBudgetThreads;
        for (int i = tid; i < n_round; i += kBudgetThreads) {
          bool valid = i < n;
          uint32_t key = 0;
          if (valid) {
            key = score_key(p.scores != nullptr ? p.scores[row0 + i] : retention_score_as(p.beta[row0 + i], p.pos[row0 + i], p.q_idx, p.score_dtype));
            valid = (key & decided) == prefix;
          }
          const int digit = valid ? (int)((key >> shift) & 255u) : 256 + lane;
          const unsigned peers = __match_any_sync(0xffffffffu, digit);
          if (valid && lane == __ffs(peers) - 1) atomicAdd(&hist[digit], __popc(peers));
        }
      }
      __syncthreads();
      // bins from the top: thread t (< 256) looks at bin 255 - t
      const int bin = 255 - tid;
      const int c = tid < 256 ? hist[bin] : 0;
      int tot;
      const int above = block_exclusive_scan<kBudgetThreads>(c, warp_sums, &tot);
      if (tid < 256 && above < k && k <= (long long)above + c) { sel_digit = bin; sel_k = (int)(k - above); }
      __syncthreads();
      prefix |= (uint32_t)sel_digit << shift;
      decided |= 255u << shift;
      k = sel_k;
      __syncthreads();
    }
    thresh = prefix; n_eq_keep = k;
  }
  if (!keep_all) {
    // Per segment: rows above the threshold and rows equal to it.
    for (int j = 0; j < nsegs; ++j) {
      const int n = s_len[j];
      const int64_t row0 = seg_of(j) * p.cap;
      const int n_round = (n + 31) / 32 * 32;
      for (int i = tid; i < n_round; i += kBudgetThreads) {
        uint32_t key = 0;
        const bool valid = i < n;
        if (valid) key = score_key(p.scores != nullptr ? p.scores[row0 + i] : retention_score_as(p.beta[row0 + i], p.pos[row0 + i], p.q_idx, p.score_dtype));
        const unsigned gt = __ballot_sync(0xffffffffu, valid && key > thresh);
        const unsigned eq = __ballot_sync(0xffffffffu, valid && key == thresh);
        if (lane == 0) {
          if (gt) atomicAdd(&s_gt[j], __popc(gt));
          if (eq) atomicAdd(&s_eq[j], __popc(eq));
        }
      }
    }
    __syncthreads();
  }
  // Ties are granted in concatenated order; then the per-head floor is applied.  Few segments: one thread.
  if (tid == 0) {
    long long eq_before = 0;
    for (int j = 0; j < nsegs; ++j) {
      const int n = s_len[j];
      int s = n;
      long long quota = 0;
      if (!keep_all) {
        quota = n_eq_keep - eq_before;
        quota = quota < 0 ? 0 : (quota > s_eq[j] ? s_eq[j] : quota);
        s = s_gt[j] + (int)quota;
        eq_before += s_eq[j];
      }
      if (p.floor_mode == 1) {
        // Is the segment's first row among the kept ones?  (needed for the attribution below)
        int first = 0;
        if (n > 0) {
          const int64_t row0 = seg_of(j) * p.cap;
          const uint32_t key0 = score_key(p.scores != nullptr ? p.scores[row0] : retention_score_as(p.beta[row0], p.pos[row0], p.q_idx, p.score_dtype));
          first = keep_all || key0 > thresh || (key0 == thresh && quota > 0);
        }
        s_eq[j] = first;
      }
      s_gt[j] = s;
    }
    for (int j = 0; j < nsegs; ++j) {
      const int n = s_len[j];
      const int s = s_gt[j];
      int c = s;
      if (p.floor_mode == 1) {
        // src/trimkv/cache_utils.py:495-499 attributes a selected flat index that equals a head boundary (the
        // first row of the next head) to the previous head, then adds the floor; kept as is for parity.
        const int attributed = s - (j > 0 ? s_eq[j] : 0) + (j + 1 < nsegs ? s_eq[j + 1] : 0);
        c = min(n, attributed + p.floor_cnt);
      } else if (p.floor_mode == 2) {
        c = max(s, min(p.floor_cnt, n));
      }
      p.keep_cnt[seg_of(j)] = c;
    }
  }
}

}  // namespace tkv

extern "C" int tkv_group_budget(const float* beta_cache, const int32_t* pos_cache, const int32_t* seg_len, int64_t cap,
                                int groups, int inner, int n_outer, int64_t outer_stride, int64_t q_idx,
                                int64_t k_total, int use_threshold, float threshold, int floor_mode, int floor_cnt,
                                int score_dtype, const float* scores, int32_t* keep_cnt, int32_t* status,
                                tkv_stream_t stream) {
  using namespace tkv;
  if (!beta_cache || !pos_cache || !seg_len || !keep_cnt) return fail(TKV_ERR_ARG, "tkv_group_budget: NULL pointer argument");
  if (groups < 0 || inner <= 0 || n_outer <= 0 || cap <= 0 || floor_mode < 0 || floor_mode > 2 || floor_cnt < 0 ||
      score_dtype < 0 || score_dtype > 2)
    return fail(TKV_ERR_ARG, "tkv_group_budget: bad sizes groups=%d inner=%d n_outer=%d", groups, inner, n_outer);
  if ((int64_t)inner * n_outer > kBudgetMaxSegs)
    return fail(TKV_ERR_UNSUPPORTED, "tkv_group_budget: %lld segments per group (limit %d)", (long long)inner * n_outer,
                kBudgetMaxSegs);
  if (groups == 0) return TKV_OK;
  BudgetParams p;
  p.beta = beta_cache; p.pos = pos_cache; p.seg_len = seg_len; p.cap = cap;
  p.inner = inner; p.n_outer = n_outer; p.outer_stride = outer_stride; p.q_idx = q_idx; p.k_total = k_total;
  p.use_threshold = use_threshold; p.threshold = threshold; p.floor_mode = floor_mode; p.floor_cnt = floor_cnt;
  p.score_dtype = score_dtype; p.scores = scores;
  p.keep_cnt = keep_cnt; p.status = status;
  group_budget_kernel<<<groups, kBudgetThreads, 0, (cudaStream_t)stream>>>(p);
  return check_launch("tkv_group_budget");
}

// ---------------------------------------------------------------------------------------------------------
// Scores of every live row, written once: for the strategies whose score reads the K rows ("knorm_alpha" and its
// threshold form on the flat caches, src/trimkv/cache_utils.py:388-390, 443-450, 757-759, 876-878) the budget
// kernel would otherwise read K five times.  One warp per row; rows beyond a segment's length are not touched.
namespace tkv {
struct ScoreParams {
  const char* k; const float* beta; const int32_t* pos; const int32_t* seg_len;
  int64_t cap; int row_vecs, kv_dtype, knorm, score_dtype; int64_t q_idx;
  float* scores;
};

__global__ void __launch_bounds__(256) flat_scores_kernel(ScoreParams p) {
  const int seg = blockIdx.y, lane = threadIdx.x & 31;
  const int n = min(max(p.seg_len[seg], 0), (int)min((int64_t)INT32_MAX, p.cap));
  const int64_t row0 = (int64_t)seg * p.cap;
  for (int i = blockIdx.x * 8 + (threadIdx.x >> 5); i < n; i += gridDim.x * 8) {
    float sc = retention_score_as(p.beta[row0 + i], p.pos[row0 + i], p.q_idx, p.score_dtype);
    if (p.knorm) {
      const float lg = log_row_norm(p.k + (row0 + i) * (int64_t)p.row_vecs * 16, p.row_vecs, p.kv_dtype, lane, p.knorm == 2);
      sc = knorm_score(sc, lg, p.score_dtype, p.kv_dtype);
    }
    if (lane == 0) p.scores[row0 + i] = sc;
  }
}
}  // namespace tkv

extern "C" int tkv_flat_scores(const void* k_cache, const float* beta_cache, const int32_t* pos_cache,
                               const int32_t* seg_len, int nseg, int64_t cap, int head_dim, int kv_dtype,
                               int64_t q_idx, int strategy, int max_len, float* scores_out, tkv_stream_t stream) {
  using namespace tkv;
  const int es = elem_size(kv_dtype);
  const int score_dtype = (strategy >> 8) & 3;
  strategy &= 0xff;
  if (!k_cache || !beta_cache || !pos_cache || !seg_len || !scores_out) return fail(TKV_ERR_ARG, "tkv_flat_scores: NULL pointer argument");
  if (es == 0 || strategy < 0 || strategy > 2 || score_dtype > 2 || nseg < 0 || cap <= 0 || head_dim <= 0 || max_len <= 0)
    return fail(TKV_ERR_ARG, "tkv_flat_scores: bad arguments");
  if (((int64_t)head_dim * es) % 16 != 0 || !aligned16(k_cache)) return fail(TKV_ERR_ARG, "tkv_flat_scores: K rows must be 16-byte multiples, 16-byte aligned");
  if (nseg == 0) return TKV_OK;
  if (nseg > 65535) return fail(TKV_ERR_UNSUPPORTED, "tkv_flat_scores: more than 65535 segments per call");
  ScoreParams p;
  p.k = (const char*)k_cache; p.beta = beta_cache; p.pos = pos_cache; p.seg_len = seg_len; p.cap = cap;
  p.row_vecs = (int)((int64_t)head_dim * es / 16); p.kv_dtype = kv_dtype; p.knorm = strategy; p.score_dtype = score_dtype;
  p.q_idx = q_idx; p.scores = scores_out;
  const int per_seg = (int)std::min<int64_t>(64, (max_len + 63) / 64);   // CTAs per segment, 8 rows at a time each
  flat_scores_kernel<<<dim3((unsigned)per_seg, (unsigned)nseg), 256, 0, (cudaStream_t)stream>>>(p);
  return check_launch("tkv_flat_scores");
}
