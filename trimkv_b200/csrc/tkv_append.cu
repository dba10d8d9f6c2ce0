// In-place append of new K/V rows, log beta and positions into the capacity-strided flat cache.
//
// Replaces TrimKVCache.update's torch.cat x4 (src/trimkv/cache_utils.py:104-108) and the four
// update_flatten_view_triton calls of the flat caches (src/trimkv/triton/db_cache_utils.py:86-186),
// which re-copy the whole cache every step.  Here a step moves only the new rows:
// 2*row_bytes + 8 bytes written per (segment, token).
#include "tkv_common.cuh"

namespace tkv {

struct AppendParams {
  char* k_cache; char* v_cache; float* beta_cache; int32_t* pos_cache;
  int32_t* seg_len; int32_t* cu_seqlens;
  const char* k_new; const char* v_new; int64_t k_sb, k_sh, k_ss;   // byte strides
  const void* beta_new; int beta_dtype; int64_t b_sb, b_sh, b_ss;   // element strides
  const int64_t* pos_new; int64_t p_sb, p_sh, p_ss;                 // element strides
  int nseg, hkv, s_new, row_vecs;  // row_vecs = 16-byte vectors per K (or V) row
  int64_t cap;
  int32_t* status;
};

__device__ __forceinline__ float load_beta(const void* p, int dtype, int64_t idx) {
  if (dtype == TKV_F32) return reinterpret_cast<const float*>(p)[idx];
  if (dtype == TKV_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[idx]);
  return __half2float(reinterpret_cast<const __half*>(p)[idx]);
}

// Decode path: one warp per segment copies its s_new (small) rows and bumps seg_len / cu_seqlens.
// The warp reads seg_len before any lane writes it, so the bump needs no second launch.
template <int kWarps>
__global__ void __launch_bounds__(kWarps * 32) append_warp_per_segment(AppendParams p) {
  const int lane = threadIdx.x & 31;
  const int seg = blockIdx.x * kWarps + (threadIdx.x >> 5);
  if (seg >= p.nseg) return;
  const int len = p.seg_len[seg];
  __syncwarp();
  if ((int64_t)len + p.s_new > p.cap || len < 0) {
    if (lane == 0) report(p.status, TKV_DEV_CAPACITY);
    return;
  }
  const int b = seg / p.hkv, h = seg - b * p.hkv;
  const int64_t row_bytes = (int64_t)p.row_vecs * 16;
  const int64_t dst_row0 = (int64_t)seg * p.cap + len;
  const int nvec = 2 * p.row_vecs;  // K vectors then V vectors
  for (int s = 0; s < p.s_new; ++s) {
    const int64_t src_off = b * p.k_sb + h * p.k_sh + s * p.k_ss;
    for (int i = lane; i < nvec; i += 32) {
      const bool is_v = i >= p.row_vecs;
      const int j = is_v ? i - p.row_vecs : i;
      const char* src = (is_v ? p.v_new : p.k_new) + src_off + (int64_t)j * 16;
      char* dst = (is_v ? p.v_cache : p.k_cache) + (dst_row0 + s) * row_bytes + (int64_t)j * 16;
      st16(dst, ld16(src));
    }
  }
  for (int s = lane; s < p.s_new; s += 32) {
    p.beta_cache[dst_row0 + s] = load_beta(p.beta_new, p.beta_dtype, b * p.b_sb + h * p.b_sh + s * p.b_ss);
    p.pos_cache[dst_row0 + s] = (int32_t)p.pos_new[b * p.p_sb + h * p.p_sh + s * p.p_ss];
  }
  if (lane == 0) {
    p.seg_len[seg] = len + p.s_new;
    if (p.cu_seqlens != nullptr) p.cu_seqlens[seg + 1] += (seg + 1) * p.s_new;
  }
}

// Chunk path (many new tokens per segment): grid (row tiles, nseg); seg_len is read-only here
// and bumped by append_bump afterwards.
constexpr int kChunkRows = 16;
__global__ void __launch_bounds__(256) append_rows_tiled(AppendParams p) {
  const int seg = blockIdx.y;
  const int s0 = blockIdx.x * kChunkRows;
  const int len = p.seg_len[seg];
  if ((int64_t)len + p.s_new > p.cap || len < 0) {
    if (threadIdx.x == 0 && blockIdx.x == 0) report(p.status, TKV_DEV_CAPACITY);
    return;
  }
  const int b = seg / p.hkv, h = seg - b * p.hkv;
  const int64_t row_bytes = (int64_t)p.row_vecs * 16;
  const int64_t dst_row0 = (int64_t)seg * p.cap + len;
  const int rows = min(kChunkRows, p.s_new - s0);
  const int nvec = 2 * p.row_vecs;
  for (int i = threadIdx.x; i < rows * nvec; i += blockDim.x) {
    const int r = i / nvec, c = i - r * nvec;
    const bool is_v = c >= p.row_vecs;
    const int j = is_v ? c - p.row_vecs : c;
    const int s = s0 + r;
    const char* src = (is_v ? p.v_new : p.k_new) + b * p.k_sb + h * p.k_sh + s * p.k_ss + (int64_t)j * 16;
    char* dst = (is_v ? p.v_cache : p.k_cache) + (dst_row0 + s) * row_bytes + (int64_t)j * 16;
    st16(dst, ld16_stream(src));
  }
  for (int r = threadIdx.x; r < rows; r += blockDim.x) {
    const int s = s0 + r;
    p.beta_cache[dst_row0 + s] = load_beta(p.beta_new, p.beta_dtype, b * p.b_sb + h * p.b_sh + s * p.b_ss);
    p.pos_cache[dst_row0 + s] = (int32_t)p.pos_new[b * p.p_sb + h * p.p_sh + s * p.p_ss];
  }
}

__global__ void append_bump(int32_t* seg_len, int32_t* cu_seqlens, int nseg, int s_new, int64_t cap) {
  const int seg = blockIdx.x * blockDim.x + threadIdx.x;
  if (seg >= nseg) return;
  const int len = seg_len[seg];
  const bool ok = len >= 0 && (int64_t)len + s_new <= cap;
  if (ok) seg_len[seg] = len + s_new;
  // cu_seqlens stays a prefix sum only if every segment was appended; a skipped segment is an
  // error the caller sees in the status word.
  if (cu_seqlens != nullptr) cu_seqlens[seg + 1] += (seg + 1) * s_new;
}

}  // namespace tkv

extern "C" int tkv_append(void* k_cache, void* v_cache, float* beta_cache, int32_t* pos_cache,
                          int32_t* seg_len, int32_t* cu_seqlens,
                          const void* k_new, const void* v_new, int64_t k_sb, int64_t k_sh, int64_t k_ss,
                          const void* beta_new, int beta_dtype, int64_t b_sb, int64_t b_sh, int64_t b_ss,
                          const int64_t* pos_new, int64_t p_sb, int64_t p_sh, int64_t p_ss,
                          int batch, int hkv, int s_new, int head_dim, int64_t cap, int kv_dtype,
                          int32_t* status, tkv_stream_t stream) {
  using namespace tkv;
  const int es = elem_size(kv_dtype);
  if (es == 0) return fail(TKV_ERR_ARG, "tkv_append: unknown kv_dtype %d", kv_dtype);
  if (elem_size(beta_dtype) == 0) return fail(TKV_ERR_ARG, "tkv_append: unknown beta_dtype %d", beta_dtype);
  if (!k_cache || !v_cache || !beta_cache || !pos_cache || !seg_len || !k_new || !v_new || !beta_new || !pos_new)
    return fail(TKV_ERR_ARG, "tkv_append: NULL pointer argument");
  if (batch < 0 || hkv <= 0 || s_new < 0 || head_dim <= 0 || cap <= 0)
    return fail(TKV_ERR_ARG, "tkv_append: bad sizes batch=%d hkv=%d s_new=%d head_dim=%d cap=%lld", batch, hkv,
                s_new, head_dim, (long long)cap);
  const int64_t row_bytes = (int64_t)head_dim * es;
  if (row_bytes % 16 != 0) return fail(TKV_ERR_ARG, "tkv_append: row of %lld bytes is not a multiple of 16", (long long)row_bytes);
  if (!aligned16(k_cache) || !aligned16(v_cache) || !aligned16(k_new) || !aligned16(v_new))
    return fail(TKV_ERR_ARG, "tkv_append: K/V pointers must be 16-byte aligned");
  if ((k_sb * es) % 16 || (k_sh * es) % 16 || (k_ss * es) % 16)
    return fail(TKV_ERR_ARG, "tkv_append: K/V strides must be multiples of 16 bytes");
  const int64_t nseg64 = (int64_t)batch * hkv;
  if (nseg64 > INT32_MAX / 2) return fail(TKV_ERR_ARG, "tkv_append: too many segments");
  if (nseg64 == 0 || s_new == 0) return TKV_OK;

  AppendParams p;
  p.k_cache = (char*)k_cache; p.v_cache = (char*)v_cache; p.beta_cache = beta_cache; p.pos_cache = pos_cache;
  p.seg_len = seg_len; p.cu_seqlens = cu_seqlens;
  p.k_new = (const char*)k_new; p.v_new = (const char*)v_new;
  p.k_sb = k_sb * es; p.k_sh = k_sh * es; p.k_ss = k_ss * es;
  p.beta_new = beta_new; p.beta_dtype = beta_dtype; p.b_sb = b_sb; p.b_sh = b_sh; p.b_ss = b_ss;
  p.pos_new = pos_new; p.p_sb = p_sb; p.p_sh = p_sh; p.p_ss = p_ss;
  p.nseg = (int)nseg64; p.hkv = hkv; p.s_new = s_new; p.row_vecs = (int)(row_bytes / 16);
  p.cap = cap; p.status = status;
  cudaStream_t st = (cudaStream_t)stream;
  if (s_new <= 8) {
    constexpr int kWarps = 4;
    append_warp_per_segment<kWarps><<<(p.nseg + kWarps - 1) / kWarps, kWarps * 32, 0, st>>>(p);
    return check_launch("tkv_append");
  }
  if (p.nseg > 65535) return fail(TKV_ERR_UNSUPPORTED, "tkv_append: more than 65535 segments with s_new > 8");
  dim3 grid((s_new + kChunkRows - 1) / kChunkRows, p.nseg);
  append_rows_tiled<<<grid, 256, 0, st>>>(p);
  int rc = check_launch("tkv_append(rows)");
  if (rc != TKV_OK) return rc;
  append_bump<<<(p.nseg + 255) / 256, 256, 0, st>>>(seg_len, cu_seqlens, p.nseg, s_new, cap);
  return check_launch("tkv_append(bump)");
}

// ---------------------------------------------------------------------------------------------------------
// Functional append on the reference's packed layout: out = per-head concatenation of old and new rows.
// Same semantics as update_flatten_view_triton (src/trimkv/triton/db_cache_utils.py:86-186: output segment h
// starts at cu[h] + h*S, old rows first, then the S new rows), in one launch, without the host sync for the
// longest head: work is split over OUTPUT rows, and each row finds its head by binary search in the shifted
// prefix sums, so heads of any length balance.
namespace tkv {

constexpr int kPackedRows = 64;

template <typename V>
__global__ void __launch_bounds__(256) flat_append_packed_kernel(const char* cache, const char* state, const int32_t* cu,
                                                                 char* out, int heads, int s_new, int64_t row_bytes,
                                                                 int64_t out_rows) {
  __shared__ int64_t s_src[kPackedRows];   // source row; >= 0: row of cache, < 0: -(row of state) - 1
  const int64_t r0 = (int64_t)blockIdx.x * kPackedRows;
  const int rows = (int)min((int64_t)kPackedRows, out_rows - r0);
  if (threadIdx.x < rows) {
    const int64_t r = r0 + threadIdx.x;
    // largest h with cu[h] + h*s_new <= r
    int lo = 0, hi = heads - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if ((int64_t)cu[mid] + (int64_t)mid * s_new <= r) lo = mid; else hi = mid - 1;
    }
    const int64_t off = r - ((int64_t)cu[lo] + (int64_t)lo * s_new);
    const int64_t old_len = (int64_t)cu[lo + 1] - cu[lo];
    s_src[threadIdx.x] = off < old_len ? (int64_t)cu[lo] + off : -((int64_t)lo * s_new + (off - old_len)) - 1;
  }
  __syncthreads();
  const int vecs = (int)(row_bytes / sizeof(V));
  for (int i = threadIdx.x; i < rows * vecs; i += blockDim.x) {
    const int r = i / vecs, c = i - r * vecs;
    const int64_t src = s_src[r];
    const char* sp = src >= 0 ? cache + src * row_bytes : state + (-src - 1) * row_bytes;
    *reinterpret_cast<V*>(out + (r0 + r) * row_bytes + (int64_t)c * sizeof(V)) =
        *reinterpret_cast<const V*>(sp + (int64_t)c * sizeof(V));
  }
}

}  // namespace tkv

extern "C" int tkv_flat_append_packed(const void* cache, const void* state, const int32_t* cu_headlens, void* out,
                                      int heads, int s_new, int64_t origin_rows, int64_t row_bytes,
                                      tkv_stream_t stream) {
  using namespace tkv;
  if (!state || !cu_headlens || !out || (origin_rows > 0 && !cache))
    return fail(TKV_ERR_ARG, "tkv_flat_append_packed: NULL pointer argument");
  if (heads <= 0 || s_new < 0 || origin_rows < 0 || row_bytes <= 0)
    return fail(TKV_ERR_ARG, "tkv_flat_append_packed: bad sizes heads=%d s_new=%d rows=%lld row_bytes=%lld", heads, s_new,
                (long long)origin_rows, (long long)row_bytes);
  const int64_t out_rows = origin_rows + (int64_t)heads * s_new;
  if (out_rows == 0) return TKV_OK;
  const unsigned grid = (unsigned)((out_rows + kPackedRows - 1) / kPackedRows);
  const uintptr_t bits = (uintptr_t)cache | (uintptr_t)state | (uintptr_t)out | (uintptr_t)row_bytes;
  cudaStream_t st = (cudaStream_t)stream;
  const char* c = (const char*)cache; const char* s = (const char*)state; char* o = (char*)out;
  if ((bits & 15) == 0) flat_append_packed_kernel<uint4><<<grid, 256, 0, st>>>(c, s, cu_headlens, o, heads, s_new, row_bytes, out_rows);
  else if ((bits & 7) == 0) flat_append_packed_kernel<uint2><<<grid, 256, 0, st>>>(c, s, cu_headlens, o, heads, s_new, row_bytes, out_rows);
  else if ((bits & 3) == 0) flat_append_packed_kernel<uint32_t><<<grid, 256, 0, st>>>(c, s, cu_headlens, o, heads, s_new, row_bytes, out_rows);
  else if ((bits & 1) == 0) flat_append_packed_kernel<uint16_t><<<grid, 256, 0, st>>>(c, s, cu_headlens, o, heads, s_new, row_bytes, out_rows);
  else flat_append_packed_kernel<uint8_t><<<grid, 256, 0, st>>>(c, s, cu_headlens, o, heads, s_new, row_bytes, out_rows);
  return check_launch("tkv_flat_append_packed");
}
