// Split-KV decode attention on the 5th-generation tensor cores (tcgen05 + TMEM), K/V tiles staged by TMA.
//
// Same contract as the CUDA-core kernel in tkv_attn.cu (it replaces flash_attn_varlen_func as called by
// src/trimkv/attn/flash_attn.py:135-145 for one query token per request).  One CTA = (segment, chunk of
// 256 cached tokens) = two tiles of 128 tokens:
//   S[128 tokens x 16] = K_tile[128 x 128] . Q^T     tcgen05.mma, A = K tile (smem, K-major, 128B swizzle, as
//                                                    written by TMA), B = Q of the G <= 16 query heads of this
//                                                    KV head (smem, K-major, no swizzle), D in TMEM
//   softmax over the chunk                           one thread per token row (tcgen05.ld 32x32b), fp32, log2 domain
//   O^T[128 dims x 16] += V_tile^T[128 x 128] . P    A = V tile (smem, MN-major, 128B swizzle: the same bytes TMA
//                                                    wrote), B = P (smem, K-major, no swizzle, bf16/f16)
// and the unnormalised O with (max, sum) goes to the workspace that decode_attn_combine_kernel merges.
// Three 32 KB stage buffers hold K0, K1, V0; V1 reuses K0's buffer once the S MMAs have completed, so two CTAs fit
// on an SM and keep ~190 KB of loads in flight.  Every mbarrier wait is bounded: on expiry the CTA records
// TKV_DEV_TIMEOUT, skips the remaining work, frees its TMEM and returns.
#include <cuda.h>
#include "tkv_common.cuh"
#include "tkv_attn.cuh"
#include "tkv_tc.cuh"

namespace tkv {

constexpr int kTcThreads = 128;
constexpr int kTileTokens = 128;
constexpr int kTcChunk = 256;
constexpr int kStageBytes = 32768;            // 128 rows x 256 B (two 64-element halves of 16 KB)
constexpr int kHalfBytes = 16384;
constexpr int kQBytes = 4096;                 // 16 heads x 128 dims
constexpr int kPBytes = 4096;                 // 16 heads x 128 tokens
constexpr int kTmemCols = 64;                 // S tile 0: [0,16)  S tile 1: [16,32)  O: [32,48)

struct TcSmem {                               // after the 1024-byte aligned stage buffers
  uint64_t bar_k[2], bar_v[2], bar_s, bar_o;
  uint32_t tmem_base;
  int abort_flag;
  float red_max[4][16];
  float red_sum[4][16];
};
constexpr int kTcSmemBytes = 3 * kStageBytes + kQBytes + 2 * kPBytes + (int)sizeof(TcSmem) + 1024;

// kG = query rows this CTA handles (<= 16).  kMulti = false: one query token, the rows are the G query heads of the
// KV head.  kMulti = true: several query tokens; blockIdx.y selects a group of 16 of the segment's q_tokens * G
// rows, row R = token * G + head, each with its own causal limit.
template <int kDtype, int kG, bool kMulti>
__global__ void __launch_bounds__(kTcThreads)
decode_attn_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  grid_dependency_wait();  // the lengths and the newest rows come from the preceding kernel of the stream
  grid_launch_dependents();  // the merge kernel may be scheduled; it waits for this grid before reading partials
  int seg, chunk, len;
  if (p.work != nullptr) {
    if ((int)blockIdx.x >= *p.work_count) return;
    const int2 item = p.work[blockIdx.x];
    seg = item.x >> 8; chunk = item.x & 255; len = item.y;
  } else {
    seg = blockIdx.x / p.nchunks; chunk = blockIdx.x - seg * p.nchunks;
    len = min(p.seg_len[seg], p.max_len);
  }
  const int t0 = chunk * kTcChunk;
  if (t0 >= len) {
    if (chunk == 0) {  // empty segment: its query heads get zeros
      const int b0 = seg / p.hkv, h0 = seg - b0 * p.hkv;
      for (int g = 0; g < kG; ++g) {
        char* op;
        if (kMulti) {
          const int R = blockIdx.y * 16 + g, Gq = p.hq / p.hkv;
          if (R >= p.rows) break;
          op = p.out + (((int64_t)b0 * p.q_tokens + R / Gq) * p.hq + h0 * Gq + R % Gq) * 256;
        } else {
          op = p.out + ((int64_t)b0 * p.hq + h0 * kG + g) * 256;
        }
        if (kDtype == TKV_BF16) reinterpret_cast<__nv_bfloat16*>(op)[threadIdx.x] = __float2bfloat16_rn(0.f);
        else reinterpret_cast<__half*>(op)[threadIdx.x] = __float2half_rn(0.f);
      }
    }
    return;
  }
  if (chunk == 0 && threadIdx.x == 0 && p.seg_len[seg] > p.max_len) report(p.status, TKV_DEV_LEN_BOUND);
  const int n_valid = min(kTcChunk, len - t0);
  const int ntiles = (n_valid + kTileTokens - 1) / kTileTokens;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = seg / p.hkv, h = seg - b * p.hkv;

  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* stage = base;                                   // 3 x 32 KB, each 1024-byte aligned
  uint8_t* q_s = base + 3 * kStageBytes;
  uint8_t* p_s = q_s + kQBytes;                            // 2 x 4 KB
  TcSmem* sm = reinterpret_cast<TcSmem*>(p_s + 2 * kPBytes);

  const int64_t row0 = (p.seg_start != nullptr ? (int64_t)p.seg_start[seg] : (int64_t)seg * p.cap) + t0;
  // Thread 0 arms the barriers and starts every copy this CTA can hold before anything else, so the rest of
  // the prologue (TMEM allocation, Q staging) runs under the latency of the loads.
  if (tid == 0) {
    mbar_init(&sm->bar_k[0], 1); mbar_init(&sm->bar_k[1], 1);
    mbar_init(&sm->bar_v[0], 1); mbar_init(&sm->bar_v[1], 1);
    mbar_init(&sm->bar_s, 1); mbar_init(&sm->bar_o, 1);
    sm->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    for (int i = 0; i < ntiles; ++i) {
      mbar_expect_tx(&sm->bar_k[i], kStageBytes);
      tma_load_2d(stage + i * kStageBytes, &map_k, &sm->bar_k[i], 0, (int)(row0 + i * kTileTokens));
      tma_load_2d(stage + i * kStageBytes + kHalfBytes, &map_k, &sm->bar_k[i], 64, (int)(row0 + i * kTileTokens));
    }
    mbar_expect_tx(&sm->bar_v[0], kStageBytes);
    tma_load_2d(stage + 2 * kStageBytes, &map_v, &sm->bar_v[0], 0, (int)row0);
    tma_load_2d(stage + 2 * kStageBytes + kHalfBytes, &map_v, &sm->bar_v[0], 64, (int)row0);
  }
  __syncwarp();
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm->tmem_base)), "r"(kTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  // Q of this KV head's query heads as the B operand: rows = heads (16, zero beyond kG), K-major without
  // swizzle: 8x8 core matrices of 128 B, K-adjacent cores 128 B apart, the second group of 8 heads 2048 B further.
  for (int i = tid; i < 256; i += kTcThreads) {
    const int hh = i >> 4, c = i & 15;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (kMulti) {
      const int R = blockIdx.y * 16 + hh, Gq = p.hq / p.hkv;
      if (hh < kG && R < p.rows)
        v = ld16(p.q + ((int64_t)b * p.q_sb + (int64_t)(R / Gq) * p.q_st + (int64_t)(h * Gq + R % Gq) * p.q_sh) * 2 + c * 16);
    } else if (hh < kG) v = ld16(p.q + ((int64_t)b * p.q_sb + (int64_t)(h * kG + hh) * p.q_sh) * 2 + c * 16);
    st16(q_s + (hh >> 3) * 2048 + c * 128 + (hh & 7) * 16, v);
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm->tmem_base;
  const uint32_t idesc_qk = make_idesc(kDtype == TKV_BF16 ? 1 : 0, 0);
  const uint32_t idesc_pv = make_idesc(kDtype == TKV_BF16 ? 1 : 0, 1);
  volatile int* abort_flag = &sm->abort_flag;
  bool v1_issued = false;

  // ---- thread 0: S = K . Q^T for both tiles
  if (tid == 0) {
    bool ok = true;
    for (int i = 0; i < ntiles && ok; ++i) {
      ok = mbar_wait(&sm->bar_k[i], 0);
      if (!ok) break;
      tc_fence_after();
      const uint32_t a0 = smem_u32(stage + i * kStageBytes);
#pragma unroll
      for (int k = 0; k < 8; ++k) {  // 16 dims per MMA; 4 steps inside a 128-byte swizzle atom, then the next half
        const uint64_t ad = make_desc(a0 + (k >> 2) * kHalfBytes + (k & 3) * 32, 16, 1024, 2);
        const uint64_t bd = make_desc(smem_u32(q_s) + k * 256, 128, 2048, 0);
        umma(tmem + 16 * i, ad, bd, idesc_qk, k > 0);
      }
    }
    if (ok) umma_commit(&sm->bar_s);
    else { *abort_flag = 1; report(p.status, TKV_DEV_TIMEOUT); }
  }
  __syncwarp();
  // ---- everyone: wait for S (bounded; leaves early if thread 0 gave up)
  if (!mbar_wait_or_abort(&sm->bar_s, 0, abort_flag)) {
    if (*abort_flag == 0) { *abort_flag = 1; report(p.status, TKV_DEV_TIMEOUT); }
  }
  tc_fence_after();
  if (tid == 0 && ntiles == 2 && *abort_flag == 0) {
    // K tile 0 has been consumed by the tensor core: its buffer takes V tile 1.
    mbar_expect_tx(&sm->bar_v[1], kStageBytes);
    tma_load_2d(stage, &map_v, &sm->bar_v[1], 0, (int)(row0 + kTileTokens));
    tma_load_2d(stage + kHalfBytes, &map_v, &sm->bar_v[1], 64, (int)(row0 + kTileTokens));
    v1_issued = true;
  }
  __syncthreads();
  const bool aborted = *abort_flag != 0;

  float s[2][kG], mloc[kG];
  int vis[kG];   // several query tokens: cached tokens each query row may see (bottom-right aligned causal mask)
#pragma unroll
  for (int g = 0; g < kG; ++g) {
    mloc[g] = -INFINITY;
    vis[g] = 0;
    if (kMulti) {
      const int R = blockIdx.y * 16 + g, Gq = p.hq / p.hkv;
      vis[g] = R < p.rows ? len - p.q_tokens + R / Gq + 1 : 0;
    }
  }
  if (!aborted) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float v[16];
      if (i < ntiles) tmem_ld16(tmem + ((uint32_t)(warp * 32) << 16) + 16 * i, v);
      const bool valid = i < ntiles && (i * kTileTokens + tid) < n_valid;
#pragma unroll
      for (int g = 0; g < kG; ++g) {
        bool seen = valid;
        if (kMulti) seen = valid && (t0 + i * kTileTokens + tid) < vis[g];   // this thread's token = t0 + i*128 + tid
        s[i][g] = seen ? v[g] * p.scale_log2 : -INFINITY;
        mloc[g] = fmaxf(mloc[g], s[i][g]);
      }
    }
  }
#pragma unroll
  for (int g = 0; g < kG; ++g) {
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) mloc[g] = fmaxf(mloc[g], __shfl_xor_sync(0xffffffffu, mloc[g], o));
    if (lane == 0) sm->red_max[warp][g] = mloc[g];
  }
  __syncthreads();
  float mx[kG], lsum[kG];
#pragma unroll
  for (int g = 0; g < kG; ++g) {
    mx[g] = fmaxf(fmaxf(sm->red_max[0][g], sm->red_max[1][g]), fmaxf(sm->red_max[2][g], sm->red_max[3][g]));
    lsum[g] = 0.f;
  }
  // P as the B operand of the second product: rows = heads, K = tokens, K-major without swizzle (same core-matrix
  // arrangement as Q).  The sum uses the rounded values so numerator and denominator see the same weights.
  if (!aborted) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      if (i < ntiles) {
        uint8_t* pt = p_s + i * kPBytes + (tid >> 3) * 128 + (tid & 7) * 2;
#pragma unroll
        for (int g = 0; g < kG; ++g) {
          const float pw = (s[i][g] == -INFINITY) ? 0.f : exp2_weight(s[i][g] - mx[g]);
          unsigned short bits;
          float back;
          if (kDtype == TKV_BF16) { __nv_bfloat16 x = __float2bfloat16_rn(pw); bits = __bfloat16_as_ushort(x); back = __bfloat162float(x); }
          else { __half x = __float2half_rn(pw); bits = __half_as_ushort(x); back = __half2float(x); }
          lsum[g] += back;
          *reinterpret_cast<unsigned short*>(pt + (g >> 3) * 2048 + (g & 7) * 16) = bits;
        }
      }
    }
  }
#pragma unroll
  for (int g = 0; g < kG; ++g) {
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) lsum[g] += __shfl_xor_sync(0xffffffffu, lsum[g], o);
    if (lane == 0) sm->red_sum[warp][g] = lsum[g];
  }
  // Rows of a V tile beyond the segment's length may hold anything (stale rows, another segment): their weight
  // is zero, but 0 x NaN would poison the product, so they are cleared in shared memory.
  if (!aborted && (n_valid & (kTileTokens - 1)) != 0) {
    const int i = ntiles - 1;
    if (!mbar_wait_or_abort(&sm->bar_v[i], 0, abort_flag)) {
      if (*abort_flag == 0) { *abort_flag = 1; report(p.status, TKV_DEV_TIMEOUT); }
    } else if (i * kTileTokens + tid >= n_valid) {
      uint8_t* vt = stage + (i == 0 ? 2 : 0) * kStageBytes + tid * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c) { st16(vt + c * 16, make_uint4(0, 0, 0, 0)); st16(vt + kHalfBytes + c * 16, make_uint4(0, 0, 0, 0)); }
    }
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // ---- thread 0: O^T += V^T . P for both tiles
  if (tid == 0 && *abort_flag == 0) {
    bool ok = true;
    for (int i = 0; i < ntiles && ok; ++i) {
      ok = mbar_wait(&sm->bar_v[i], 0);
      if (!ok) break;
      tc_fence_after();
      const uint32_t a0 = smem_u32(stage + (i == 0 ? 2 : 0) * kStageBytes);
#pragma unroll
      for (int k = 0; k < 8; ++k) {  // 16 tokens per MMA = 2048 bytes further down both 64-dim halves
        const uint64_t ad = make_desc(a0 + k * 2048, kHalfBytes, 1024, 2);
        const uint64_t bd = make_desc(smem_u32(p_s + i * kPBytes) + k * 256, 128, 2048, 0);
        umma(tmem + 32, ad, bd, idesc_pv, (i > 0 || k > 0));
      }
    }
    if (ok) umma_commit(&sm->bar_o);
    else { *abort_flag = 1; report(p.status, TKV_DEV_TIMEOUT); }
  }
  __syncwarp();
  bool have_o = *abort_flag == 0 && mbar_wait_or_abort(&sm->bar_o, 0, abort_flag);
  if (!have_o && *abort_flag == 0) { *abort_flag = 1; report(p.status, TKV_DEV_TIMEOUT); }
  tc_fence_after();
  if (have_o) {
    float o[16];
    tmem_ld16(tmem + ((uint32_t)(warp * 32) << 16) + 32, o);   // this thread owns output dimension `tid`
    const int64_t item = (int64_t)seg * p.nchunks + chunk;
#pragma unroll
    for (int g = 0; g < kG; ++g) {
      const float ls = sm->red_sum[0][g] + sm->red_sum[1][g] + sm->red_sum[2][g] + sm->red_sum[3][g];
      int R = g, rows = kG;
      char* op = p.out + ((int64_t)b * p.hq + h * kG + g) * 256;
      if (kMulti) {
        const int Gq = p.hq / p.hkv;
        R = blockIdx.y * 16 + g; rows = p.rows;
        if (R >= rows) break;
        op = p.out + (((int64_t)b * p.q_tokens + R / Gq) * p.hq + h * Gq + R % Gq) * 256;
      }
      if (p.nchunks == 1) {
        const float r = ls > 0.f ? o[g] / ls : 0.f;
        if (kDtype == TKV_BF16) reinterpret_cast<__nv_bfloat16*>(op)[tid] = __float2bfloat16_rn(r);
        else reinterpret_cast<__half*>(op)[tid] = __float2half_rn(r);
      } else {
        p.part_o[(item * rows + R) * 128 + tid] = o[g];
        if (tid == 0) { p.part_ml[(item * rows + R) * 2] = mx[g]; p.part_ml[(item * rows + R) * 2 + 1] = ls; }
      }
    }
  }
  // An aborting CTA still drains the copies it started before its shared memory is released.
  if (tid == 0 && *abort_flag != 0) {
    for (int i = 0; i < ntiles; ++i) mbar_wait(&sm->bar_k[i], 0);
    mbar_wait(&sm->bar_v[0], 0);
    if (v1_issued) mbar_wait(&sm->bar_v[1], 0);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols));
  }
}

// ------------------------------------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

int make_map_2d(CUtensorMap* map, const void* base, int64_t cols, int64_t rows, int box_cols, int box_rows, int kv_dtype) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return fail(TKV_ERR_LAUNCH, "cuTensorMapEncodeTiled is not available");
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, kv_dtype == TKV_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(TKV_ERR_LAUNCH, "cuTensorMapEncodeTiled failed with %d", (int)r);
  return TKV_OK;
}

int attn_tc_chunk_tokens() { return kTcChunk; }

template <int kDtype, int kG, bool kMulti = false>
static int launch_tc(const CUtensorMap& mk, const CUtensorMap& mv, const AttnParams& p, int nseg, cudaStream_t st) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(decode_attn_tc_kernel<kDtype, kG, kMulti>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kTcSmemBytes);
    if (e != cudaSuccess) return fail(TKV_ERR_LAUNCH, "tkv_decode_attn(tc): %s", cudaGetErrorString(e));
    configured = true;
  }
  const int64_t grid = p.work != nullptr ? (int64_t)p.work_capacity : (int64_t)nseg * p.nchunks;
  const unsigned groups = kMulti ? (unsigned)((p.rows + 15) / 16) : 1u;   // 16 query rows per CTA
  cudaError_t e = launch_pdl(decode_attn_tc_kernel<kDtype, kG, kMulti>, dim3((unsigned)grid, groups), dim3(kTcThreads),
                             (size_t)kTcSmemBytes, st, mk, mv, p);
  if (e != cudaSuccess) return fail(TKV_ERR_LAUNCH, "tkv_decode_attn(tc): %s", cudaGetErrorString(e));
  return check_launch("tkv_decode_attn(tc)");
}

template <int kDtype>
static int launch_tc_g(const CUtensorMap& mk, const CUtensorMap& mv, const AttnParams& p, int nseg, int G, cudaStream_t st) {
  if (p.q_tokens > 1) {   // several query tokens: rows = q_tokens * G, 16 per CTA
    if (p.rows <= 2) return launch_tc<kDtype, 2, true>(mk, mv, p, nseg, st);
    if (p.rows <= 4) return launch_tc<kDtype, 4, true>(mk, mv, p, nseg, st);
    if (p.rows <= 8) return launch_tc<kDtype, 8, true>(mk, mv, p, nseg, st);
    return launch_tc<kDtype, 16, true>(mk, mv, p, nseg, st);
  }
  switch (G) {
    case 1: return launch_tc<kDtype, 1>(mk, mv, p, nseg, st);
    case 2: return launch_tc<kDtype, 2>(mk, mv, p, nseg, st);
    case 3: return launch_tc<kDtype, 3>(mk, mv, p, nseg, st);
    case 4: return launch_tc<kDtype, 4>(mk, mv, p, nseg, st);
    case 5: return launch_tc<kDtype, 5>(mk, mv, p, nseg, st);
    case 6: return launch_tc<kDtype, 6>(mk, mv, p, nseg, st);
    case 7: return launch_tc<kDtype, 7>(mk, mv, p, nseg, st);
    case 8: return launch_tc<kDtype, 8>(mk, mv, p, nseg, st);
    default: return fail(TKV_ERR_UNSUPPORTED, "tkv_decode_attn(tc): %d query heads per KV head", G);
  }
}

// Work list for ragged lengths: one item per present (segment, chunk) pair, segments in order, so that the grid of
// the split kernel can be sized by the total number of cached tokens instead of nseg * (max_len / chunk).  An empty
// segment still gets one item (its CTA writes the zero output).  One CTA: nseg is a few thousand at most.
__global__ void __launch_bounds__(1024) attn_worklist_kernel(AttnParams p, int nseg, int2* work, int32_t* count) {
  __shared__ int warp_sums[1024 / 32 + 1];
  grid_dependency_wait();
  grid_launch_dependents();
  int running = 0;
  for (int base = 0; base < nseg; base += 1024) {
    const int i = base + threadIdx.x;
    const int len = i < nseg ? max(min(p.seg_len[i], p.max_len), 0) : 0;
    const int c = i < nseg ? max(1, (len + kTcChunk - 1) / kTcChunk) : 0;
    int total;
    const int off = running + block_exclusive_scan<1024>(c, warp_sums, &total);
    for (int j = 0; j < c; ++j)
      if (off + j < p.work_capacity) work[off + j] = make_int2((i << 8) | j, len);
    running += total;
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    if (running > p.work_capacity) report(p.status, TKV_DEV_LEN_BOUND);   // more tokens than the caller's bound
    *count = min(running, p.work_capacity);
  }
}

int launch_attn_worklist(const AttnParams& p, int nseg, cudaStream_t st) {
  cudaError_t e = launch_pdl(attn_worklist_kernel, dim3(1), dim3(1024), (size_t)0, st, p, nseg,
                             const_cast<int2*>(p.work), const_cast<int32_t*>(p.work_count));
  if (e != cudaSuccess) return fail(TKV_ERR_LAUNCH, "tkv_decode_attn_ragged(work list): %s", cudaGetErrorString(e));
  return check_launch("tkv_decode_attn_ragged(work list)");
}

// Launches the tensor-core split kernel; `rows` = number of rows addressable behind k/v (bounds of the tensor maps).
int launch_decode_attn_tc(const AttnParams& p, int nseg, int G, int kv_dtype, int64_t rows, cudaStream_t st) {
  CUtensorMap mk, mv;
  int rc = make_map_2d(&mk, p.k, 128, rows, 64, 128, kv_dtype);
  if (rc != TKV_OK) return rc;
  rc = make_map_2d(&mv, p.v, 128, rows, 64, 128, kv_dtype);
  if (rc != TKV_OK) return rc;
  return kv_dtype == TKV_BF16 ? launch_tc_g<TKV_BF16>(mk, mv, p, nseg, G, st) : launch_tc_g<TKV_F16>(mk, mv, p, nseg, G, st);
}

}  // namespace tkv
