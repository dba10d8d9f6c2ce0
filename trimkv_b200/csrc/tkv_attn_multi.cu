// Several query tokens per request on the tensor cores, 32 query rows per CTA.
//
// Same arithmetic as the multi-token form of decode_attn_tc_kernel (tkv_attn_tc.cu), which keeps 16 query rows per CTA
// and therefore reads a K/V chunk once per 16 rows.  For the pieces of a chunked prefill (tens of tokens times G
// query heads per KV head; the reference hands them to flash_attn_varlen_func with causal=True,
// src/trimkv/attn/flash_attn.py:118-145) this kernel puts 32 rows (token, head) on the MMA's N dimension, so a chunk
// of 256 cached tokens is read once per 32 rows:
//   S[128 tokens x 32] = K_tile . Q^T        8 x tcgen05.mma (M=128, N=32, K=16) per tile, D in TMEM columns [0,64)
//   softmax per column over the chunk        one thread per token row; column maxima / sums by warp shuffles
//   O^T[128 dims x 32] += V_tile^T . P       TMEM columns [64,96)
// P (the B operand of the second product) is written over the second K tile, which the tensor core has consumed by
// then, so that two CTAs fit on an SM (107 KB of shared memory each) and overlap each other's phases.
// Row R of a segment = token R / G of the new ones, head R % G; it sees the first len - q_tokens + R / G + 1 cached
// tokens (bottom-right aligned causal mask).  Partials go to the same [segment, chunk, row] workspace that
// decode_attn_combine_kernel merges.  Every wait is bounded.
#include <cuda.h>
#include "tkv_common.cuh"
#include "tkv_attn.cuh"
#include "tkv_tc.cuh"

namespace tkv {

constexpr int kMtThreads = 128;
constexpr int kMtTile = 128;                  // tokens per tile
constexpr int kMtChunk = 256;                 // tokens per CTA (must equal the decode kernel's chunk: shared workspace)
constexpr int kMtRows = 32;                   // query rows per CTA
constexpr int kMtStageBytes = 32768;
constexpr int kMtHalfBytes = 16384;
constexpr int kMtQBytes = kMtRows * 256;      // rows x 128 dims
constexpr int kMtPBytes = kMtRows * 256;      // rows x 128 tokens, per tile
constexpr int kMtTmemCols = 128;              // S tile 0: [0,32)  S tile 1: [32,64)  O: [64,96)
static_assert(2 * kMtPBytes <= kMtStageBytes, "both P tiles live in the second K tile's buffer");

struct MtSmem {
  uint64_t bar_k[2], bar_v[2], bar_s, bar_o;
  uint32_t tmem_base;
  int abort_flag;
  int vis[kMtRows];                           // cached tokens each row may see (0: row does not exist)
  float red_max[4][kMtRows];
  float red_sum[4][kMtRows];
};
constexpr int kMtSmemBytes = 3 * kMtStageBytes + kMtQBytes + (int)sizeof(MtSmem) + 1024;

// Column-wise reduction over the 32 lanes of a warp of 32 values per lane: returns, on lane l, the reduction of
// column l.  Each step halves the columns a lane still carries (it keeps the half selected by one bit of its lane
// index and hands the other half to its partner), so 16+8+4+2+1 = 31 shuffles do the work of 32 x 5.
template <typename Op>
__device__ __forceinline__ float warp_reduce_columns(float (&v)[32], int lane, Op op) {
#pragma unroll
  for (int w = 16; w >= 1; w >>= 1) {
    const bool upper = (lane & w) != 0;
#pragma unroll
    for (int j = 0; j < w; ++j) {
      const float send = upper ? v[j] : v[j + w];
      const float keep = upper ? v[j + w] : v[j];
      v[j] = op(keep, __shfl_xor_sync(0xffffffffu, send, w));
    }
  }
  return v[0];
}

template <int kDtype>
__global__ void __launch_bounds__(kMtThreads)
multi_attn_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  grid_dependency_wait();
  grid_launch_dependents();
  const int seg = blockIdx.x / p.nchunks, chunk = blockIdx.x - seg * p.nchunks;
  const int len = min(p.seg_len[seg], p.max_len);
  const int t0 = chunk * kMtChunk;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = seg / p.hkv, h = seg - b * p.hkv;
  const int G = p.hq / p.hkv;
  const int row_base = blockIdx.y * kMtRows;
  if (t0 >= len) {
    if (chunk == 0) {  // empty segment: zeros for its rows
      for (int c = 0; c < kMtRows; ++c) {
        const int R = row_base + c;
        if (R >= p.rows) break;
        char* op = p.out + (((int64_t)b * p.q_tokens + R / G) * p.hq + h * G + R % G) * 256;
        if (kDtype == TKV_BF16) reinterpret_cast<__nv_bfloat16*>(op)[tid] = __float2bfloat16_rn(0.f);
        else reinterpret_cast<__half*>(op)[tid] = __float2half_rn(0.f);
      }
    }
    return;
  }
  if (chunk == 0 && blockIdx.y == 0 && tid == 0 && p.seg_len[seg] > p.max_len) report(p.status, TKV_DEV_LEN_BOUND);
  const int n_valid = min(kMtChunk, len - t0);
  const int ntiles = (n_valid + kMtTile - 1) / kMtTile;

  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* stage = base;
  uint8_t* q_s = base + 3 * kMtStageBytes;
  uint8_t* p_s = stage + kMtStageBytes;        // over K tile 1, written only after the S MMAs have completed
  MtSmem* sm = reinterpret_cast<MtSmem*>(q_s + kMtQBytes);
  const int64_t row0 = (int64_t)seg * p.cap + t0;

  if (tid == 0) {
    mbar_init(&sm->bar_k[0], 1); mbar_init(&sm->bar_k[1], 1);
    mbar_init(&sm->bar_v[0], 1); mbar_init(&sm->bar_v[1], 1);
    mbar_init(&sm->bar_s, 1); mbar_init(&sm->bar_o, 1);
    sm->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    for (int i = 0; i < ntiles; ++i) {
      mbar_expect_tx(&sm->bar_k[i], kMtStageBytes);
      tma_load_2d(stage + i * kMtStageBytes, &map_k, &sm->bar_k[i], 0, (int)(row0 + i * kMtTile));
      tma_load_2d(stage + i * kMtStageBytes + kMtHalfBytes, &map_k, &sm->bar_k[i], 64, (int)(row0 + i * kMtTile));
    }
    mbar_expect_tx(&sm->bar_v[0], kMtStageBytes);
    tma_load_2d(stage + 2 * kMtStageBytes, &map_v, &sm->bar_v[0], 0, (int)row0);
    tma_load_2d(stage + 2 * kMtStageBytes + kMtHalfBytes, &map_v, &sm->bar_v[0], 64, (int)row0);
  }
  __syncwarp();
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm->tmem_base)), "r"(kMtTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  if (tid < kMtRows) {
    const int R = row_base + tid;
    sm->vis[tid] = R < p.rows ? max(len - p.q_tokens + R / G + 1, 0) : 0;
  }
  // Q rows as the B operand: K-major without swizzle, 8x8 core matrices of 128 B, K-adjacent cores 128 B apart,
  // groups of 8 rows 2048 B apart.
  for (int i = tid; i < kMtRows * 16; i += kMtThreads) {
    const int rr = i >> 4, c = i & 15;
    const int R = row_base + rr;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (R < p.rows)
      v = ld16(p.q + ((int64_t)b * p.q_sb + (int64_t)(R / G) * p.q_st + (int64_t)(h * G + R % G) * p.q_sh) * 2 + c * 16);
    st16(q_s + (rr >> 3) * 2048 + c * 128 + (rr & 7) * 16, v);
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm->tmem_base;
  const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
  const uint32_t idesc_qk = make_idesc(kDtype == TKV_BF16 ? 1 : 0, 0, kMtRows);
  const uint32_t idesc_pv = make_idesc(kDtype == TKV_BF16 ? 1 : 0, 1, kMtRows);
  volatile int* abort_flag = &sm->abort_flag;
  bool v1_issued = false;

  // ---- thread 0: S = K . Q^T for both tiles
  if (tid == 0) {
    bool ok = true;
    for (int i = 0; i < ntiles && ok; ++i) {
      ok = mbar_wait(&sm->bar_k[i], 0);
      if (!ok) break;
      tc_fence_after();
      const uint32_t a0 = smem_u32(stage + i * kMtStageBytes);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const uint64_t ad = make_desc(a0 + (k >> 2) * kMtHalfBytes + (k & 3) * 32, 16, 1024, 2);
        const uint64_t bd = make_desc(smem_u32(q_s) + k * 256, 128, 2048, 0);
        umma(tmem + kMtRows * i, ad, bd, idesc_qk, k > 0);
      }
    }
    if (ok) umma_commit(&sm->bar_s);
    else { *abort_flag = 1; report(p.status, TKV_DEV_TIMEOUT); }
  }
  __syncwarp();
  if (!mbar_wait_or_abort(&sm->bar_s, 0, abort_flag)) {
    if (*abort_flag == 0) { *abort_flag = 1; report(p.status, TKV_DEV_TIMEOUT); }
  }
  tc_fence_after();
  if (tid == 0 && ntiles == 2 && *abort_flag == 0) {
    mbar_expect_tx(&sm->bar_v[1], kMtStageBytes);     // K tile 0 has been consumed: its buffer takes V tile 1
    tma_load_2d(stage, &map_v, &sm->bar_v[1], 0, (int)(row0 + kMtTile));
    tma_load_2d(stage + kMtHalfBytes, &map_v, &sm->bar_v[1], 64, (int)(row0 + kMtTile));
    v1_issued = true;
  }
  __syncthreads();
  const bool aborted = *abort_flag != 0;

  // ---- softmax over the chunk, this thread = token `tid` of each tile.  Shared memory allows two CTAs per SM, so a
  // thread may use up to 256 registers: the masked scores of both tiles stay in registers between the maximum and
  // the exponentials (one TMEM read each).
  float s[2][kMtRows];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int tok = t0 + i * kMtTile + tid;
#pragma unroll
    for (int cg = 0; cg < kMtRows / 16; ++cg) {
      float v[16];
      if (!aborted && i < ntiles) tmem_ld16(tmem + lane_base + kMtRows * i + 16 * cg, v);
#pragma unroll
      for (int g = 0; g < 16; ++g) {
        const int c = cg * 16 + g;
        s[i][c] = (!aborted && i < ntiles && tok < sm->vis[c]) ? v[g] * p.scale_log2 : -INFINITY;
      }
    }
  }
  static_assert(kMtRows == 32, "warp_reduce_columns leaves column l on lane l");
  {
    float m[kMtRows];
#pragma unroll
    for (int c = 0; c < kMtRows; ++c) m[c] = fmaxf(s[0][c], s[1][c]);
    sm->red_max[warp][lane] = warp_reduce_columns(m, lane, [](float a, float b) { return fmaxf(a, b); });
  }
  __syncthreads();
  // P = exp2(s - max) rounded to the K/V dtype into shared memory (B operand of the second product); the column sums
  // use the rounded weights so that numerator and denominator see the same values.
  {
    float l[kMtRows];
#pragma unroll
    for (int c = 0; c < kMtRows; ++c) {
      const float mx = fmaxf(fmaxf(sm->red_max[0][c], sm->red_max[1][c]), fmaxf(sm->red_max[2][c], sm->red_max[3][c]));
      l[c] = 0.f;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const float pw = s[i][c] == -INFINITY ? 0.f : exp2_weight(s[i][c] - mx);
        unsigned short bits;
        float back;
        if (kDtype == TKV_BF16) { __nv_bfloat16 x = __float2bfloat16_rn(pw); bits = __bfloat16_as_ushort(x); back = __bfloat162float(x); }
        else { __half x = __float2half_rn(pw); bits = __half_as_ushort(x); back = __half2float(x); }
        l[c] += back;
        if (i < ntiles)
          *reinterpret_cast<unsigned short*>(p_s + i * kMtPBytes + (tid >> 3) * 128 + (tid & 7) * 2 + (c >> 3) * 2048 + (c & 7) * 16) = bits;
      }
    }
    sm->red_sum[warp][lane] = warp_reduce_columns(l, lane, [](float a, float b) { return a + b; });
  }
  // Rows of a V tile beyond the segment's length may hold anything: their weight is zero, but 0 x NaN would poison
  // the product, so they are cleared in shared memory.
  if (!aborted && (n_valid & (kMtTile - 1)) != 0) {
    const int i = ntiles - 1;
    if (!mbar_wait_or_abort(&sm->bar_v[i], 0, abort_flag)) {
      if (*abort_flag == 0) { *abort_flag = 1; report(p.status, TKV_DEV_TIMEOUT); }
    } else if (i * kMtTile + tid >= n_valid) {
      uint8_t* vt = stage + (i == 0 ? 2 : 0) * kMtStageBytes + tid * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c) { st16(vt + c * 16, make_uint4(0, 0, 0, 0)); st16(vt + kMtHalfBytes + c * 16, make_uint4(0, 0, 0, 0)); }
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
      const uint32_t a0 = smem_u32(stage + (i == 0 ? 2 : 0) * kMtStageBytes);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const uint64_t ad = make_desc(a0 + k * 2048, kMtHalfBytes, 1024, 2);
        const uint64_t bd = make_desc(smem_u32(p_s + i * kMtPBytes) + k * 256, 128, 2048, 0);
        umma(tmem + 2 * kMtRows, ad, bd, idesc_pv, (i > 0 || k > 0));
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
    const int64_t item = (int64_t)seg * p.nchunks + chunk;
    for (int cg = 0; cg < kMtRows / 16; ++cg) {
      float o[16];
      tmem_ld16(tmem + lane_base + 2 * kMtRows + 16 * cg, o);   // this thread owns output dimension `tid`
#pragma unroll
      for (int g = 0; g < 16; ++g) {
        const int c = cg * 16 + g, R = row_base + c;
        if (R >= p.rows) break;
        const float ls = sm->red_sum[0][c] + sm->red_sum[1][c] + sm->red_sum[2][c] + sm->red_sum[3][c];
        if (p.nchunks == 1) {
          const float r = ls > 0.f ? o[g] / ls : 0.f;
          char* op = p.out + (((int64_t)b * p.q_tokens + R / G) * p.hq + h * G + R % G) * 256;
          if (kDtype == TKV_BF16) reinterpret_cast<__nv_bfloat16*>(op)[tid] = __float2bfloat16_rn(r);
          else reinterpret_cast<__half*>(op)[tid] = __float2half_rn(r);
        } else {
          p.part_o[(item * p.rows + R) * 128 + tid] = o[g];
          if (tid == 0) {
            const float mxc = fmaxf(fmaxf(sm->red_max[0][c], sm->red_max[1][c]), fmaxf(sm->red_max[2][c], sm->red_max[3][c]));
            p.part_ml[(item * p.rows + R) * 2] = mxc; p.part_ml[(item * p.rows + R) * 2 + 1] = ls;
          }
        }
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
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kMtTmemCols));
  }
}

template <int kDtype>
static int launch_multi(const CUtensorMap& mk, const CUtensorMap& mv, const AttnParams& p, int nseg, cudaStream_t st) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(multi_attn_tc_kernel<kDtype>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMtSmemBytes);
    if (e != cudaSuccess) return fail(TKV_ERR_LAUNCH, "tkv_decode_attn_multi: %s", cudaGetErrorString(e));
    configured = true;
  }
  const unsigned groups = (unsigned)((p.rows + kMtRows - 1) / kMtRows);
  cudaError_t e = launch_pdl(multi_attn_tc_kernel<kDtype>, dim3((unsigned)((int64_t)nseg * p.nchunks), groups), dim3(kMtThreads),
                             (size_t)kMtSmemBytes, st, mk, mv, p);
  if (e != cudaSuccess) return fail(TKV_ERR_LAUNCH, "tkv_decode_attn_multi: %s", cudaGetErrorString(e));
  return check_launch("tkv_decode_attn_multi");
}

// kMtRows query rows per CTA; `rows` = rows addressable behind k/v (bounds of the tensor maps).
int launch_multi_attn_tc(const AttnParams& p, int nseg, int kv_dtype, int64_t rows, cudaStream_t st) {
  static_assert(kMtChunk == 256, "the partial workspace is laid out for 256-token chunks");
  CUtensorMap mk, mv;
  int rc = make_map_2d(&mk, p.k, 128, rows, 64, 128, kv_dtype);
  if (rc != TKV_OK) return rc;
  rc = make_map_2d(&mv, p.v, 128, rows, 64, 128, kv_dtype);
  if (rc != TKV_OK) return rc;
  return kv_dtype == TKV_BF16 ? launch_multi<TKV_BF16>(mk, mv, p, nseg, st) : launch_multi<TKV_F16>(mk, mv, p, nseg, st);
}

}  // namespace tkv
