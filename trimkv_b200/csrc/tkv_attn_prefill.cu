// Query-resident varlen GQA attention for many query tokens per request (prompt passes, pieces of a chunked
// prefill) on tcgen05 + TMEM, K/V streamed once per query block by TMA with an online softmax.
//
// What flash_attn_varlen_func(causal=True) computes for the reference when Q > 1
// (src/trimkv/attn/flash_attn.py:118-145): segment s = (request, KV head) holds seg_len[s] cached tokens including the
// q_tokens new ones; query row R = token * G + head of the segment sees its first seg_len - q_tokens + token + 1
// tokens (bottom-right aligned causal mask).
//
// One CTA = (segment, block of 128 query rows).  The 128 rows sit on the MMA's M dimension, one TMEM lane and one
// thread per row, so the softmax never crosses threads:
//   S[128 rows x 128 tokens]  = Q[128 x 128 dims] . K_tile^T     A = Q (smem, K-major, 128B swizzle, staged once),
//                                                                B = K tile as TMA wrote it; D in TMEM, two buffers
//   row max / exp2 / sum      thread = row, its 128 scores read from TMEM once and held in registers; P rounded to the
//                             K/V dtype into smem
//   O[128 rows x 128 dims]   += P[128 x 128 tokens] . V_tile      A = P (smem, K-major, 128B swizzle), B = V tile read
//                                                                MN-major from the bytes TMA wrote; D in TMEM
// O is rescaled in TMEM only when a row's maximum grew by more than 2^8 since the reference maximum was fixed (the
// weights stay below 2^8 meanwhile, well inside fp32 / bf16 range), which after the first tiles is rare.  S of tile
// j+1 is issued before the softmax of tile j starts and P.V of tile j runs under the first half of the softmax of
// tile j+1, K tiles are requested two ahead and V tiles one ahead (two 32 KB stages each).  No workspace, no merge
// kernel.  Every mbarrier wait is bounded; on expiry the CTA records TKV_DEV_TIMEOUT, drains its copies, frees its
// TMEM and returns.
#include <cuda.h>
#include "tkv_common.cuh"
#include "tkv_attn.cuh"
#include "tkv_tc.cuh"

namespace tkv {

constexpr int kPfSoftmaxThreads = 256;         // two threads per query row: columns 0..63 and 64..127 of a tile
constexpr int kPfThreads = kPfSoftmaxThreads + 32;   // plus one warp that issues the TMA copies and the MMAs
constexpr int kPfTile = 128;                  // query rows per CTA, cached tokens per tile
constexpr int kPfTileBytes = 32768;           // 128 rows x 256 B, as two 64-element halves of 16 KB
constexpr int kPfHalf = 16384;
constexpr int kPfTmemCols = 512;              // S buffers at columns 0 and 128, O at 256
constexpr float kPfRescaleGap = 8.0f;         // log2 of the largest weight tolerated before O is rescaled

struct PfSmem {
  uint64_t bar_k[2], bar_v[2], bar_s[2], bar_o, bar_p, bar_x;
  uint32_t tmem_base;
  int abort_flag;
  float red[2][2][kPfTile];                   // [tile parity][column half][row]: row maxima, at the end row sums
};
constexpr int kPfSmemBytes = 6 * kPfTileBytes + (int)sizeof(PfSmem) + 1024;

__device__ __forceinline__ uint32_t pf_idesc(int fmt /*0 f16, 1 bf16*/, int b_mn_major) {
  // kind::f16, D = f32, M = 128, N = 128, A K-major, B K-major or MN-major
  return (1u << 4) | ((uint32_t)fmt << 7) | ((uint32_t)fmt << 10) | ((uint32_t)b_mn_major << 16) | ((128u >> 3) << 17) |
         ((128u >> 4) << 24);
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
        "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])),
        "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
        "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
        "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])),
        "r"(__float_as_uint(v[19])), "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])),
        "r"(__float_as_uint(v[23])), "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])),
        "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])),
        "r"(__float_as_uint(v[31]))
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// 32 consecutive TMEM columns of this thread's lane, without waiting: several of these are issued back to back and
// completed by one pf_wait_ld(), so that a thread's share of a row of S costs one TMEM round trip.
__device__ __forceinline__ void pf_ld32_nowait(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void pf_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void pf_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

template <int kDtype>
__device__ __forceinline__ uint32_t pf_pack2(float a, float b) {
  if (kDtype == TKV_BF16) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&v);
  }
  const __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// Byte offset of 16-byte chunk `c` (0..15: 8 elements each) of row `r` in a 128-row K-major tile with 128-byte swizzle,
// stored as two 64-element halves.
__device__ __forceinline__ uint32_t pf_swz(int r, int c) {
  return (uint32_t)((c >> 3) * kPfHalf + r * 128 + (((c & 7) ^ (r & 7)) << 4));
}

// grid.x = nseg * nblocks, segment-major: the query blocks of one segment are neighbours in launch order, so they run
// at the same time and the K/V tiles they all stream are fetched from HBM once and then found in L2 (with the blocks of
// different segments side by side instead, a long causal pass re-read its K/V from HBM once per block and was bound
// by that).  Within a segment the blocks go in descending order: the last block of a causal pass sees the most tokens,
// so the longest CTAs start first.
//
// Roles: warps 0-7 are the softmax warps.  TMEM lane = query row, and a warp may only touch the 32 lanes of its
// quadrant (warp index mod 4), so row r is shared by thread r (columns 0..63 of every tile, dims 0..63 of O) and thread
// 128 + r (the other halves); the two exchange their row maximum through shared memory once per tile.  Warp 8 issues
// every TMA copy and every MMA (one lane), so no softmax warp ever waits for a copy.  All hand-offs are mbarriers with
// bounded waits: bar_s (S of a tile is in TMEM), bar_x (all 256 partial maxima are in shared memory), bar_p (all of P
// is in shared memory and O has been rescaled if it had to be), bar_o (P.V of a tile has completed).
template <int kDtype>
__global__ void __launch_bounds__(kPfThreads, 1)
prefill_attn_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, AttnParams p,
                    int nseg, int nblocks) {
  extern __shared__ uint8_t smem_raw[];
  grid_dependency_wait();
  grid_launch_dependents();
  const int seg = (int)(blockIdx.x / (unsigned)nblocks);
  const int blk = nblocks - 1 - (int)(blockIdx.x % (unsigned)nblocks);
  const int tid = threadIdx.x, warp = tid >> 5;
  const bool is_ctrl = warp == 8;
  const int row = tid & (kPfTile - 1), half = (tid >> 7) & 1;
  const int G = p.hq / p.hkv;
  const int b = seg / p.hkv, h = seg - b * p.hkv;
  int len = p.seg_len != nullptr ? p.seg_len[seg] : p.max_len;
  if (p.seg_len != nullptr && len > p.max_len) {
    if (tid == 0 && blk == 0) report(p.status, TKV_DEV_LEN_BOUND);
    len = p.max_len;
  }
  const int R = blk * kPfTile + row;                       // this thread's query row of the segment
  const bool row_valid = !is_ctrl && R < p.rows;
  const int token = R / G, head = h * G + (R - token * G);
  // cached tokens this row may see, and the most any row of this CTA may see (CTA-uniform)
  const int vis = row_valid ? max(0, min(len, len - p.q_tokens + token + 1)) : 0;
  const int r_last = min(blk * kPfTile + kPfTile - 1, p.rows - 1);
  const int vis_max = max(0, min(len, len - p.q_tokens + r_last / G + 1));
  const int ntiles = (vis_max + kPfTile - 1) / kPfTile;
  char* const out_row = p.out + (((int64_t)b * p.q_tokens + token) * p.hq + head) * 256 + half * 128;
  if (ntiles == 0) {                                       // nothing visible (an empty segment): zeros
    if (row_valid)
      for (int c = 0; c < 8; ++c) st16(out_row + c * 16, make_uint4(0, 0, 0, 0));
    return;
  }

  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* q_s = base;
  uint8_t* p_s = base + kPfTileBytes;
  uint8_t* k_s = base + 2 * kPfTileBytes;                  // two stages
  uint8_t* v_s = base + 4 * kPfTileBytes;                  // two stages
  PfSmem* sm = reinterpret_cast<PfSmem*>(base + 6 * kPfTileBytes);
  volatile int* abort_flag = &sm->abort_flag;
  const int64_t row0 = (int64_t)seg * p.cap;

  int k_issued = 0, v_issued = 0;                          // control lane: tiles whose copies have been started
  auto load_k = [&](int j) {
    const int st = j & 1;
    mbar_expect_tx(&sm->bar_k[st], kPfTileBytes);
    tma_load_2d(k_s + st * kPfTileBytes, &map_k, &sm->bar_k[st], 0, (int)(row0 + j * kPfTile));
    tma_load_2d(k_s + st * kPfTileBytes + kPfHalf, &map_k, &sm->bar_k[st], 64, (int)(row0 + j * kPfTile));
    ++k_issued;
  };
  auto load_v = [&](int j) {
    const int st = j & 1;
    mbar_expect_tx(&sm->bar_v[st], kPfTileBytes);
    tma_load_2d(v_s + st * kPfTileBytes, &map_v, &sm->bar_v[st], 0, (int)(row0 + j * kPfTile));
    tma_load_2d(v_s + st * kPfTileBytes + kPfHalf, &map_v, &sm->bar_v[st], 64, (int)(row0 + j * kPfTile));
    ++v_issued;
  };
  if (tid == kPfSoftmaxThreads) {
    for (int i = 0; i < 2; ++i) { mbar_init(&sm->bar_k[i], 1); mbar_init(&sm->bar_v[i], 1); mbar_init(&sm->bar_s[i], 1); }
    mbar_init(&sm->bar_o, 1);
    mbar_init(&sm->bar_p, kPfSoftmaxThreads);
    mbar_init(&sm->bar_x, kPfSoftmaxThreads);
    sm->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    for (int i = 0; i < 2 && i < ntiles; ++i) load_k(i);
    load_v(0);
  }
  __syncwarp();
  if (is_ctrl) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm->tmem_base)), "r"(kPfTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  } else {
    // Q block as the A operand: row = query row, K-major with 128-byte swizzle (the layout TMA gives the K tiles);
    // each of the row's two threads stages its 64 dims.
    const char* qp = p.q + ((int64_t)b * p.q_sb + (int64_t)token * p.q_st + (int64_t)head * p.q_sh) * 2 + half * 128;
#pragma unroll
    for (int c = 0; c < 8; ++c)
      st16(q_s + pf_swz(row, half * 8 + c), row_valid ? ld16(qp + c * 16) : make_uint4(0, 0, 0, 0));
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm->tmem_base;

  if (is_ctrl) {
    // ------------------------------------------------------------------------------------ TMA + MMA issue (one lane)
    if (tid == kPfSoftmaxThreads) {
      const uint32_t idesc_s = pf_idesc(kDtype == TKV_BF16 ? 1 : 0, 0);
      const uint32_t idesc_pv = pf_idesc(kDtype == TKV_BF16 ? 1 : 0, 1);
      const uint32_t q_addr = smem_u32(q_s), p_addr = smem_u32(p_s);
      auto issue_s = [&](int j) -> bool {       // S of tile j into S buffer j & 1
        if (!mbar_wait_or_abort(&sm->bar_k[j & 1], (j >> 1) & 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(k_s + (j & 1) * kPfTileBytes);
#pragma unroll
        for (int k = 0; k < 8; ++k) {   // 16 dims per MMA: 4 steps inside a 128-byte swizzle atom, then the other half
          const uint32_t off = (k >> 2) * kPfHalf + (k & 3) * 32;
          umma(tmem + 128 * (j & 1), make_desc(q_addr + off, 16, 1024, 2), make_desc(k_addr + off, 16, 1024, 2), idesc_s, k > 0);
        }
        umma_commit(&sm->bar_s[j & 1]);
        return true;
      };
      bool ok = issue_s(0);
      for (int j = 0; j < ntiles && ok; ++j) {
        // S of the next tile: its buffer was read for tile j-1, whose P has been waited for below (bar_p) already
        if (j + 1 < ntiles) ok = issue_s(j + 1);
        // V of the next tile goes where V of tile j-1 was: free once P.V of tile j-1 has completed
        if (ok && j + 1 < ntiles) {
          if (j > 0) ok = mbar_wait_or_abort(&sm->bar_o, (j - 1) & 1, abort_flag);
          if (ok) load_v(j + 1);
        }
        // K two tiles ahead goes where K of this tile is: free once S of this tile has completed
        if (ok && j + 2 < ntiles) {
          ok = mbar_wait_or_abort(&sm->bar_s[j & 1], (j >> 1) & 1, abort_flag);
          if (ok) load_k(j + 2);
        }
        // O += P . V once the softmax warps have written all of P (and rescaled O if they had to)
        if (ok) ok = mbar_wait_or_abort(&sm->bar_p, j & 1, abort_flag);
        if (ok) ok = mbar_wait_or_abort(&sm->bar_v[j & 1], (j >> 1) & 1, abort_flag);
        if (ok) {
          tc_fence_after();
          const uint32_t v_addr = smem_u32(v_s + (j & 1) * kPfTileBytes);
#pragma unroll
          for (int k = 0; k < 8; ++k) {   // 16 tokens per MMA: along K of P inside the swizzle atom, 2048 B down the V tile
            const uint64_t ad = make_desc(p_addr + (k >> 2) * kPfHalf + (k & 3) * 32, 16, 1024, 2);
            const uint64_t bd = make_desc(v_addr + k * 2048, kPfHalf, 1024, 2);
            umma(tmem + 256, ad, bd, idesc_pv, (j > 0 || k > 0));
          }
          umma_commit(&sm->bar_o);
        }
      }
      if (!ok && *abort_flag == 0) { *abort_flag = 1; report(p.status, TKV_DEV_TIMEOUT); }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------------------------------------ softmax warps
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    float m_ref = -INFINITY, l_sum = 0.f;   // reference maximum of the row (log2 domain), weight sum of this thread's columns
    bool alive = true;                      // warp-uniform
    for (int j = 0; j < ntiles && alive; ++j) {
      const int sb = j & 1;
      const int t0 = j * kPfTile;
      bool ok = mbar_wait_or_abort(&sm->bar_s[sb], (j >> 1) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { alive = false; break; }
      tc_fence_after();
      const int limit = vis - t0 - half * 64;   // columns of this thread's half the row may see (<= 0: none, >= 64: all)
      const uint32_t s_addr = lane_base + 128 * sb + 64 * half;
      uint32_t sv[64];                           // the scores stay in registers from here to the exponentials
      pf_ld32_nowait(s_addr, sv);
      pf_ld32_nowait(s_addr + 32, sv + 32);
      pf_wait_ld();
      float m_part = -INFINITY;
      if (limit >= 64) {                         // every column visible (all tiles but those on the causal diagonal)
        float mr[4] = {__uint_as_float(sv[0]), __uint_as_float(sv[1]), __uint_as_float(sv[2]), __uint_as_float(sv[3])};
#pragma unroll
        for (int i = 4; i < 64; i += 4) {
          mr[0] = fmaxf(mr[0], __uint_as_float(sv[i])); mr[1] = fmaxf(mr[1], __uint_as_float(sv[i + 1]));
          mr[2] = fmaxf(mr[2], __uint_as_float(sv[i + 2])); mr[3] = fmaxf(mr[3], __uint_as_float(sv[i + 3]));
        }
        m_part = fmaxf(fmaxf(mr[0], mr[1]), fmaxf(mr[2], mr[3])) * p.scale_log2;   // the scale is positive (checked on the host)
      } else {
#pragma unroll
        for (int i = 0; i < 64; ++i)
          if (i < limit) m_part = fmaxf(m_part, __uint_as_float(sv[i]) * p.scale_log2);
      }
      // the row's other half
      sm->red[sb][half][row] = m_part;
      pf_arrive(&sm->bar_x);
      ok = mbar_wait_or_abort(&sm->bar_x, j & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { alive = false; break; }
      const float m_tile = fmaxf(m_part, sm->red[sb][half ^ 1][row]);
      const bool grow = m_tile > m_ref + kPfRescaleGap || (m_ref == -INFINITY && m_tile > -INFINITY);
      const bool rescale = __any_sync(0xffffffffu, grow);   // the row's two warps hold the same values and decide alike
      // ---- P.V of the previous tile must be complete before O or the P buffer are touched
      if (j > 0) {
        ok = mbar_wait_or_abort(&sm->bar_o, (j - 1) & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { alive = false; break; }
        tc_fence_after();
      }
      if (rescale) {
        const float m_new = fmaxf(m_ref, m_tile);
        if (j > 0) {
          const float alpha = (m_ref == -INFINITY) ? 1.0f : exp2_weight(m_ref - m_new);   // O of such a row is still zero
#pragma unroll
          for (int c2 = 0; c2 < 2; ++c2) {       // this thread's 64 dims of the row
            float o[32];
            tmem_ld32(lane_base + 256 + 64 * half + c2 * 32, o);
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] *= alpha;
            tmem_st32(lane_base + 256 + 64 * half + c2 * 32, o);
          }
          l_sum *= alpha;
        }
        m_ref = m_new;
      }
      // ---- P = 2^(s - m_ref) rounded to the K/V dtype for the tensor core; the row sum is taken in fp32
      const float neg_m = -m_ref;
      float ls[4] = {0.f, 0.f, 0.f, 0.f};
      if (limit >= 64) {
#pragma unroll
        for (int c2 = 0; c2 < 2; ++c2) {
          uint32_t w[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float a = exp2_weight(fmaf(__uint_as_float(sv[c2 * 32 + i]), p.scale_log2, neg_m));
            const float bb = exp2_weight(fmaf(__uint_as_float(sv[c2 * 32 + i + 1]), p.scale_log2, neg_m));
            ls[(i >> 1) & 3] += a + bb;
            w[i >> 1] = pf_pack2<kDtype>(a, bb);
          }
#pragma unroll
          for (int c = 0; c < 4; ++c)
            st16(p_s + pf_swz(row, half * 8 + c2 * 4 + c), make_uint4(w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]));
        }
      } else {
#pragma unroll
        for (int c2 = 0; c2 < 2; ++c2) {
          uint32_t w[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const int col = c2 * 32 + i;
            const float a = (col < limit) ? exp2_weight(fmaf(__uint_as_float(sv[col]), p.scale_log2, neg_m)) : 0.f;
            const float bb = (col + 1 < limit) ? exp2_weight(fmaf(__uint_as_float(sv[col + 1]), p.scale_log2, neg_m)) : 0.f;
            ls[(i >> 1) & 3] += a + bb;
            w[i >> 1] = pf_pack2<kDtype>(a, bb);
          }
#pragma unroll
          for (int c = 0; c < 4; ++c)
            st16(p_s + pf_swz(row, half * 8 + c2 * 4 + c), make_uint4(w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]));
        }
      }
      l_sum += (ls[0] + ls[1]) + (ls[2] + ls[3]);
      // Rows of the last V tile beyond the segment's length may hold anything (stale rows, another segment): their
      // weight is zero, but 0 x NaN would poison the product, so they are cleared in shared memory (a thread clears
      // its half of the token row with its own index).
      if (t0 + kPfTile > len) {
        ok = mbar_wait_or_abort(&sm->bar_v[sb], (j >> 1) & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { alive = false; break; }
        if (t0 + row >= len) {
          uint8_t* vt = v_s + sb * kPfTileBytes + half * kPfHalf + row * 128;
#pragma unroll
          for (int c = 0; c < 8; ++c) st16(vt + c * 16, make_uint4(0, 0, 0, 0));
        }
      }
      fence_async_smem();
      tc_fence_before();
      pf_arrive(&sm->bar_p);
    }
    // ---- epilogue: O / sum -> out
    if (alive) {
      bool ok = mbar_wait_or_abort(&sm->bar_o, (ntiles - 1) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      alive = ok;
    }
    if (alive) {
      tc_fence_after();
      sm->red[ntiles & 1][half][row] = l_sum;
      pf_arrive(&sm->bar_x);
      bool ok = mbar_wait_or_abort(&sm->bar_x, ntiles & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      alive = ok;
    }
    if (alive) {
      const float total = l_sum + sm->red[ntiles & 1][half ^ 1][row];
      const float inv = total > 0.f ? 1.0f / total : 0.f;
#pragma unroll
      for (int c2 = 0; c2 < 2; ++c2) {
        float o[32];
        tmem_ld32(lane_base + 256 + 64 * half + c2 * 32, o);
        if (row_valid) {
          uint32_t w[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) w[i >> 1] = pf_pack2<kDtype>(o[i] * inv, o[i + 1] * inv);
#pragma unroll
          for (int c = 0; c < 4; ++c)
            st16(out_row + (c2 * 4 + c) * 16, make_uint4(w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]));
        }
      }
    } else if ((tid & 31) == 0 && *abort_flag == 0) {
      *abort_flag = 1; report(p.status, TKV_DEV_TIMEOUT);
    }
  }
  tc_fence_before();
  __syncthreads();
  // An aborting CTA drains the copies it started before its shared memory is released.
  if (tid == kPfSoftmaxThreads && *abort_flag != 0) {
    for (int i = max(0, k_issued - 2); i < k_issued; ++i) mbar_wait(&sm->bar_k[i & 1], (i >> 1) & 1);
    for (int i = max(0, v_issued - 2); i < v_issued; ++i) mbar_wait(&sm->bar_v[i & 1], (i >> 1) & 1);
  }
  __syncthreads();
  if (is_ctrl) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kPfTmemCols));
}

template <int kDtype>
static int launch_prefill(const CUtensorMap& mk, const CUtensorMap& mv, const AttnParams& p, int nseg, int nblocks,
                          cudaStream_t st) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(prefill_attn_kernel<kDtype>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPfSmemBytes);
    if (e != cudaSuccess) return fail(TKV_ERR_LAUNCH, "tkv_prefill_attn: %s", cudaGetErrorString(e));
    configured = true;
  }
  cudaError_t e = launch_pdl(prefill_attn_kernel<kDtype>, dim3((unsigned)((int64_t)nseg * nblocks)), dim3(kPfThreads),
                             (size_t)kPfSmemBytes, st, mk, mv, p, nseg, nblocks);
  if (e != cudaSuccess) return fail(TKV_ERR_LAUNCH, "tkv_prefill_attn: %s", cudaGetErrorString(e));
  return check_launch("tkv_prefill_attn");
}

}  // namespace tkv

extern "C" int tkv_prefill_attn(const void* q, int64_t q_sb, int64_t q_st, int64_t q_sh,
                                const void* k_cache, const void* v_cache, const int32_t* seg_len, int64_t cap,
                                void* out, int batch, int hq, int hkv, int head_dim, int kv_dtype,
                                float scale, int max_len, int q_tokens, int32_t* status, tkv_stream_t stream) {
  using namespace tkv;
  if (!q || !k_cache || !v_cache || !out) return fail(TKV_ERR_ARG, "tkv_prefill_attn: NULL pointer argument");
  if (!(scale > 0.f)) return fail(TKV_ERR_ARG, "tkv_prefill_attn: scale must be positive");
  if (batch < 0 || hq <= 0 || hkv <= 0 || hq % hkv != 0 || max_len <= 0 || q_tokens < 1 || cap < max_len)
    return fail(TKV_ERR_ARG, "tkv_prefill_attn: bad sizes batch=%d hq=%d hkv=%d max_len=%d q_tokens=%d cap=%lld", batch, hq,
                hkv, max_len, q_tokens, (long long)cap);
  if (head_dim != 128 || (kv_dtype != TKV_BF16 && kv_dtype != TKV_F16))
    return fail(TKV_ERR_UNSUPPORTED, "tkv_prefill_attn: head_dim=%d dtype=%d (supported: 128, bf16/f16)", head_dim, kv_dtype);
  if (!aligned16(q) || !aligned16(k_cache) || !aligned16(v_cache) || !aligned16(out))
    return fail(TKV_ERR_ARG, "tkv_prefill_attn: pointers must be 16-byte aligned");
  if ((q_sb * 2) % 16 || (q_st * 2) % 16 || (q_sh * 2) % 16)
    return fail(TKV_ERR_ARG, "tkv_prefill_attn: q strides must be multiples of 16 bytes");
  if (batch == 0) return TKV_OK;
  const int nseg = batch * hkv, G = hq / hkv;
  const int64_t rows = (int64_t)q_tokens * G;
  const int64_t nblocks = (rows + kPfTile - 1) / kPfTile;
  if ((int64_t)nseg * nblocks > INT32_MAX || (int64_t)nseg * cap < kPfTile || (int64_t)nseg * cap + kPfTile > INT32_MAX)
    return fail(TKV_ERR_UNSUPPORTED, "tkv_prefill_attn: %lld query blocks x %d segments, %lld cache rows", (long long)nblocks,
                nseg, (long long)nseg * cap);
  AttnParams p;
  p.q = (const char*)q; p.q_sb = q_sb; p.q_sh = q_sh; p.q_st = q_st;
  p.k = (const char*)k_cache; p.v = (const char*)v_cache;
  p.seg_len = seg_len; p.seg_start = nullptr; p.cap = cap;
  p.out = (char*)out;
  p.part_ml = nullptr; p.part_o = nullptr; p.chunk = kPfTile; p.nchunks = 0;
  p.hq = hq; p.hkv = hkv; p.max_len = max_len;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  p.work = nullptr; p.work_count = nullptr; p.work_capacity = 0;
  p.q_tokens = q_tokens; p.rows = (int)rows;
  if (rows > INT32_MAX) return fail(TKV_ERR_UNSUPPORTED, "tkv_prefill_attn: too many query rows per segment");
  CUtensorMap mk, mv;
  int rc = make_map_2d(&mk, k_cache, 128, (int64_t)nseg * cap, 64, 128, kv_dtype);
  if (rc != TKV_OK) return rc;
  rc = make_map_2d(&mv, v_cache, 128, (int64_t)nseg * cap, 64, 128, kv_dtype);
  if (rc != TKV_OK) return rc;
  return kv_dtype == TKV_BF16 ? launch_prefill<TKV_BF16>(mk, mv, p, nseg, (int)nblocks, (cudaStream_t)stream)
                              : launch_prefill<TKV_F16>(mk, mv, p, nseg, (int)nblocks, (cudaStream_t)stream);
}
