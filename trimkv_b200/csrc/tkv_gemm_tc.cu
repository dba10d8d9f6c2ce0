// Weight-streaming GEMM for the decode step: y[M <= 32, N] = x[M, K] . W[N, K]^T, on tcgen05 with TMA.
//
// In the reference these are nn.Linear calls on a handful of rows (q/k/v/gate, o_proj, gate/up, down of
// src/trimkv/models/qwen3/modeling_trimkv_qwen3.py:328-333,383,436): at one token per request they are pure weight
// streaming (2*N*K bytes for 2*M*N*K flop), and a library GEMM leaves more than half of the HBM bandwidth unused at
// these shapes.  Here the weight rows sit on the MMA's M dimension (128 rows of W per CTA), the few activation rows
// on its N dimension (32 columns), and K is split across CTAs so that every SM streams:
//   CTA (n_tile, split) : for its K range, 64 columns at a time:  TMA W[128 x 64] + x[32 x 64] -> 8-stage ring
//                         -> 4 x tcgen05.mma (M=128, N=32, K=16) accumulating D[128 x 32] fp32 in TMEM
//   epilogue            : D -> partial[split][m][n0 + lane] (fp32, coalesced per activation row).
// The partial sums are added up in a fixed order by whoever consumes the result (tkv_decode_prep,
// tkv_add_rmsnorm, tkv_silu_mul), which also adds the bias and rounds to the model dtype: same value as a GEMM with
// fp32 accumulation followed by one rounding, deterministic, no atomics.
// One thread feeds TMA, one issues MMAs, all four warps run the epilogue; every wait has an iteration limit.
#include "tkv_tc.cuh"

namespace tkv {

constexpr int kGemmThreads = 128;
constexpr int kGemmStages = 5;
constexpr int kGemmBK = 64;                       // K columns per stage (one 128-byte swizzle atom of bf16)
constexpr int kGemmWBytes = 128 * kGemmBK * 2;    // 16 KB
constexpr int kGemmXBytes = 32 * kGemmBK * 2;     // 4 KB
constexpr int kGemmStageBytes = kGemmWBytes + kGemmXBytes;
constexpr int kGemmTmemCols = 32;

struct GemmSmem {
  uint64_t full[kGemmStages], empty[kGemmStages], done;
  uint32_t tmem_base;
  int abort_flag;
};
constexpr int kGemmSmemBytes = kGemmStages * kGemmStageBytes + (int)sizeof(GemmSmem) + 1024;

struct GemmParams {
  float* partial;      // [splits, m, n]
  int m, n, k_steps, splits, is_bf16;
  int32_t* status;
};

__global__ void __launch_bounds__(kGemmThreads)
skinny_gemm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  GemmSmem* sm = reinterpret_cast<GemmSmem*>(base + kGemmStages * kGemmStageBytes);
  const int tid = threadIdx.x, warp = tid >> 5;
  const int n_tile = blockIdx.x / p.splits, split = blockIdx.x - n_tile * p.splits;
  const int ks0 = (int)((int64_t)split * p.k_steps / p.splits), ks1 = (int)((int64_t)(split + 1) * p.k_steps / p.splits);
  const int steps = ks1 - ks0;
  volatile int* abort_flag = &sm->abort_flag;

  if (tid == 0) {
    for (int s = 0; s < kGemmStages; ++s) { mbar_init(&sm->full[s], 1); mbar_init(&sm->empty[s], 1); }
    mbar_init(&sm->done, 1);
    sm->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm->tmem_base)), "r"(kGemmTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm->tmem_base;
  // The weights do not depend on the preceding kernel of the stream, the activations do: the first ring of weight
  // tiles is requested before the dependency wait, so that under programmatic dependent launch the pipeline fills
  // while the predecessor is still running.
  const int pre = min(steps, kGemmStages);
  if (tid == 0) {
    for (int i = 0; i < pre; ++i) {
      mbar_expect_tx(&sm->full[i], kGemmStageBytes);
      tma_load_2d(base + i * kGemmStageBytes, &map_w, &sm->full[i], (ks0 + i) * kGemmBK, n_tile * 128);
    }
  }
  grid_dependency_wait();  // x is produced by the preceding kernel of the stream
  grid_launch_dependents();  // the consumer of the partial sums may be scheduled; it waits for this grid before reading

  if (tid == 0) {
    // ---- producer: keeps up to kGemmStages tiles of W and x in flight
    for (int i = 0; i < pre; ++i)
      tma_load_2d(base + i * kGemmStageBytes + kGemmWBytes, &map_x, &sm->full[i], (ks0 + i) * kGemmBK, 0);
    for (int i = pre; i < steps; ++i) {
      const int s = i % kGemmStages;
      if (!mbar_wait_or_abort(&sm->empty[s], ((i / kGemmStages) - 1) & 1, abort_flag)) {
        if (*abort_flag == 0) { *abort_flag = 1; report(p.status, TKV_DEV_TIMEOUT); }
        break;
      }
      uint8_t* st = base + s * kGemmStageBytes;
      mbar_expect_tx(&sm->full[s], kGemmStageBytes);
      tma_load_2d(st, &map_w, &sm->full[s], (ks0 + i) * kGemmBK, n_tile * 128);
      tma_load_2d(st + kGemmWBytes, &map_x, &sm->full[s], (ks0 + i) * kGemmBK, 0);
    }
  } else if (tid == 32) {
    // ---- MMA issuer
    const uint32_t idesc = make_idesc(p.is_bf16 ? 1 : 0, 0, 32);
    bool ok = true;
    for (int i = 0; i < steps && ok; ++i) {
      const int s = i % kGemmStages;
      ok = mbar_wait_or_abort(&sm->full[s], (i / kGemmStages) & 1, abort_flag);
      if (!ok) break;
      tc_fence_after();
      const uint32_t wa = smem_u32(base + s * kGemmStageBytes), xa = wa + kGemmWBytes;
#pragma unroll
      for (int k = 0; k < 4; ++k)
        umma(tmem, make_desc(wa + k * 32, 16, 1024, 2), make_desc(xa + k * 32, 16, 1024, 2), idesc, (i > 0 || k > 0));
      umma_commit(&sm->empty[s]);   // the stage may be refilled once these MMAs have read it
    }
    if (ok && steps > 0) umma_commit(&sm->done);
    else if (!ok && *abort_flag == 0) { *abort_flag = 1; report(p.status, TKV_DEV_TIMEOUT); }
  }
  __syncwarp();
  // ---- epilogue: lane = weight row of the tile, 32 TMEM columns = activation rows
  if (steps > 0 && !mbar_wait_or_abort(&sm->done, 0, abort_flag) && *abort_flag == 0) {
    *abort_flag = 1; report(p.status, TKV_DEV_TIMEOUT);
  }
  __syncthreads();                                   // one decision for the whole CTA
  const bool have = steps > 0 && *abort_flag == 0;
  tc_fence_after();
  const int n = n_tile * 128 + tid;
  float acc[32];
  if (have) tmem_ld32(tmem + ((uint32_t)(warp * 32) << 16), acc);
  if (n < p.n) {
    float* out = p.partial + (int64_t)split * p.m * p.n + n;
#pragma unroll
    for (int m = 0; m < 32; ++m)
      if (m < p.m) out[(int64_t)m * p.n] = have ? acc[m] : 0.f;
  }
  // An aborting CTA drains the copies it started before its shared memory is released.
  if (tid == 0 && *abort_flag != 0)
    for (int i = 0; i < steps && i < kGemmStages; ++i) mbar_wait(&sm->full[i % kGemmStages], 0);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kGemmTmemCols));
}

// Number of K splits: fill the 148 SMs, keep a few K steps per CTA, avoid a short second wave.
static int choose_splits(int n_tiles, int k_steps) {
  int best = 1; long best_cost = -1;
  for (int s = 1; s <= 16 && s <= k_steps; ++s) {
    const long waves = ((long)n_tiles * s + 295) / 296;  // two CTAs fit on an SM
    const long cost = waves * ((k_steps + s - 1) / s + 3);
    if (best_cost < 0 || cost < best_cost) { best = s; best_cost = cost; }
  }
  return best;
}

}  // namespace tkv

extern "C" int tkv_skinny_gemm_splits(int m, int n, int k) {
  if (m <= 0 || m > 32 || n <= 0 || k <= 0 || k % tkv::kGemmBK != 0) return 0;
  return tkv::choose_splits((n + 127) / 128, k / tkv::kGemmBK);
}

extern "C" int tkv_skinny_gemm(const void* x, const void* w, float* partial, int m, int n, int k, int dtype,
                               int32_t* status, tkv_stream_t stream) {
  using namespace tkv;
  if (!x || !w || !partial) return fail(TKV_ERR_ARG, "tkv_skinny_gemm: NULL pointer argument");
  if (dtype != TKV_BF16 && dtype != TKV_F16) return fail(TKV_ERR_UNSUPPORTED, "tkv_skinny_gemm: dtype %d", dtype);
  if (m <= 0 || m > 32 || n <= 0 || k <= 0 || k % kGemmBK != 0)
    return fail(TKV_ERR_UNSUPPORTED, "tkv_skinny_gemm: m=%d n=%d k=%d (supported: m <= 32, k %% 64 == 0)", m, n, k);
  if (!aligned16(x) || !aligned16(w) || !aligned16(partial)) return fail(TKV_ERR_ARG, "tkv_skinny_gemm: pointers must be 16-byte aligned");
  CUtensorMap mw, mx;
  int rc = make_map_2d(&mw, w, k, n, kGemmBK, 128, dtype);
  if (rc != TKV_OK) return rc;
  rc = make_map_2d(&mx, x, k, m, kGemmBK, 32, dtype);
  if (rc != TKV_OK) return rc;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(skinny_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmemBytes);
    if (e != cudaSuccess) return fail(TKV_ERR_LAUNCH, "tkv_skinny_gemm: %s", cudaGetErrorString(e));
    configured = true;
  }
  GemmParams p;
  p.partial = partial; p.m = m; p.n = n; p.k_steps = k / kGemmBK;
  const int n_tiles = (n + 127) / 128;
  p.splits = choose_splits(n_tiles, p.k_steps);
  p.is_bf16 = dtype == TKV_BF16; p.status = status;
  cudaError_t e = launch_pdl(skinny_gemm_kernel, dim3((unsigned)(n_tiles * p.splits)), dim3(kGemmThreads),
                             (size_t)kGemmSmemBytes, (cudaStream_t)stream, mw, mx, p);
  if (e != cudaSuccess) return fail(TKV_ERR_LAUNCH, "tkv_skinny_gemm: %s", cudaGetErrorString(e));
  return check_launch("tkv_skinny_gemm");
}
