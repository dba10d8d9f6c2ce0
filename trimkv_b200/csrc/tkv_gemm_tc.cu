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
  uint64_t full_x[kGemmStages];     // SwiGLU variant: the activation tile of a stage has been written by the converter warps
  uint32_t tmem_base;
  int abort_flag;
};
constexpr int kGemmSmemBytes = kGemmStages * kGemmStageBytes + (int)sizeof(GemmSmem) + 1024;

struct GemmParams {
  float* partial;      // [splits, m, n]
  int m, n, k_steps, splits, is_bf16;
  int32_t* status;
  const char* gate_up; // SwiGLU variant: [m, 2 * k] of the model dtype, gate in columns [0, k), up in [k, 2k)
};

constexpr int kGemmConverters = 64;  // warps 2 and 3

// act = round(round(SiLU(g)) * u): the two roundings of F.silu(gate) * up on 16-bit tensors.
template <bool kBf16>
__device__ __forceinline__ uint32_t swiglu2(uint32_t g, uint32_t u) {
  float g0, g1, u0, u1;
  if (kBf16) {
    g0 = __uint_as_float(g << 16); g1 = __uint_as_float(g & 0xffff0000u);
    u0 = __uint_as_float(u << 16); u1 = __uint_as_float(u & 0xffff0000u);
    const float a0 = __bfloat162float(__float2bfloat16_rn(g0 / (1.0f + expf(-g0))));
    const float a1 = __bfloat162float(__float2bfloat16_rn(g1 / (1.0f + expf(-g1))));
    const __nv_bfloat162 v = __floats2bfloat162_rn(a0 * u0, a1 * u1);
    return *reinterpret_cast<const uint32_t*>(&v);
  }
  const float2 gf = __half22float2(*reinterpret_cast<const __half2*>(&g));
  const float2 uf = __half22float2(*reinterpret_cast<const __half2*>(&u));
  g0 = gf.x; g1 = gf.y; u0 = uf.x; u1 = uf.y;
  const float a0 = __half2float(__float2half_rn(g0 / (1.0f + expf(-g0))));
  const float a1 = __half2float(__float2half_rn(g1 / (1.0f + expf(-g1))));
  const __half2 v = __floats2half2_rn(a0 * u0, a1 * u1);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// kSwiglu: the activation operand is not loaded but computed, x[m, k] = SiLU(gate[m, k]) * up[m, k] from the output of
// the gate|up projection (what Qwen3MLP.forward feeds down_proj, src/trimkv/models/qwen3/modeling_trimkv_qwen3.py:
// 120-122): warps 2 and 3 read the two 32 x 64 tiles of a K step, apply the activation with the eager sequence's
// roundings and write the tile into the stage in the layout TMA would have given it, so the separate SiLU*up kernel
// and its round trip through memory disappear.
template <bool kSwiglu>
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
    for (int s = 0; s < kGemmStages; ++s) {
      mbar_init(&sm->full[s], 1); mbar_init(&sm->empty[s], 1); mbar_init(&sm->full_x[s], kGemmConverters);
    }
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
      mbar_expect_tx(&sm->full[i], kSwiglu ? kGemmWBytes : kGemmStageBytes);
      tma_load_2d(base + i * kGemmStageBytes, &map_w, &sm->full[i], (ks0 + i) * kGemmBK, n_tile * 128);
    }
  }
  grid_dependency_wait();  // x is produced by the preceding kernel of the stream
  grid_launch_dependents();  // the consumer of the partial sums may be scheduled; it waits for this grid before reading

  if (tid == 0) {
    // ---- producer: keeps up to kGemmStages tiles of W and x in flight
    if (!kSwiglu)
      for (int i = 0; i < pre; ++i)
        tma_load_2d(base + i * kGemmStageBytes + kGemmWBytes, &map_x, &sm->full[i], (ks0 + i) * kGemmBK, 0);
    for (int i = pre; i < steps; ++i) {
      const int s = i % kGemmStages;
      if (!mbar_wait_or_abort(&sm->empty[s], ((i / kGemmStages) - 1) & 1, abort_flag)) {
        if (*abort_flag == 0) { *abort_flag = 1; report(p.status, TKV_DEV_TIMEOUT); }
        break;
      }
      uint8_t* st = base + s * kGemmStageBytes;
      mbar_expect_tx(&sm->full[s], kSwiglu ? kGemmWBytes : kGemmStageBytes);
      tma_load_2d(st, &map_w, &sm->full[s], (ks0 + i) * kGemmBK, n_tile * 128);
      if (!kSwiglu) tma_load_2d(st + kGemmWBytes, &map_x, &sm->full[s], (ks0 + i) * kGemmBK, 0);
    }
  } else if (kSwiglu && warp >= 2) {
    // ---- converters: 64 threads, 256 16-byte chunks per K step (32 rows x 8 chunks), 4 per thread
    const int ct = tid - 64;
    const int64_t k_total = (int64_t)p.k_steps * kGemmBK;
    for (int i = 0; i < steps; ++i) {
      const int s = i % kGemmStages;
      if (i >= kGemmStages && !mbar_wait_or_abort(&sm->empty[s], ((i / kGemmStages) - 1) & 1, abort_flag)) {
        if (*abort_flag == 0) { *abort_flag = 1; report(p.status, TKV_DEV_TIMEOUT); }
        break;
      }
      uint8_t* xt = base + s * kGemmStageBytes + kGemmWBytes;
      const int64_t k0 = (int64_t)(ks0 + i) * kGemmBK;
      uint4 g[4], u[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int idx = ct + kGemmConverters * q, r = idx >> 3, c = idx & 7;
        g[q] = make_uint4(0, 0, 0, 0); u[q] = make_uint4(0, 0, 0, 0);
        if (r < p.m) {
          const char* row = p.gate_up + ((int64_t)r * 2 * k_total + k0 + c * 8) * 2;
          g[q] = ld16(row);
          u[q] = ld16(row + k_total * 2);
        }
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int idx = ct + kGemmConverters * q, r = idx >> 3, c = idx & 7;
        uint4 o;
        if (p.is_bf16) {
          o.x = swiglu2<true>(g[q].x, u[q].x); o.y = swiglu2<true>(g[q].y, u[q].y);
          o.z = swiglu2<true>(g[q].z, u[q].z); o.w = swiglu2<true>(g[q].w, u[q].w);
        } else {
          o.x = swiglu2<false>(g[q].x, u[q].x); o.y = swiglu2<false>(g[q].y, u[q].y);
          o.z = swiglu2<false>(g[q].z, u[q].z); o.w = swiglu2<false>(g[q].w, u[q].w);
        }
        st16(xt + r * 128 + ((c ^ (r & 7)) << 4), o);     // K-major rows of 128 bytes, 128-byte swizzle
      }
      fence_async_smem();
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&sm->full_x[s])) : "memory");
    }
  } else if (tid == 32) {
    // ---- MMA issuer
    const uint32_t idesc = make_idesc(p.is_bf16 ? 1 : 0, 0, 32);
    bool ok = true;
    for (int i = 0; i < steps && ok; ++i) {
      const int s = i % kGemmStages;
      ok = mbar_wait_or_abort(&sm->full[s], (i / kGemmStages) & 1, abort_flag);
      if (ok && kSwiglu) ok = mbar_wait_or_abort(&sm->full_x[s], (i / kGemmStages) & 1, abort_flag);
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

static int launch_skinny(const void* x, const void* gate_up, const void* w, float* partial, int m, int n, int k, int dtype,
                         int32_t* status, tkv_stream_t stream, const char* who) {
  using namespace tkv;
  const bool swiglu = gate_up != nullptr;
  if ((!swiglu && !x) || !w || !partial) return fail(TKV_ERR_ARG, "%s: NULL pointer argument", who);
  if (dtype != TKV_BF16 && dtype != TKV_F16) return fail(TKV_ERR_UNSUPPORTED, "%s: dtype %d", who, dtype);
  if (m <= 0 || m > 32 || n <= 0 || k <= 0 || k % kGemmBK != 0)
    return fail(TKV_ERR_UNSUPPORTED, "%s: m=%d n=%d k=%d (supported: m <= 32, k %% 64 == 0)", who, m, n, k);
  if ((!swiglu && !aligned16(x)) || (swiglu && !aligned16(gate_up)) || !aligned16(w) || !aligned16(partial))
    return fail(TKV_ERR_ARG, "%s: pointers must be 16-byte aligned", who);
  CUtensorMap mw, mx;
  int rc = make_map_2d(&mw, w, k, n, kGemmBK, 128, dtype);
  if (rc != TKV_OK) return rc;
  // the SwiGLU variant loads nothing through the activation map; it gets the weight map as a valid placeholder
  rc = swiglu ? make_map_2d(&mx, w, k, n, kGemmBK, 128, dtype) : make_map_2d(&mx, x, k, m, kGemmBK, 32, dtype);
  if (rc != TKV_OK) return rc;
  static bool configured[2] = {false, false};
  if (!configured[swiglu]) {
    cudaError_t e = swiglu ? cudaFuncSetAttribute(skinny_gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmemBytes)
                           : cudaFuncSetAttribute(skinny_gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmemBytes);
    if (e != cudaSuccess) return fail(TKV_ERR_LAUNCH, "%s: %s", who, cudaGetErrorString(e));
    configured[swiglu] = true;
  }
  GemmParams p;
  p.partial = partial; p.m = m; p.n = n; p.k_steps = k / kGemmBK;
  const int n_tiles = (n + 127) / 128;
  p.splits = choose_splits(n_tiles, p.k_steps);
  p.is_bf16 = dtype == TKV_BF16; p.status = status; p.gate_up = (const char*)gate_up;
  cudaError_t e = swiglu
      ? launch_pdl(skinny_gemm_kernel<true>, dim3((unsigned)(n_tiles * p.splits)), dim3(kGemmThreads), (size_t)kGemmSmemBytes,
                   (cudaStream_t)stream, mw, mx, p)
      : launch_pdl(skinny_gemm_kernel<false>, dim3((unsigned)(n_tiles * p.splits)), dim3(kGemmThreads), (size_t)kGemmSmemBytes,
                   (cudaStream_t)stream, mw, mx, p);
  if (e != cudaSuccess) return fail(TKV_ERR_LAUNCH, "%s: %s", who, cudaGetErrorString(e));
  return check_launch(who);
}

extern "C" int tkv_skinny_gemm(const void* x, const void* w, float* partial, int m, int n, int k, int dtype,
                               int32_t* status, tkv_stream_t stream) {
  if (!x) return tkv::fail(TKV_ERR_ARG, "tkv_skinny_gemm: NULL pointer argument");
  return launch_skinny(x, nullptr, w, partial, m, n, k, dtype, status, stream, "tkv_skinny_gemm");
}

extern "C" int tkv_skinny_gemm_swiglu(const void* gate_up, const void* w, float* partial, int m, int n, int k, int dtype,
                                      int32_t* status, tkv_stream_t stream) {
  if (!gate_up) return tkv::fail(TKV_ERR_ARG, "tkv_skinny_gemm_swiglu: NULL pointer argument");
  return launch_skinny(nullptr, gate_up, w, partial, m, n, k, dtype, status, stream, "tkv_skinny_gemm_swiglu");
}
