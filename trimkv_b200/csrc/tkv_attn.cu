// Split-KV varlen GQA decode attention over the capacity-strided (or packed) flat cache.
//
// Replaces batched_dynamic_kv_budget_attention_forward -> flash_attn_varlen_func
// (src/trimkv/attn/flash_attn.py:79-151): there every (request, KV head) pair becomes one varlen
// "sequence" of an MQA problem after a split/stack/permute of Q and a host sync for max_seqlen_k.
// Here the segment table is read on the device; a work item is (segment, chunk of kChunk tokens); each
// item produces an unnormalised partial output and its (max, sum) in log2 domain, and a combine kernel
// merges the chunks of a segment.  Per cached token the kernel reads 2*D*elem bytes exactly once.
#include "tkv_common.cuh"
#include "tkv_attn.cuh"

namespace tkv {

template <int kDtype> struct Cvt;
template <> struct Cvt<TKV_BF16> {
  static __device__ __forceinline__ void unpack(uint32_t w, float& lo, float& hi) {
    lo = __uint_as_float(w << 16);
    hi = __uint_as_float(w & 0xffff0000u);
  }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
};
template <> struct Cvt<TKV_F16> {
  static __device__ __forceinline__ void unpack(uint32_t w, float& lo, float& hi) {
    float2 f = __half22float2(*reinterpret_cast<__half2*>(&w));
    lo = f.x; hi = f.y;
  }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
};

template <int kDtype>
__device__ __forceinline__ void unpack8(uint4 v, float* f) {
  Cvt<kDtype>::unpack(v.x, f[0], f[1]);
  Cvt<kDtype>::unpack(v.y, f[2], f[3]);
  Cvt<kDtype>::unpack(v.z, f[4], f[5]);
  Cvt<kDtype>::unpack(v.w, f[6], f[7]);
}

constexpr int kAttnWarps = 4;
constexpr int kAttnThreads = kAttnWarps * 32;
constexpr int kTokUnroll = 4;

// One CTA = one (segment, chunk).  kLanes = D/8 lanes cover one row with 16-byte loads, so a warp
// handles 32/kLanes tokens per step; each such lane group keeps its own online-softmax state.
template <int kDtype, int kD, int kG>
__global__ void __launch_bounds__(kAttnThreads)
decode_attn_split_kernel(AttnParams p) {
  constexpr int kLanes = kD / 8;
  constexpr int kGroupsPerWarp = 32 / kLanes;
  constexpr int kStates = kAttnWarps * kGroupsPerWarp;
  extern __shared__ __align__(16) float smem[];  // [kStates][kG][kD] partial outputs, then [kStates][kG][2]
  const int seg = blockIdx.x / p.nchunks, chunk = blockIdx.x - seg * p.nchunks;
  const int len = min(p.seg_len[seg], p.max_len);
  const int t0 = chunk * p.chunk;
  if (t0 >= len) return;
  const int t1 = min(len, t0 + p.chunk);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int grp = lane / kLanes, gl = lane - grp * kLanes;
  const int b = seg / p.hkv, h = seg - b * p.hkv;
  const int64_t row_bytes = (int64_t)kD * 2;
  const int64_t start = p.seg_start != nullptr ? (int64_t)p.seg_start[seg] : (int64_t)seg * p.cap;
  const char* kb = p.k + start * row_bytes + gl * 16;
  const char* vb = p.v + start * row_bytes + gl * 16;

  float qf[kG][8];
#pragma unroll
  for (int g = 0; g < kG; ++g) {
    const char* qp = p.q + ((int64_t)b * p.q_sb + (int64_t)(h * kG + g) * p.q_sh) * 2 + gl * 16;
    unpack8<kDtype>(ld16(qp), qf[g]);
#pragma unroll
    for (int d = 0; d < 8; ++d) qf[g][d] *= p.scale_log2;
  }
  float m[kG], l[kG], acc[kG][8];
#pragma unroll
  for (int g = 0; g < kG; ++g) {
    m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
    for (int d = 0; d < 8; ++d) acc[g][d] = 0.f;
  }

  constexpr int kStride = kStates;  // tokens advanced by the whole CTA per sub-step
#pragma unroll 1
  for (int tb = t0 + warp * kGroupsPerWarp; tb < t1; tb += kStride * kTokUnroll) {
    const int t = tb + grp;  // the loop bound is warp-uniform; tokens past t1 are masked below
    uint4 kr[kTokUnroll], vr[kTokUnroll];
#pragma unroll
    for (int u = 0; u < kTokUnroll; ++u) {
      const int tt = t + u * kStride;
      if (tt < t1) {
        kr[u] = ld16_stream(kb + (int64_t)tt * row_bytes);
        vr[u] = ld16_stream(vb + (int64_t)tt * row_bytes);
      } else {
        kr[u] = make_uint4(0, 0, 0, 0); vr[u] = make_uint4(0, 0, 0, 0);
      }
    }
    float s[kTokUnroll][kG];
#pragma unroll
    for (int u = 0; u < kTokUnroll; ++u) {
      float kf[8];
      unpack8<kDtype>(kr[u], kf);
#pragma unroll
      for (int g = 0; g < kG; ++g) {
        float x = 0.f;
#pragma unroll
        for (int d = 0; d < 8; ++d) x = fmaf(qf[g][d], kf[d], x);
        s[u][g] = x;
      }
    }
#pragma unroll
    for (int u = 0; u < kTokUnroll; ++u)
#pragma unroll
      for (int g = 0; g < kG; ++g) {
        float x = s[u][g];
#pragma unroll
        for (int o = kLanes / 2; o >= 1; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
        s[u][g] = (t + u * kStride < t1) ? x : -INFINITY;
      }
#pragma unroll
    for (int g = 0; g < kG; ++g) {
      float mn = m[g];
#pragma unroll
      for (int u = 0; u < kTokUnroll; ++u) mn = fmaxf(mn, s[u][g]);
      if (mn == -INFINITY) continue;  // only masked tokens so far (uniform inside the lane group)
      const float corr = exp2f(m[g] - mn);
      m[g] = mn;
      l[g] *= corr;
#pragma unroll
      for (int d = 0; d < 8; ++d) acc[g][d] *= corr;
    }
#pragma unroll
    for (int u = 0; u < kTokUnroll; ++u) {
      float vf[8];
      unpack8<kDtype>(vr[u], vf);
#pragma unroll
      for (int g = 0; g < kG; ++g) {
        const float pw = (m[g] == -INFINITY) ? 0.f : exp2f(s[u][g] - m[g]);
        l[g] += pw;
#pragma unroll
        for (int d = 0; d < 8; ++d) acc[g][d] = fmaf(pw, vf[d], acc[g][d]);
      }
    }
  }

  // Merge the kStates lane-group states of this CTA.
  float* so = smem;                           // [kStates][kG][kD]
  float* sml = smem + kStates * kG * kD;      // [kStates][kG][2]
  const int state = warp * kGroupsPerWarp + grp;
#pragma unroll
  for (int g = 0; g < kG; ++g) {
    float* dst = so + ((state * kG + g) * kD) + gl * 8;
    *reinterpret_cast<float4*>(dst) = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
    *reinterpret_cast<float4*>(dst + 4) = make_float4(acc[g][4], acc[g][5], acc[g][6], acc[g][7]);
    if (gl == 0) { sml[(state * kG + g) * 2] = m[g]; sml[(state * kG + g) * 2 + 1] = l[g]; }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kG * kD; i += kAttnThreads) {
    const int g = i / kD, d = i - g * kD;
    float mx = -INFINITY;
#pragma unroll
    for (int s_ = 0; s_ < kStates; ++s_) mx = fmaxf(mx, sml[(s_ * kG + g) * 2]);
    float o = 0.f, ls = 0.f;
#pragma unroll
    for (int s_ = 0; s_ < kStates; ++s_) {
      const float ms = sml[(s_ * kG + g) * 2];
      const float w = (ms == -INFINITY) ? 0.f : exp2f(ms - mx);
      o = fmaf(so[(s_ * kG + g) * kD + d], w, o);
      ls = fmaf(sml[(s_ * kG + g) * 2 + 1], w, ls);
    }
    if (p.nchunks == 1) {
      // Single chunk: normalise and write the final output here.
      const float r = ls > 0.f ? o / ls : 0.f;
      char* op = p.out + ((int64_t)b * p.hq + h * kG + g) * row_bytes;
      if (kDtype == TKV_BF16) reinterpret_cast<__nv_bfloat16*>(op)[d] = __float2bfloat16_rn(r);
      else reinterpret_cast<__half*>(op)[d] = __float2half_rn(r);
    } else {
      const int64_t item = (int64_t)seg * p.nchunks + chunk;
      p.part_o[(item * kG + g) * kD + d] = o;
      if (d == 0) { p.part_ml[(item * kG + g) * 2] = mx; p.part_ml[(item * kG + g) * 2 + 1] = ls; }
    }
  }
}

// Merged output value of (segment, query head g, dimension d) from the chunk partials; 0 for an empty segment.
// Called by every thread of a kD-thread block (it synchronises the block).
constexpr int kMergeEarly = 32;   // partial outputs per thread requested before anything else is known

// Requests this thread's dimension of the first kMergeEarly chunk partials of (segment, row g).  Nothing here depends
// on the segment's length, so the loads go out together with the length load; chunks beyond the live ones are
// read too (the workspace covers nchunks per segment) and discarded by merge_partials.
//
// That pays while most of the requested chunks exist (segments of one length: the decode benchmark has 17 chunks of
// which 16-17 are live).  Where the grid allows many more chunks than a typical segment has (ragged lengths: up to 32
// chunks for a mean of 11), the blind loads would mostly fetch stale partials, so beyond kMergeBlind chunks the length is
// read first and only the live chunks are requested: one more dependent round trip, a third of the traffic.
constexpr int kMergeBlind = 24;
template <int kD>
__device__ __forceinline__ void load_partials_early(const AttnParams& p, int seg, int g, int d, float (&early)[kMergeEarly]) {
  const int64_t it0 = ((int64_t)seg * p.nchunks) * p.rows + g;
  int live = p.nchunks;
  if (p.nchunks > kMergeBlind) live = (min(p.seg_len[seg], p.max_len) + p.chunk - 1) / p.chunk;
#pragma unroll
  for (int c = 0; c < kMergeEarly; ++c)
    early[c] = (p.nchunks > 1 && c < live) ? p.part_o[(it0 + (int64_t)c * p.rows) * kD + d] : 0.f;
}

template <int kD>
__device__ __forceinline__ float merge_partials(const AttnParams& p, int seg, int g, int d, int len,
                                                float (&early)[kMergeEarly]) {
  const int G = p.rows;   // query rows per segment (the G query heads, times the query tokens if there are several)
  float r = 0.f;
  const int nact = (len + p.chunk - 1) / p.chunk;
  const int64_t it0 = ((int64_t)seg * p.nchunks) * G + g;  // partial of chunk c: it0 + c*G
  if (nact <= kD) {
    // One round trip for everything: the first partial outputs of this thread's dimension were requested by the
    // caller before the length was known; thread c takes chunk c's (max, sum) pair, the block reduces them and the
    // weights go to shared memory; by then the outputs have arrived and only need the weighted sum.
    constexpr int kEarly = kMergeEarly;
    __shared__ float s_w[kD];
    __shared__ float s_red[2][kD / 32];
    const int lane = d & 31, warp = d >> 5;
#pragma unroll
    for (int c = 0; c < kEarly; ++c) early[c] = c < nact ? early[c] : 0.f;   // chunks without tokens hold stale bytes
    float mc = -INFINITY, lc = 0.f;
    if (d < nact) {
      const float2 ml = *reinterpret_cast<const float2*>(&p.part_ml[(it0 + (int64_t)d * G) * 2]);
      mc = ml.x; lc = ml.y;
    }
    float mx = mc;
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) s_red[0][warp] = mx;
    __syncthreads();
    mx = s_red[0][0];
#pragma unroll
    for (int w = 1; w < kD / 32; ++w) mx = fmaxf(mx, s_red[0][w]);
    const float wgt = (mc == -INFINITY) ? 0.f : exp2f(mc - mx);
    s_w[d] = d < nact ? wgt : 0.f;
    float ls = lc * wgt;
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) ls += __shfl_xor_sync(0xffffffffu, ls, o);
    if (lane == 0) s_red[1][warp] = ls;
    __syncthreads();
    ls = 0.f;
#pragma unroll
    for (int w = 0; w < kD / 32; ++w) ls += s_red[1][w];
    float o = 0.f;
#pragma unroll
    for (int c = 0; c < kEarly; ++c) o = fmaf(early[c], s_w[c], o);   // same order of additions as a plain loop
#pragma unroll 8
    for (int c = kEarly; c < nact; ++c) o = fmaf(p.part_o[(it0 + (int64_t)c * G) * kD + d], s_w[c], o);
    r = ls > 0.f ? o / ls : 0.f;
  } else {
    float mx = -INFINITY;
    for (int c = 0; c < nact; ++c) mx = fmaxf(mx, p.part_ml[(it0 + (int64_t)c * G) * 2]);
    float o = 0.f, ls = 0.f;
    for (int c = 0; c < nact; ++c) {
      const int64_t it = it0 + (int64_t)c * G;
      const float mc = p.part_ml[it * 2];
      const float w = (mc == -INFINITY) ? 0.f : exp2f(mc - mx);
      o = fmaf(p.part_o[it * kD + d], w, o);
      ls = fmaf(p.part_ml[it * 2 + 1], w, ls);
    }
    r = ls > 0.f ? o / ls : 0.f;
  }
  return r;
}

// Merges the chunk partials of one segment; also writes zeros for empty segments.
template <int kDtype, int kD>
__global__ void __launch_bounds__(kD) decode_attn_combine_kernel(AttnParams p) {
  const int seg = blockIdx.x, g = blockIdx.y, d = threadIdx.x;
  grid_dependency_wait();  // launched with programmatic serialization behind the split kernel
  float early[kMergeEarly];
  load_partials_early<kD>(p, seg, g, d, early);
  if (p.seg_len[seg] > p.max_len && g == 0 && d == 0) report(p.status, TKV_DEV_LEN_BOUND);
  const int len = min(p.seg_len[seg], p.max_len);
  const int b = seg / p.hkv, h = seg - b * p.hkv;
  const int G = p.hq / p.hkv;
  // g is the query row of the segment: head g, or (several query tokens) token g / G, head g % G
  char* op = p.out + (((int64_t)b * p.q_tokens + g / G) * p.hq + h * G + g % G) * (int64_t)kD * 2;
  float r = 0.f;
  if (len > 0) {
    if (p.nchunks == 1) return;  // written by the split kernel
    r = merge_partials<kD>(p, seg, g, d, len, early);
  }
  if (kDtype == TKV_BF16) reinterpret_cast<__nv_bfloat16*>(op)[d] = __float2bfloat16_rn(r);
  else reinterpret_cast<__half*>(op)[d] = __float2half_rn(r);
}

__device__ __forceinline__ void st_release_sys(int32_t* p, int v) {
  asm volatile("st.release.sys.global.b32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int32_t* p) {
  int v;
  asm volatile("ld.acquire.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// The merge of a head-sharded decode step, fused with the exchange that follows it: each value goes to this
// rank's column block of the gathered [batch, Hq_total * D] buffer of EVERY rank with a plain store (peer memory,
// NVLink); when the whole grid has stored (fence + counter), the last CTA raises this rank's flag on every peer
// with a system-scope release.  Nothing is read from peer memory.
template <int kDtype, int kD>
__global__ void __launch_bounds__(kD) decode_attn_combine_push_kernel(AttnParams p, PushParams pp) {
  const int seg = blockIdx.x, g = blockIdx.y, d = threadIdx.x;
  grid_dependency_wait();
  float early[kMergeEarly];
  load_partials_early<kD>(p, seg, g, d, early);
  if (p.seg_len[seg] > p.max_len && g == 0 && d == 0) report(p.status, TKV_DEV_LEN_BOUND);
  const int len = min(p.seg_len[seg], p.max_len);
  const int b = seg / p.hkv, h = seg - b * p.hkv;
  const int G = p.hq / p.hkv;
  uint16_t bits = 0;
  if (len > 0) {
    if (p.nchunks == 1) {
      bits = reinterpret_cast<const uint16_t*>(p.out + ((int64_t)b * p.hq + h * G + g) * (int64_t)kD * 2)[d];
    } else {
      const float r = merge_partials<kD>(p, seg, g, d, len, early);
      if (kDtype == TKV_BF16) bits = __bfloat16_as_ushort(__float2bfloat16_rn(r));
      else bits = __half_as_ushort(__float2half_rn(r));
    }
  }
  const int64_t off = ((int64_t)b * pp.row_stride + pp.col_offset + (int64_t)(h * G + g) * kD + d) * 2;
  for (int r = 0; r < pp.world; ++r) *reinterpret_cast<uint16_t*>(pp.peer_out[r] + off) = bits;
  __threadfence_system();
  __syncthreads();
  if (d == 0) {
    const int total = gridDim.x * gridDim.y;
    if (atomicAdd(&pp.sync[0], 1) == total - 1) {
      pp.sync[0] = 0;
      __threadfence_system();
      const int epoch = pp.sync[1] + 1;
      pp.sync[1] = epoch;
      for (int r = 0; r < pp.world; ++r)
        if (r != pp.rank) st_release_sys(pp.peer_flags[r] + pp.rank, epoch);
    }
  }
}

// Waits until every peer has raised its flag for the next exchange (the counterpart of the kernel above on the
// receiving side).  One warp, lane r watches rank r; bounded: after about four seconds the lane gives up, the
// status word says TKV_DEV_TIMEOUT and the stream carries on, so a missing peer cannot hang the GPU.
__global__ void __launch_bounds__(32) peer_wait_kernel(const int32_t* flags, int32_t* sync, int world, int rank,
                                                       int max_polls, int32_t* status) {
  const int lane = threadIdx.x;
  const int expected = sync[2] + 1;
  __syncwarp();
  if (lane < world && lane != rank) {
    int spins = 0;
    while (ld_acquire_sys(flags + lane) - expected < 0) {
      if (++spins > max_polls) { report(status, TKV_DEV_TIMEOUT); break; }
      __nanosleep(200);
    }
  }
  __syncwarp();
  if (lane == 0) sync[2] = expected;
}

template <int kDtype, int kD, int kG>
static int launch_split(const AttnParams& p, int nseg, cudaStream_t st) {
  constexpr int kStates = kAttnWarps * (32 / (kD / 8));
  const size_t smem = (size_t)kStates * kG * (kD + 2) * sizeof(float);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(decode_attn_split_kernel<kDtype, kD, kG>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(TKV_ERR_LAUNCH, "tkv_decode_attn: %s", cudaGetErrorString(e));
  }
  decode_attn_split_kernel<kDtype, kD, kG><<<(unsigned)((int64_t)nseg * p.nchunks), kAttnThreads, smem, st>>>(p);
  return check_launch("tkv_decode_attn(split)");
}

template <int kDtype, int kD>
static int launch_for_g(const AttnParams& p, int nseg, int G, cudaStream_t st, const PushParams* push) {
  int rc;
  switch (G) {
    case 1: rc = launch_split<kDtype, kD, 1>(p, nseg, st); break;
    case 2: rc = launch_split<kDtype, kD, 2>(p, nseg, st); break;
    case 3: rc = launch_split<kDtype, kD, 3>(p, nseg, st); break;
    case 4: rc = launch_split<kDtype, kD, 4>(p, nseg, st); break;
    case 5: rc = launch_split<kDtype, kD, 5>(p, nseg, st); break;
    case 6: rc = launch_split<kDtype, kD, 6>(p, nseg, st); break;
    case 7: rc = launch_split<kDtype, kD, 7>(p, nseg, st); break;
    case 8: rc = launch_split<kDtype, kD, 8>(p, nseg, st); break;
    default: return fail(TKV_ERR_UNSUPPORTED, "tkv_decode_attn: %d query heads per KV head (supported: 1..8)", G);
  }
  if (rc != TKV_OK) return rc;
  if (push != nullptr) decode_attn_combine_push_kernel<kDtype, kD><<<dim3(nseg, G), kD, 0, st>>>(p, *push);
  else decode_attn_combine_kernel<kDtype, kD><<<dim3(nseg, G), kD, 0, st>>>(p);
  return check_launch("tkv_decode_attn(combine)");
}

int launch_decode_attn_combine(const AttnParams& p, int nseg, int G, int head_dim, int kv_dtype, cudaStream_t st,
                               const PushParams* push) {
  cudaError_t e;
  if (push != nullptr && head_dim == 128 && kv_dtype == TKV_BF16) e = launch_pdl(decode_attn_combine_push_kernel<TKV_BF16, 128>, dim3(nseg, G), dim3(128), 0, st, p, *push);
  else if (push != nullptr && head_dim == 128 && kv_dtype == TKV_F16) e = launch_pdl(decode_attn_combine_push_kernel<TKV_F16, 128>, dim3(nseg, G), dim3(128), 0, st, p, *push);
  else if (head_dim == 128 && kv_dtype == TKV_BF16) e = launch_pdl(decode_attn_combine_kernel<TKV_BF16, 128>, dim3(nseg, p.rows), dim3(128), 0, st, p);
  else if (head_dim == 128 && kv_dtype == TKV_F16) e = launch_pdl(decode_attn_combine_kernel<TKV_F16, 128>, dim3(nseg, p.rows), dim3(128), 0, st, p);
  else return fail(TKV_ERR_UNSUPPORTED, "tkv_decode_attn(combine): head_dim=%d dtype=%d", head_dim, kv_dtype);
  if (e != cudaSuccess) return fail(TKV_ERR_LAUNCH, "tkv_decode_attn(combine): %s", cudaGetErrorString(e));
  return check_launch("tkv_decode_attn(combine)");
}

// Which split kernel serves a problem: the tensor-core one whenever its requirements hold (16-bit, head_dim 128,
// at most 8 query heads per KV head, and at least one 128-row TMA box of rows whose count the caller stated);
// everything else (head_dim 64, tiny caches, a packed layout of unstated size) runs on the CUDA-core kernel.
static bool use_tensor_core_path(int head_dim, int kv_dtype, int G, int64_t rows) {
  return head_dim == 128 && (kv_dtype == TKV_BF16 || kv_dtype == TKV_F16) && G <= 8 && rows >= 128;
}

int attn_chunk_tokens(int nseg, int max_len) {
  // Enough work items to fill 148 SMs several times over, but chunks long enough to amortise the merge.
  int chunk = 512;
  while (chunk > 64 && (int64_t)nseg * ((max_len + chunk - 1) / chunk) < 148 * 8) chunk >>= 1;
  return chunk;
}

int launch_decode_attn_simt(const AttnParams& p, int nseg, int G, int head_dim, int kv_dtype, cudaStream_t st,
                            const PushParams* push = nullptr) {
  if (kv_dtype == TKV_BF16 && head_dim == 128) return launch_for_g<TKV_BF16, 128>(p, nseg, G, st, push);
  if (kv_dtype == TKV_F16 && head_dim == 128) return launch_for_g<TKV_F16, 128>(p, nseg, G, st, push);
  if (kv_dtype == TKV_BF16 && head_dim == 64) return launch_for_g<TKV_BF16, 64>(p, nseg, G, st, push);
  if (kv_dtype == TKV_F16 && head_dim == 64) return launch_for_g<TKV_F16, 64>(p, nseg, G, st, push);
  return fail(TKV_ERR_UNSUPPORTED, "tkv_decode_attn: head_dim=%d dtype=%d (supported: bf16/f16, 64 or 128)", head_dim,
              kv_dtype);
}

}  // namespace tkv

extern "C" size_t tkv_decode_attn_workspace_bytes(int batch, int hq, int hkv, int head_dim, int max_len) {
  if (batch <= 0 || hq <= 0 || hkv <= 0 || head_dim <= 0 || max_len <= 0 || hq % hkv != 0) return 0;
  const int nseg = batch * hkv, G = hq / hkv;
  // Large enough for either split kernel (they cut segments into chunks of different lengths).
  int chunk = tkv::attn_chunk_tokens(nseg, max_len);
  if (head_dim == 128 && tkv::attn_tc_chunk_tokens() < chunk) chunk = tkv::attn_tc_chunk_tokens();
  const int64_t items = (int64_t)nseg * ((max_len + chunk - 1) / chunk);
  return (size_t)(items * G * (head_dim + 2) * sizeof(float) + 256);
}

namespace tkv {
// Work items the ragged entry point sizes its grid for: every segment has at least one, and a segment of n tokens
// has ceil(n / chunk) <= n / chunk + 1.
static int64_t ragged_items(int nseg, int max_len, int64_t total_len_bound) {
  const int chunk = attn_tc_chunk_tokens();
  const int64_t dense = (int64_t)nseg * ((max_len + chunk - 1) / chunk);
  const int64_t bound = total_len_bound / chunk + nseg;
  return bound < dense ? bound : dense;
}
}  // namespace tkv

extern "C" size_t tkv_decode_attn_ragged_workspace_bytes(int batch, int hq, int hkv, int head_dim, int max_len,
                                                         int64_t total_len_bound) {
  const size_t base = tkv_decode_attn_workspace_bytes(batch, hq, hkv, head_dim, max_len);
  if (base == 0 || total_len_bound < 0) return 0;
  return ((base + 255) / 256) * 256 + 256 + (size_t)tkv::ragged_items(batch * hkv, max_len, total_len_bound) * sizeof(int2);
}

static int decode_attn_impl(const char* who, const void* q, int64_t q_sb, int64_t q_sh,
                            const void* k_cache, const void* v_cache,
                            const int32_t* seg_len, const int32_t* seg_start, int64_t cap,
                            void* out, void* workspace, size_t workspace_bytes,
                            int batch, int hq, int hkv, int head_dim, int kv_dtype,
                            float scale, int max_len, int64_t total_len_bound, int32_t* status, tkv_stream_t stream,
                            const tkv::PushParams* push = nullptr, int q_tokens = 1, int64_t q_st = 0) {
  using namespace tkv;
  if (!q || !k_cache || !v_cache || !seg_len || !out) return fail(TKV_ERR_ARG, "%s: NULL pointer argument", who);
  if (batch < 0 || hq <= 0 || hkv <= 0 || hq % hkv != 0 || head_dim <= 0 || max_len <= 0)
    return fail(TKV_ERR_ARG, "%s: bad sizes batch=%d hq=%d hkv=%d head_dim=%d max_len=%d", who, batch, hq, hkv,
                head_dim, max_len);
  if (seg_start == nullptr && cap <= 0) return fail(TKV_ERR_ARG, "%s: cap=%lld without seg_start", who, (long long)cap);
  if (!aligned16(q) || !aligned16(k_cache) || !aligned16(v_cache) || !aligned16(out))
    return fail(TKV_ERR_ARG, "%s: pointers must be 16-byte aligned", who);
  if ((q_sb * 2) % 16 || (q_sh * 2) % 16) return fail(TKV_ERR_ARG, "%s: q strides must be multiples of 16 bytes", who);
  if (batch == 0) return TKV_OK;
  const bool ragged = total_len_bound >= 0;
  const size_t base = q_tokens > 1 ? tkv_decode_attn_multi_workspace_bytes(batch, hq, hkv, head_dim, max_len, q_tokens)
                                   : tkv_decode_attn_workspace_bytes(batch, hq, hkv, head_dim, max_len);
  const size_t need = ragged ? tkv_decode_attn_ragged_workspace_bytes(batch, hq, hkv, head_dim, max_len, total_len_bound) : base;
  if (workspace == nullptr || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255u))
    return fail(TKV_ERR_ARG, "%s: workspace of %zu bytes (256-byte aligned) required, got %zu", who, need, workspace_bytes);
  const int nseg = batch * hkv, G = hq / hkv;
  AttnParams p;
  p.q = (const char*)q; p.q_sb = q_sb; p.q_sh = q_sh;
  p.k = (const char*)k_cache; p.v = (const char*)v_cache;
  p.seg_len = seg_len; p.seg_start = seg_start; p.cap = cap;
  p.out = (char*)out;
  // Rows the K/V tensors hold: capacity-strided segments, or the stated size of a packed cache.
  const int64_t kv_rows = seg_start != nullptr ? (cap > 0 ? cap : 0) : (int64_t)nseg * cap;
  const bool tc = use_tensor_core_path(head_dim, kv_dtype, G, kv_rows);
  if (q_tokens > 1 && !tc)
    return fail(TKV_ERR_UNSUPPORTED, "%s: several query tokens need bf16/f16, head_dim 128 and K/V tensors of stated size", who);
  p.chunk = tc ? attn_tc_chunk_tokens() : attn_chunk_tokens(nseg, max_len);
  p.nchunks = (max_len + p.chunk - 1) / p.chunk;
  p.q_tokens = q_tokens; p.rows = q_tokens * G; p.q_st = q_st;
  p.part_ml = reinterpret_cast<float*>(workspace);
  p.part_o = p.part_ml + (((int64_t)nseg * p.nchunks * p.rows * 2 + 63) / 64) * 64;
  p.hq = hq; p.hkv = hkv; p.max_len = max_len;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  p.work = nullptr; p.work_count = nullptr; p.work_capacity = 0;
  if (!tc) return launch_decode_attn_simt(p, nseg, G, head_dim, kv_dtype, (cudaStream_t)stream, push);
  if (ragged && p.nchunks < 256) {
    const int64_t items = ragged_items(nseg, max_len, total_len_bound);
    // Only worth the extra launch when it removes a good part of the grid.
    if (items * 4 <= (int64_t)nseg * p.nchunks * 3 && items < INT32_MAX) {
      char* w = reinterpret_cast<char*>(workspace) + ((base + 255) / 256) * 256;
      p.work_count = reinterpret_cast<const int32_t*>(w);
      p.work = reinterpret_cast<const int2*>(w + 256);
      p.work_capacity = (int)items;
      int rc = launch_attn_worklist(p, nseg, (cudaStream_t)stream);
      if (rc != TKV_OK) return rc;
    }
  }
  int rc = (q_tokens > 1 && p.rows > 16) ? launch_multi_attn_tc(p, nseg, kv_dtype, kv_rows, (cudaStream_t)stream)
                                         : launch_decode_attn_tc(p, nseg, G, kv_dtype, kv_rows, (cudaStream_t)stream);
  if (rc != TKV_OK) return rc;
  return launch_decode_attn_combine(p, nseg, G, head_dim, kv_dtype, (cudaStream_t)stream, push);
}

extern "C" int tkv_decode_attn(const void* q, int64_t q_sb, int64_t q_sh,
                               const void* k_cache, const void* v_cache,
                               const int32_t* seg_len, const int32_t* seg_start, int64_t cap,
                               void* out, void* workspace, size_t workspace_bytes,
                               int batch, int hq, int hkv, int head_dim, int kv_dtype,
                               float scale, int max_len, int32_t* status, tkv_stream_t stream) {
  return decode_attn_impl("tkv_decode_attn", q, q_sb, q_sh, k_cache, v_cache, seg_len, seg_start, cap, out, workspace,
                          workspace_bytes, batch, hq, hkv, head_dim, kv_dtype, scale, max_len, -1, status, stream);
}

extern "C" int tkv_decode_attn_ragged(const void* q, int64_t q_sb, int64_t q_sh,
                                      const void* k_cache, const void* v_cache,
                                      const int32_t* seg_len, const int32_t* seg_start, int64_t cap,
                                      void* out, void* workspace, size_t workspace_bytes,
                                      int batch, int hq, int hkv, int head_dim, int kv_dtype,
                                      float scale, int max_len, int64_t total_len_bound,
                                      int32_t* status, tkv_stream_t stream) {
  if (total_len_bound < 0) return tkv::fail(TKV_ERR_ARG, "tkv_decode_attn_ragged: total_len_bound=%lld", (long long)total_len_bound);
  return decode_attn_impl("tkv_decode_attn_ragged", q, q_sb, q_sh, k_cache, v_cache, seg_len, seg_start, cap, out,
                          workspace, workspace_bytes, batch, hq, hkv, head_dim, kv_dtype, scale, max_len, total_len_bound,
                          status, stream);
}

extern "C" size_t tkv_decode_attn_multi_workspace_bytes(int batch, int hq, int hkv, int head_dim, int max_len, int q_tokens) {
  if (batch <= 0 || hq <= 0 || hkv <= 0 || head_dim <= 0 || max_len <= 0 || hq % hkv != 0 || q_tokens <= 0) return 0;
  if (q_tokens == 1) return tkv_decode_attn_workspace_bytes(batch, hq, hkv, head_dim, max_len);
  const int64_t items = (int64_t)batch * hkv * ((max_len + tkv::attn_tc_chunk_tokens() - 1) / tkv::attn_tc_chunk_tokens());
  return (size_t)(items * q_tokens * (hq / hkv) * (head_dim + 2) * sizeof(float) + 256);
}

extern "C" int tkv_decode_attn_multi(const void* q, int64_t q_sb, int64_t q_st, int64_t q_sh,
                                     const void* k_cache, const void* v_cache, const int32_t* seg_len, int64_t cap,
                                     void* out, void* workspace, size_t workspace_bytes,
                                     int batch, int hq, int hkv, int head_dim, int kv_dtype,
                                     float scale, int max_len, int q_tokens, int32_t* status, tkv_stream_t stream) {
  if (q_tokens < 1 || (q_st * 2) % 16 != 0)
    return tkv::fail(TKV_ERR_ARG, "tkv_decode_attn_multi: q_tokens=%d, token stride %lld", q_tokens, (long long)q_st);
  if (hq > 0 && hkv > 0 && (int64_t)q_tokens * (hq / hkv) > 16 * 65535)
    return tkv::fail(TKV_ERR_UNSUPPORTED, "tkv_decode_attn_multi: too many query rows per segment");
  return decode_attn_impl("tkv_decode_attn_multi", q, q_sb, q_sh, k_cache, v_cache, seg_len, nullptr, cap, out, workspace,
                          workspace_bytes, batch, hq, hkv, head_dim, kv_dtype, scale, max_len, -1, status, stream, nullptr,
                          q_tokens, q_st);
}

extern "C" int tkv_decode_attn_push(const void* q, int64_t q_sb, int64_t q_sh,
                                    const void* k_cache, const void* v_cache,
                                    const int32_t* seg_len, const int32_t* seg_start, int64_t cap,
                                    void* out, void* workspace, size_t workspace_bytes,
                                    int batch, int hq, int hkv, int head_dim, int kv_dtype,
                                    float scale, int max_len,
                                    void* const* peer_out, int32_t* const* peer_flags, int world, int rank,
                                    int64_t out_row_stride, int64_t out_col_offset, int32_t* sync_state,
                                    int32_t* status, tkv_stream_t stream) {
  using namespace tkv;
  if (!peer_out || !peer_flags || !sync_state) return fail(TKV_ERR_ARG, "tkv_decode_attn_push: NULL pointer argument");
  if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world)
    return fail(TKV_ERR_ARG, "tkv_decode_attn_push: world=%d (limit %d) rank=%d", world, kMaxPeers, rank);
  if (out_row_stride < (int64_t)hq * head_dim || out_col_offset < 0 || out_col_offset + (int64_t)hq * head_dim > out_row_stride)
    return fail(TKV_ERR_ARG, "tkv_decode_attn_push: column block [%lld, +%d) does not fit rows of %lld elements",
                (long long)out_col_offset, hq * head_dim, (long long)out_row_stride);
  PushParams pp;
  for (int r = 0; r < kMaxPeers; ++r) { pp.peer_out[r] = nullptr; pp.peer_flags[r] = nullptr; }
  for (int r = 0; r < world; ++r) {
    if (!peer_out[r] || !peer_flags[r]) return fail(TKV_ERR_ARG, "tkv_decode_attn_push: NULL pointer for rank %d", r);
    pp.peer_out[r] = (char*)peer_out[r]; pp.peer_flags[r] = peer_flags[r];
  }
  pp.world = world; pp.rank = rank; pp.row_stride = out_row_stride; pp.col_offset = out_col_offset; pp.sync = sync_state;
  return decode_attn_impl("tkv_decode_attn_push", q, q_sb, q_sh, k_cache, v_cache, seg_len, seg_start, cap, out, workspace,
                          workspace_bytes, batch, hq, hkv, head_dim, kv_dtype, scale, max_len, -1, status, stream, &pp);
}

extern "C" int tkv_peer_wait(const int32_t* flags, int32_t* sync_state, int world, int rank, int max_polls,
                             int32_t* status, tkv_stream_t stream) {
  using namespace tkv;
  if (!flags || !sync_state) return fail(TKV_ERR_ARG, "tkv_peer_wait: NULL pointer argument");
  if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world)
    return fail(TKV_ERR_ARG, "tkv_peer_wait: world=%d rank=%d", world, rank);
  peer_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(flags, sync_state, world, rank, max_polls > 0 ? max_polls : (1 << 24), status);
  return check_launch("tkv_peer_wait");
}

// ---------------------------------------------------------------------------------------------------------
// Decode attention for callers that cannot allocate device memory.
//
// tkv_decode_attn needs a caller-provided workspace for the per-chunk partial results.  Some hosts have no way
// to provide one: an inference server that handed the whole device to its own block arena at start-up and has
// nothing left to carve a workspace from, a plug-in slot whose host does not expose its allocator, or a
// latency-critical loop where the implicit device-wide synchronisation of cudaMalloc/cudaFree is not acceptable.
// For them the partials live in the fixed array below, which is part of the library image: every GPU that
// loads the library holds these TKV_STATIC_SCRATCH_BYTES until the process exits.
//
// The array's name is only a host-side handle in host code; the kernels need its device address, which is
// looked up once per device with cudaGetSymbolAddress while that device is current.  The address is remembered per
// device ordinal for the life of the process: a host that calls cudaDeviceReset (or otherwise replaces the device's
// primary context) must not call this entry point afterwards, since the remembered address belongs to the old context.
static __device__ __align__(256) unsigned char g_attn_scratch[TKV_STATIC_SCRATCH_BYTES];

namespace tkv {
constexpr int kMaxDevices = 64;
static void* g_scratch_addr[kMaxDevices];   // device address of g_attn_scratch on each device (0 = not looked up)
}  // namespace tkv

extern "C" int tkv_decode_attn_static(const void* q, int64_t q_sb, int64_t q_sh,
                                      const void* k_cache, const void* v_cache,
                                      const int32_t* seg_len, const int32_t* seg_start, int64_t cap,
                                      void* out, int batch, int hq, int hkv, int head_dim, int kv_dtype,
                                      float scale, int max_len, int32_t* status, tkv_stream_t stream) {
  using namespace tkv;
  if (!q || !k_cache || !v_cache || !seg_len || !out)
    return fail(TKV_ERR_ARG, "tkv_decode_attn_static: NULL pointer argument");
  if (batch < 0 || hq <= 0 || hkv <= 0 || hq % hkv != 0 || head_dim <= 0 || max_len <= 0)
    return fail(TKV_ERR_ARG, "tkv_decode_attn_static: bad sizes batch=%d hq=%d hkv=%d head_dim=%d max_len=%d", batch,
                hq, hkv, head_dim, max_len);
  if (seg_start == nullptr && cap <= 0)
    return fail(TKV_ERR_ARG, "tkv_decode_attn_static: cap=%lld without seg_start", (long long)cap);
  if (!aligned16(q) || !aligned16(k_cache) || !aligned16(v_cache) || !aligned16(out))
    return fail(TKV_ERR_ARG, "tkv_decode_attn_static: pointers must be 16-byte aligned");
  if ((q_sb * 2) % 16 || (q_sh * 2) % 16)
    return fail(TKV_ERR_ARG, "tkv_decode_attn_static: q strides must be multiples of 16 bytes");
  if (batch == 0) return TKV_OK;
  // This entry point always runs the CUDA-core split kernel, so the scratch is sized by that kernel's chunk length
  // alone (tkv_decode_attn_workspace_bytes also covers the tensor-core kernel's shorter chunks).
  const int static_chunk = attn_chunk_tokens(batch * hkv, max_len);
  const size_t need = (size_t)((int64_t)batch * hkv * ((max_len + static_chunk - 1) / static_chunk) * (hq / hkv) *
                               (head_dim + 2) * sizeof(float) + 256);
  if (need > (size_t)TKV_STATIC_SCRATCH_BYTES)
    return fail(TKV_ERR_UNSUPPORTED,
                "tkv_decode_attn_static: this problem needs %zu bytes of scratch but the built-in array holds %zu; "
                "use tkv_decode_attn with a caller-provided workspace", need, (size_t)TKV_STATIC_SCRATCH_BYTES);
  // Set-up on the first call per device: resolve the device address of the array (no allocation happens).
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(TKV_ERR_LAUNCH, "tkv_decode_attn_static: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(TKV_ERR_UNSUPPORTED, "tkv_decode_attn_static: device %d", dev);
  void* scratch = __atomic_load_n(&g_scratch_addr[dev], __ATOMIC_ACQUIRE);
  if (scratch == nullptr) {
    e = cudaGetSymbolAddress(&scratch, g_attn_scratch);
    if (e != cudaSuccess || scratch == nullptr)
      return fail(TKV_ERR_LAUNCH, "tkv_decode_attn_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    __atomic_store_n(&g_scratch_addr[dev], scratch, __ATOMIC_RELEASE);  // same value from every thread
  }
  const int nseg = batch * hkv, G = hq / hkv;
  AttnParams p;
  p.q = (const char*)q; p.q_sb = q_sb; p.q_sh = q_sh;
  p.k = (const char*)k_cache; p.v = (const char*)v_cache;
  p.seg_len = seg_len; p.seg_start = seg_start; p.cap = cap;
  p.out = (char*)out;
  p.chunk = attn_chunk_tokens(nseg, max_len);
  p.nchunks = (max_len + p.chunk - 1) / p.chunk;
  // Nothing in the scratch has to start at zero: the merge step reads only the partials of the chunks that the
  // first step of this same call has written.
  p.part_ml = reinterpret_cast<float*>(scratch);
  p.part_o = p.part_ml + (((int64_t)nseg * p.nchunks * G * 2 + 63) / 64) * 64;
  p.hq = hq; p.hkv = hkv; p.max_len = max_len;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  p.work = nullptr; p.work_count = nullptr; p.work_capacity = 0;
  p.q_tokens = 1; p.rows = G; p.q_st = 0;
  return launch_decode_attn_simt(p, nseg, G, head_dim, kv_dtype, (cudaStream_t)stream);
}
