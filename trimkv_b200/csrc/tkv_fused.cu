// Fused producer-side kernels of one decode step (one new token per request).
//
// The reference runs the producer of the cache path as ~50 small PyTorch kernels per layer
// (src/trimkv/models/qwen3/modeling_trimkv_qwen3.py:328-353: q_norm/k_norm, retention gate tail, RoPE,
// transposes, then cache.update).  Here:
//   decode_prep_kernel : q/k RMSNorm (where the family has one) + RoPE, retention-gate tail (SiLU -> linear2 -> +bias -> logsigmoid),
//                        and the append of K, V, log beta, position into the flat cache, one launch;
//   add_rmsnorm_kernel : residual += delta, out = RMSNorm(residual) * weight;
//   silu_mul_kernel    : SiLU(gate) * up of the MLP.
// Every intermediate is rounded to the model dtype exactly where the eager PyTorch sequence rounds
// (one rounding per PyTorch op), so the results track the reference's bf16 pipeline.
#include "tkv_common.cuh"

namespace tkv {

template <int kDtype> struct T16;
template <> struct T16<TKV_BF16> {
  static __device__ __forceinline__ float lo(uint32_t w) { return __uint_as_float(w << 16); }
  static __device__ __forceinline__ float hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
  static __device__ __forceinline__ float round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ float ld(const void* p, int64_t i) {
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  }
};
template <> struct T16<TKV_F16> {
  static __device__ __forceinline__ float lo(uint32_t w) { return __half2float(__ushort_as_half((unsigned short)(w & 0xffff))); }
  static __device__ __forceinline__ float hi(uint32_t w) { return __half2float(__ushort_as_half((unsigned short)(w >> 16))); }
  static __device__ __forceinline__ float round(float x) { return __half2float(__float2half_rn(x)); }
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ float ld(const void* p, int64_t i) {
    return __half2float(reinterpret_cast<const __half*>(p)[i]);
  }
};

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

// A GEMM result can arrive either in the model dtype or as `splits` fp32 partial sums [splits][rows][cols] of
// tkv_skinny_gemm; in the second form the consumer adds the partials in order, adds the bias and rounds once, which
// is what a GEMM with fp32 accumulation and a rounded output does.
template <typename T>
__device__ __forceinline__ float gemm_out(const void* base, int splits, int64_t split_stride, const void* bias,
                                          int64_t idx, int col) {
  if (splits == 0) return T::ld(base, idx);
  const float* part = reinterpret_cast<const float*>(base);
  float a = part[idx];
  for (int s = 1; s < splits; ++s) a += part[idx + s * split_stride];
  if (bias != nullptr) a += T::ld(bias, col);
  return T::round(a);
}
template <typename T>
__device__ __forceinline__ void gemm_out4(const void* base, int splits, int64_t split_stride, const void* bias,
                                          int64_t idx, int col, float* out) {
  if (splits == 0) {
    const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const char*>(base) + idx * 2);
    out[0] = T::lo(raw.x); out[1] = T::hi(raw.x); out[2] = T::lo(raw.y); out[3] = T::hi(raw.y);
    return;
  }
  const float* part = reinterpret_cast<const float*>(base);
  float4 a = *reinterpret_cast<const float4*>(part + idx);
  for (int s = 1; s < splits; ++s) {
    const float4 b = *reinterpret_cast<const float4*>(part + idx + s * split_stride);
    a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
  }
  if (bias != nullptr) { a.x += T::ld(bias, col); a.y += T::ld(bias, col + 1); a.z += T::ld(bias, col + 2); a.w += T::ld(bias, col + 3); }
  out[0] = T::round(a.x); out[1] = T::round(a.y); out[2] = T::round(a.z); out[3] = T::round(a.w);
}

struct PrepParams {
  const void* qkvg; int64_t row_elems;       // [B, (Hq + 2 Hkv) * 128 + gate_inter], or fp32 partials of it
  int in_splits; int64_t split_stride; const void* in_bias;
  const void* q_norm_w; const void* k_norm_w; float eps;
  const void* cos; const void* sin;          // [128] of the model dtype
  const void* gate_w2; const void* gate_bias; int gate_inter;
  const int64_t* pos;
  char* q_out;                               // [B, Hq, 128]
  char* k_cache; char* v_cache; float* beta_cache; int32_t* pos_cache;
  int32_t* seg_len; int32_t* cu_seqlens; int64_t cap;
  int batch, hq, hkv;
  int32_t* status;
};

constexpr int kPrepWarps = 4;

// One warp per (request, head); head < hq: a query head, else KV head (head - hq).  D = 128: lane l owns
// elements 4l..4l+3; RoPE pairs element i with i +- 64, i.e. lane l with lane l ^ 16.
template <int kDtype>
__global__ void __launch_bounds__(kPrepWarps * 32) decode_prep_kernel(PrepParams p) {
  using T = T16<kDtype>;
  const int lane = threadIdx.x & 31;
  const int w = blockIdx.x * kPrepWarps + (threadIdx.x >> 5);
  const int heads = p.hq + p.hkv;
  if (w >= p.batch * heads) return;
  grid_dependency_wait();
  grid_launch_dependents();  // the attention kernel may be scheduled early; it waits for this grid before reading
  const int b = w / heads, head = w - b * heads;
  const bool is_q = head < p.hq;
  const int kvh = head - p.hq;
  const int64_t row = (int64_t)b * p.row_elems;          // element offset of this request's row
  const int col = (is_q ? head : p.hq + kvh) * 128 + lane * 4;
  float x[4];
  gemm_out4<T>(p.qkvg, p.in_splits, p.split_stride, p.in_bias, row + col, col, x);
  // A KV-head warp requests everything else it will need right away (the segment's length, its V row, its share of
  // the gate's hidden layer and second-layer weights), so that the memory round trips overlap instead of adding up.
  constexpr int kGatePre = 4;                              // hidden values per lane held in registers (gate_inter <= 128)
  const int seg = b * p.hkv + kvh;
  const int gcol = (p.hq + 2 * p.hkv) * 128;
  int len = 0;
  float vv[4] = {0.f, 0.f, 0.f, 0.f}, gate_h[kGatePre], gate_w[kGatePre];
  if (!is_q) {
    len = p.seg_len[seg];
    const int vcol = (p.hq + p.hkv + kvh) * 128 + lane * 4;
    gemm_out4<T>(p.qkvg, p.in_splits, p.split_stride, p.in_bias, row + vcol, vcol, vv);
#pragma unroll
    for (int j = 0; j < kGatePre; ++j) {
      const int i = lane + 32 * j;
      gate_h[j] = 0.f; gate_w[j] = 0.f;
      if (i < p.gate_inter) {
        gate_h[j] = gemm_out<T>(p.qkvg, p.in_splits, p.split_stride, p.in_bias, row + gcol + i, gcol + i);
        gate_w[j] = T::ld(p.gate_w2, (int64_t)kvh * p.gate_inter + i);
      }
    }
  }
  // RMSNorm over the head: fp32 statistics, normalised value rounded, then multiplied by the weight.  Families
  // without a per-head norm (Llama, Phi-3) pass no weights and the projection goes to RoPE as it is.
  const void* nw = is_q ? p.q_norm_w : p.k_norm_w;
  float y[4], rot[4], o[4];
  if (nw != nullptr) {
    const float ss = warp_sum(x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3]);
    const float rstd = rsqrtf(ss * (1.0f / 128.0f) + p.eps);
#pragma unroll
    for (int i = 0; i < 4; ++i) y[i] = T::round(T::ld(nw, lane * 4 + i) * T::round(x[i] * rstd));
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) y[i] = x[i];
  }
  // RoPE: out = round(round(y * cos) + round(rotate_half(y) * sin)).
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float partner = __shfl_xor_sync(0xffffffffu, y[i], 16);
    rot[i] = lane < 16 ? -partner : partner;
    const float c = T::ld(p.cos, lane * 4 + i), s = T::ld(p.sin, lane * 4 + i);
    o[i] = T::round(T::round(y[i] * c) + T::round(rot[i] * s));
  }
  const uint2 packed = make_uint2(T::pack(o[0], o[1]), T::pack(o[2], o[3]));
  if (is_q) {
    *reinterpret_cast<uint2*>(p.q_out + ((int64_t)b * p.hq + head) * 256 + lane * 8) = packed;
    return;
  }
  // KV head: append K (normalised + rotated), V (as is), log beta and the position.
  __syncwarp();
  // Retention gate tail: log beta = logsigmoid(linear2(SiLU(hidden)) + bias), rounded after every op.
  float acc = 0.f;
#pragma unroll
  for (int j = 0; j < kGatePre; ++j) {
    if (lane + 32 * j < p.gate_inter) {
      const float act = T::round(gate_h[j] / (1.0f + expf(-gate_h[j])));
      acc = fmaf(act, gate_w[j], acc);
    }
  }
  for (int i = lane + 32 * kGatePre; i < p.gate_inter; i += 32) {
    const float g = gemm_out<T>(p.qkvg, p.in_splits, p.split_stride, p.in_bias, row + gcol + i, gcol + i);
    const float act = T::round(g / (1.0f + expf(-g)));
    acc = fmaf(act, T::ld(p.gate_w2, (int64_t)kvh * p.gate_inter + i), acc);
  }
  acc = warp_sum(acc);
  const float z = T::round(T::round(acc) + T::ld(p.gate_bias, kvh));
  const float log_beta = T::round(fminf(z, 0.f) - log1pf(expf(-fabsf(z))));
  if (len < 0 || (int64_t)len + 1 > p.cap) {
    if (lane == 0) report(p.status, TKV_DEV_CAPACITY);
    return;
  }
  const int64_t dst = (int64_t)seg * p.cap + len;
  *reinterpret_cast<uint2*>(p.k_cache + dst * 256 + lane * 8) = packed;
  *reinterpret_cast<uint2*>(p.v_cache + dst * 256 + lane * 8) = make_uint2(T::pack(vv[0], vv[1]), T::pack(vv[2], vv[3]));
  if (lane == 0) {
    p.beta_cache[dst] = log_beta;
    p.pos_cache[dst] = (int32_t)p.pos[0];
    p.seg_len[seg] = len + 1;
    if (p.cu_seqlens != nullptr) p.cu_seqlens[seg + 1] += seg + 1;
  }
}

// residual[r] += delta[r] (if delta), out[r] = weight * round(residual[r] * rstd).  One CTA per row.
template <int kDtype>
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(char* residual, const char* delta, const void* weight,
                                                          char* out, int cols, float eps, int in_splits,
                                                          int64_t split_stride, const void* in_bias) {
  using T = T16<kDtype>;
  __shared__ float red[8];
  const int64_t off = (int64_t)blockIdx.x * cols * 2;
  const int nvec = cols / 8;  // 16-byte vectors per row
  float ss = 0.f;
  // Rows of up to 256 * kKeep vectors (hidden size 8192) stay in registers between the two passes.  The norm weights
  // do not depend on the preceding kernel, so they are requested before the dependency wait and arrive under it.
  constexpr int kKeep = 4;
  const bool in_regs = nvec <= 256 * kKeep;
  uint4 keep[kKeep], wkeep[kKeep];
  if (in_regs) {
#pragma unroll
    for (int j = 0; j < kKeep; ++j) {
      const int i = threadIdx.x + j * 256;
      if (i < nvec) wkeep[j] = ld16(reinterpret_cast<const char*>(weight) + (int64_t)i * 16);
    }
  }
  grid_dependency_wait();
  grid_launch_dependents();  // a following weight-streaming GEMM may start fetching weights; it waits before reading `out`
  // Pass 1: update the residual stream and accumulate the sum of squares.
  for (int i = threadIdx.x, j = 0; i < nvec; i += 256, ++j) {
    uint4 r = ld16(residual + off + (int64_t)i * 16);
    if (delta != nullptr && in_splits > 0) {
      float d[8];
      const int64_t e0 = (int64_t)blockIdx.x * cols + (int64_t)i * 8;
      gemm_out4<T>(delta, in_splits, split_stride, in_bias, e0, i * 8, d);
      gemm_out4<T>(delta, in_splits, split_stride, in_bias, e0 + 4, i * 8 + 4, d + 4);
      r.x = T::pack(T::lo(r.x) + d[0], T::hi(r.x) + d[1]);
      r.y = T::pack(T::lo(r.y) + d[2], T::hi(r.y) + d[3]);
      r.z = T::pack(T::lo(r.z) + d[4], T::hi(r.z) + d[5]);
      r.w = T::pack(T::lo(r.w) + d[6], T::hi(r.w) + d[7]);
      st16(residual + off + (int64_t)i * 16, r);
    } else if (delta != nullptr) {
      const uint4 d = ld16(delta + off + (int64_t)i * 16);
      r.x = T::pack(T::lo(r.x) + T::lo(d.x), T::hi(r.x) + T::hi(d.x));
      r.y = T::pack(T::lo(r.y) + T::lo(d.y), T::hi(r.y) + T::hi(d.y));
      r.z = T::pack(T::lo(r.z) + T::lo(d.z), T::hi(r.z) + T::hi(d.z));
      r.w = T::pack(T::lo(r.w) + T::lo(d.w), T::hi(r.w) + T::hi(d.w));
      st16(residual + off + (int64_t)i * 16, r);
    }
    const uint32_t ws[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) { const float a = T::lo(ws[q]), c = T::hi(ws[q]); ss += a * a + c * c; }
    if (in_regs) {
#pragma unroll
      for (int q = 0; q < kKeep; ++q) if (q == j) keep[q] = r;
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += red[i];
  const float rstd = rsqrtf(tot / (float)cols + eps);
  // Pass 2: from the registers, or (longer rows) from L1/L2 where this CTA has just written the row.
  for (int i = threadIdx.x, j = 0; i < nvec; i += 256, ++j) {
    uint4 r, wv;
    if (in_regs) {
#pragma unroll
      for (int q = 0; q < kKeep; ++q) if (q == j) { r = keep[q]; wv = wkeep[q]; }
    } else {
      r = ld16(residual + off + (int64_t)i * 16);
      wv = ld16(reinterpret_cast<const char*>(weight) + (int64_t)i * 16);
    }
    uint4 o;
    o.x = T::pack(T::lo(wv.x) * T::round(T::lo(r.x) * rstd), T::hi(wv.x) * T::round(T::hi(r.x) * rstd));
    o.y = T::pack(T::lo(wv.y) * T::round(T::lo(r.y) * rstd), T::hi(wv.y) * T::round(T::hi(r.y) * rstd));
    o.z = T::pack(T::lo(wv.z) * T::round(T::lo(r.z) * rstd), T::hi(wv.z) * T::round(T::hi(r.z) * rstd));
    o.w = T::pack(T::lo(wv.w) * T::round(T::lo(r.w) * rstd), T::hi(wv.w) * T::round(T::hi(r.w) * rstd));
    st16(out + off + (int64_t)i * 16, o);
  }
}

// out[r, j] = round(round(SiLU(gu[r, j])) * gu[r, inter + j]).
template <int kDtype>
__global__ void __launch_bounds__(256) silu_mul_kernel(const char* gu, char* out, int rows, int inter, int in_splits,
                                                       int64_t split_stride, const void* in_bias) {
  using T = T16<kDtype>;
  const int nvec = inter / 8;
  const int64_t total = (int64_t)rows * nvec;
  grid_dependency_wait();
  grid_launch_dependents();  // as in add_rmsnorm_kernel
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (int64_t)gridDim.x * 256) {
    const int64_t r = i / nvec, c = i - r * nvec;
    auto f = [](float gg, float uu) {
      const float act = T::round(gg / (1.0f + expf(-gg)));
      return act * uu;
    };
    uint4 o;
    if (in_splits > 0) {
      float g8[8], u8[8];
      const int64_t e0 = r * 2 * inter + c * 8;
      gemm_out4<T>(gu, in_splits, split_stride, in_bias, e0, (int)(c * 8), g8);
      gemm_out4<T>(gu, in_splits, split_stride, in_bias, e0 + 4, (int)(c * 8 + 4), g8 + 4);
      gemm_out4<T>(gu, in_splits, split_stride, in_bias, e0 + inter, (int)(inter + c * 8), u8);
      gemm_out4<T>(gu, in_splits, split_stride, in_bias, e0 + inter + 4, (int)(inter + c * 8 + 4), u8 + 4);
      o.x = T::pack(f(g8[0], u8[0]), f(g8[1], u8[1])); o.y = T::pack(f(g8[2], u8[2]), f(g8[3], u8[3]));
      o.z = T::pack(f(g8[4], u8[4]), f(g8[5], u8[5])); o.w = T::pack(f(g8[6], u8[6]), f(g8[7], u8[7]));
      st16(out + (r * inter) * 2 + c * 16, o);
      continue;
    }
    const uint4 g = ld16(gu + (r * 2 * inter) * 2 + c * 16);
    const uint4 u = ld16(gu + (r * 2 * inter + inter) * 2 + c * 16);
    o.x = T::pack(f(T::lo(g.x), T::lo(u.x)), f(T::hi(g.x), T::hi(u.x)));
    o.y = T::pack(f(T::lo(g.y), T::lo(u.y)), f(T::hi(g.y), T::hi(u.y)));
    o.z = T::pack(f(T::lo(g.z), T::lo(u.z)), f(T::hi(g.z), T::hi(u.z)));
    o.w = T::pack(f(T::lo(g.w), T::lo(u.w)), f(T::hi(g.w), T::hi(u.w)));
    st16(out + (r * inter) * 2 + c * 16, o);
  }
}

}  // namespace tkv

extern "C" int tkv_decode_prep(const void* qkvg, int64_t row_stride,
                               const void* q_norm_w, const void* k_norm_w, float eps,
                               const void* cos, const void* sin,
                               const void* gate_w2, const void* gate_bias, int gate_inter,
                               const int64_t* pos, void* q_out,
                               void* k_cache, void* v_cache, float* beta_cache, int32_t* pos_cache,
                               int32_t* seg_len, int32_t* cu_seqlens, int64_t cap,
                               int batch, int hq, int hkv, int head_dim, int dtype,
                               int in_splits, const void* in_bias,
                               int32_t* status, tkv_stream_t stream) {
  using namespace tkv;
  if ((q_norm_w == nullptr) != (k_norm_w == nullptr))
    return fail(TKV_ERR_ARG, "tkv_decode_prep: q_norm_w and k_norm_w must both be given or both be NULL");
  if (!qkvg || !cos || !sin || !gate_w2 || !gate_bias || !pos || !q_out || !k_cache ||
      !v_cache || !beta_cache || !pos_cache || !seg_len)
    return fail(TKV_ERR_ARG, "tkv_decode_prep: NULL pointer argument");
  if (head_dim != 128) return fail(TKV_ERR_UNSUPPORTED, "tkv_decode_prep: head_dim=%d (only 128)", head_dim);
  if (dtype != TKV_BF16 && dtype != TKV_F16) return fail(TKV_ERR_UNSUPPORTED, "tkv_decode_prep: dtype %d", dtype);
  if (batch < 0 || hq <= 0 || hkv <= 0 || gate_inter <= 0 || cap <= 0) return fail(TKV_ERR_ARG, "tkv_decode_prep: bad sizes");
  if (row_stride < (int64_t)(hq + 2 * hkv) * 128 + gate_inter || (row_stride * 2) % 8 || in_splits < 0)
    return fail(TKV_ERR_ARG, "tkv_decode_prep: row_stride=%lld too small or misaligned", (long long)row_stride);
  if (in_splits > 0 && (row_stride % 4 || (reinterpret_cast<uintptr_t>(qkvg) & 15u)))
    return fail(TKV_ERR_ARG, "tkv_decode_prep: fp32 partial input must be 16-byte aligned with row_stride %% 4 == 0");
  if ((reinterpret_cast<uintptr_t>(qkvg) | reinterpret_cast<uintptr_t>(q_out) | reinterpret_cast<uintptr_t>(k_cache) |
       reinterpret_cast<uintptr_t>(v_cache)) & 7u)
    return fail(TKV_ERR_ARG, "tkv_decode_prep: pointers must be 8-byte aligned");
  if (batch == 0) return TKV_OK;
  PrepParams p;
  p.qkvg = qkvg; p.row_elems = row_stride;
  p.in_splits = in_splits; p.split_stride = (int64_t)batch * row_stride; p.in_bias = in_bias;
  p.q_norm_w = q_norm_w; p.k_norm_w = k_norm_w; p.eps = eps; p.cos = cos; p.sin = sin;
  p.gate_w2 = gate_w2; p.gate_bias = gate_bias; p.gate_inter = gate_inter; p.pos = pos;
  p.q_out = (char*)q_out; p.k_cache = (char*)k_cache; p.v_cache = (char*)v_cache;
  p.beta_cache = beta_cache; p.pos_cache = pos_cache; p.seg_len = seg_len; p.cu_seqlens = cu_seqlens; p.cap = cap;
  p.batch = batch; p.hq = hq; p.hkv = hkv; p.status = status;
  const int warps = batch * (hq + hkv);
  const int grid = (warps + kPrepWarps - 1) / kPrepWarps;
  cudaError_t e = dtype == TKV_BF16
      ? launch_pdl(decode_prep_kernel<TKV_BF16>, dim3(grid), dim3(kPrepWarps * 32), 0, (cudaStream_t)stream, p)
      : launch_pdl(decode_prep_kernel<TKV_F16>, dim3(grid), dim3(kPrepWarps * 32), 0, (cudaStream_t)stream, p);
  if (e != cudaSuccess) return fail(TKV_ERR_LAUNCH, "tkv_decode_prep: %s", cudaGetErrorString(e));
  return check_launch("tkv_decode_prep");
}

extern "C" int tkv_add_rmsnorm(void* residual, const void* delta, const void* weight, void* out,
                               int rows, int cols, float eps, int dtype, int in_splits, const void* in_bias,
                               tkv_stream_t stream) {
  using namespace tkv;
  if (!residual || !weight || !out) return fail(TKV_ERR_ARG, "tkv_add_rmsnorm: NULL pointer argument");
  if (dtype != TKV_BF16 && dtype != TKV_F16) return fail(TKV_ERR_UNSUPPORTED, "tkv_add_rmsnorm: dtype %d", dtype);
  if (rows < 0 || cols <= 0 || cols % 8) return fail(TKV_ERR_ARG, "tkv_add_rmsnorm: cols=%d must be a positive multiple of 8", cols);
  if (!aligned16(residual) || !aligned16(weight) || !aligned16(out) || (delta && !aligned16(delta)))
    return fail(TKV_ERR_ARG, "tkv_add_rmsnorm: pointers must be 16-byte aligned");
  if (rows == 0) return TKV_OK;
  cudaError_t e = dtype == TKV_BF16
      ? launch_pdl(add_rmsnorm_kernel<TKV_BF16>, dim3(rows), dim3(256), 0, (cudaStream_t)stream, (char*)residual,
                   (const char*)delta, weight, (char*)out, cols, eps, in_splits, (int64_t)rows * cols, in_bias)
      : launch_pdl(add_rmsnorm_kernel<TKV_F16>, dim3(rows), dim3(256), 0, (cudaStream_t)stream, (char*)residual,
                   (const char*)delta, weight, (char*)out, cols, eps, in_splits, (int64_t)rows * cols, in_bias);
  if (e != cudaSuccess) return fail(TKV_ERR_LAUNCH, "tkv_add_rmsnorm: %s", cudaGetErrorString(e));
  return check_launch("tkv_add_rmsnorm");
}

extern "C" int tkv_silu_mul(const void* gate_up, void* out, int rows, int inter, int dtype, int in_splits,
                            const void* in_bias, tkv_stream_t stream) {
  using namespace tkv;
  if (!gate_up || !out) return fail(TKV_ERR_ARG, "tkv_silu_mul: NULL pointer argument");
  if (dtype != TKV_BF16 && dtype != TKV_F16) return fail(TKV_ERR_UNSUPPORTED, "tkv_silu_mul: dtype %d", dtype);
  if (rows < 0 || inter <= 0 || inter % 8) return fail(TKV_ERR_ARG, "tkv_silu_mul: inter=%d must be a positive multiple of 8", inter);
  if (!aligned16(gate_up) || !aligned16(out)) return fail(TKV_ERR_ARG, "tkv_silu_mul: pointers must be 16-byte aligned");
  if (rows == 0) return TKV_OK;
  const int64_t total = (int64_t)rows * (inter / 8);
  const int grid = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  cudaError_t e = dtype == TKV_BF16
      ? launch_pdl(silu_mul_kernel<TKV_BF16>, dim3(grid), dim3(256), 0, (cudaStream_t)stream, (const char*)gate_up, (char*)out,
                   rows, inter, in_splits, (int64_t)rows * 2 * inter, in_bias)
      : launch_pdl(silu_mul_kernel<TKV_F16>, dim3(grid), dim3(256), 0, (cudaStream_t)stream, (const char*)gate_up, (char*)out,
                   rows, inter, in_splits, (int64_t)rows * 2 * inter, in_bias);
  if (e != cudaSuccess) return fail(TKV_ERR_LAUNCH, "tkv_silu_mul: %s", cudaGetErrorString(e));
  return check_launch("tkv_silu_mul");
}
