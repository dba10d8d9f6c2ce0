// Shared helpers of the trimkv_b200 kernels (sm_100a).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include "../../include/trimkv_b200.h"

namespace tkv {

// Records a host-side error message for tkv_last_error() and returns `code`.
int fail(int code, const char* fmt, ...);
// Checks cudaGetLastError() after a launch.
int check_launch(const char* what);

inline int elem_size(int dtype) {
  return dtype == TKV_F32 ? 4 : (dtype == TKV_BF16 || dtype == TKV_F16) ? 2 : 0;
}
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

__device__ __forceinline__ void report(int32_t* status, int code) {
  if (status != nullptr) atomicMax(status, code);
}

// Order-preserving map fp32 -> uint32 with the selection's conventions:
// larger score = larger key, -0.0 and +0.0 share a key, NaN is the largest key.
__device__ __forceinline__ uint32_t score_key(float s) {
  if (s != s) return 0xFFFFFFFFu;
  s = s + 0.0f;  // -0.0 -> +0.0
  uint32_t u = __float_as_uint(s);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// score = f32(log beta) * f32(q_idx - pos): exactly one rounding, never contracted.
__device__ __forceinline__ float retention_score(float log_beta, int32_t pos, int64_t q_idx) {
  return __fmul_rn(log_beta, __ll2float_rn(q_idx - (int64_t)pos));
}

// The flat budget-sharing caches of the reference multiply in the dtype the gate output is stored in
// (src/trimkv/cache_utils.py:386,441,755: `(q_idx - kv_pos) * rw` with rw in the model dtype): torch casts the
// int64 age to that dtype, multiplies in fp32 and rounds the product to it.  score_dtype: 0 = fp32 (one rounding,
// as TrimKVCache does after its explicit upcast), 1 = bf16, 2 = f16.  log_beta holds the stored value exactly.
__device__ __forceinline__ float retention_score_as(float log_beta, int32_t pos, int64_t q_idx, int score_dtype) {
  const float age = __ll2float_rn(q_idx - (int64_t)pos);
  if (score_dtype == 1) return __bfloat162float(__float2bfloat16_rn(__fmul_rn(log_beta, __bfloat162float(__float2bfloat16_rn(age)))));
  if (score_dtype == 2) return __half2float(__float2half_rn(__fmul_rn(log_beta, __half2float(__float2half_rn(age)))));
  return __fmul_rn(log_beta, age);
}

__device__ __forceinline__ uint4 ld16(const void* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ void st16(void* p, uint4 v) { *reinterpret_cast<uint4*>(p) = v; }

// Streaming (evict-first) 16-byte accesses for data that is touched once.
__device__ __forceinline__ uint4 ld16_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// Programmatic dependent launch: a kernel launched with launch_pdl() may be scheduled while its predecessor in
// the stream is still draining; it must call grid_dependency_wait() before touching anything the predecessor wrote.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Lets the next kernel of the stream (if launched with launch_pdl) be scheduled now; its own grid_dependency_wait()
// still holds it until this whole grid has finished and its writes are visible, so only its launch latency overlaps.
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

template <int kThreads>
__device__ __forceinline__ int block_exclusive_scan(int v, int* warp_sums /* [kThreads/32 + 1] */, int* total) {
  // Inclusive warp scan, then scan of the warp totals by warp 0.
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int x = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int y = __shfl_up_sync(0xffffffffu, x, o);
    if (lane >= o) x += y;
  }
  if (lane == 31) warp_sums[warp] = x;
  __syncthreads();
  if (warp == 0) {
    constexpr int kWarps = kThreads / 32;
    int w = lane < kWarps ? warp_sums[lane] : 0;
    int s = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int y = __shfl_up_sync(0xffffffffu, s, o);
      if (lane >= o) s += y;
    }
    if (lane < kWarps) warp_sums[lane] = s - w;  // exclusive
    if (lane == kWarps - 1) warp_sums[kWarps] = s;
  }
  __syncthreads();
  int excl = warp_sums[warp] + x - v;
  *total = warp_sums[kThreads / 32];
  __syncthreads();  // warp_sums may be reused by the caller right away
  return excl;
}

}  // namespace tkv
