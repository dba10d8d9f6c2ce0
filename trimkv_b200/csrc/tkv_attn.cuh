// Parameters shared by the decode-attention kernels.
#pragma once
#include <stdint.h>
#include <cuda_runtime.h>

namespace tkv {

struct AttnParams {
  const char* q; int64_t q_sb, q_sh;      // element strides of q[b, head, :]
  const char* k; const char* v;
  const int32_t* seg_len; const int32_t* seg_start; int64_t cap;
  char* out;                              // [batch, hq, D]
  float* part_ml;                         // [nseg, nchunks, G, 2]  (max, sum) in log2 domain
  float* part_o;                          // [nseg, nchunks, G, D]  unnormalised partial outputs
  int chunk, nchunks;
  int hq, hkv, max_len;
  float scale_log2;                       // softmax scale * log2(e)
  int32_t* status;
  // Optional compact work list (ragged lengths): item i = {segment << 8 | chunk, clamped length of the segment};
  // *work_count items are valid.  NULL: the grid covers every (segment, chunk) pair and absent chunks exit.
  const int2* work; const int32_t* work_count; int work_capacity;
};

// Tokens per work item, a pure function of the problem size (the workspace size depends on it).
int attn_chunk_tokens(int nseg, int max_len);


// Tensor-core (tcgen05 + TMA) split kernel: fixed chunk, needs the capacity-strided layout and head_dim 128.
int attn_tc_chunk_tokens();
int launch_decode_attn_tc(const AttnParams& p, int nseg, int G, int kv_dtype, int64_t rows, cudaStream_t st);
// Builds the compact work list of the tensor-core split kernel from the lengths (one small kernel).
int launch_attn_worklist(const AttnParams& p, int nseg, cudaStream_t st);
// Merge kernel shared by both split kernels.
int launch_decode_attn_combine(const AttnParams& p, int nseg, int G, int head_dim, int kv_dtype, cudaStream_t st);

}  // namespace tkv
