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
  // Several query tokens per request (q_tokens > 1; tensor-core path only): a segment then has rows = q_tokens * G
  // query rows, row R = token i * G + head g, and token i sees the first len - q_tokens + i + 1 cached tokens
  // (bottom-right aligned causal mask).  q is [batch, q_tokens, hq, D] with token stride q_st (elements), out
  // [batch, q_tokens, hq, D] contiguous, partials are [nseg, nchunks, rows, ...].  rows == G for plain decode.
  int q_tokens, rows; int64_t q_st;
};

// Head-sharded decode: the merge kernel stores this rank's heads straight into every rank's gathered buffer (plain
// stores to peer memory over NVLink) and the last CTA raises a flag on every peer.
constexpr int kMaxPeers = 8;
struct PushParams {
  char* peer_out[kMaxPeers];        // [batch, row_stride] of K/V dtype on every rank (own rank included)
  int32_t* peer_flags[kMaxPeers];   // [world] int32 on every rank; entry `rank` is written by this rank
  int world, rank;
  int64_t row_stride;               // elements between consecutive requests in peer_out
  int64_t col_offset;               // element offset of this rank's first head in a row
  int32_t* sync;                    // device, this rank: [0] CTA counter, [1] exchanges sent, [2] exchanges received
};

// Tokens per work item, a pure function of the problem size (the workspace size depends on it).
int attn_chunk_tokens(int nseg, int max_len);


// Tensor-core (tcgen05 + TMA) split kernel: fixed chunk, needs the capacity-strided layout and head_dim 128.
int attn_tc_chunk_tokens();
int launch_decode_attn_tc(const AttnParams& p, int nseg, int G, int kv_dtype, int64_t rows, cudaStream_t st);
// Several query tokens with more than 16 query rows per segment: 32 rows per CTA (tkv_attn_multi.cu).
int launch_multi_attn_tc(const AttnParams& p, int nseg, int kv_dtype, int64_t rows, cudaStream_t st);
// Builds the compact work list of the tensor-core split kernel from the lengths (one small kernel).
int launch_attn_worklist(const AttnParams& p, int nseg, cudaStream_t st);
// Merge kernel shared by both split kernels.
int launch_decode_attn_combine(const AttnParams& p, int nseg, int G, int head_dim, int kv_dtype, cudaStream_t st,
                               const PushParams* push = nullptr);

}  // namespace tkv
