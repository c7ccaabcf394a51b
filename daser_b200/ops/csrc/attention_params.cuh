// Shared between the paged-attention kernels: launch parameters and small PTX helpers.
#pragma once
#include "common.cuh"
#include "kv_paged.h"

namespace daser {

constexpr int ATT_D = 128;          // head dim
constexpr int ATT_B = 16;           // tokens per page
constexpr int ATT_STAGES = 4;       // cp.async ring depth per warp
constexpr int ATT_WARPS = 4;
constexpr int ATT_STAGE_BYTES = 2 * ATT_B * ATT_D + 2 * ATT_B * (ATT_D / 16) * 4;  // K, V payload + K, V scales = 5120

struct AttnParams {
  const __nv_bfloat16* q;    // [Tq, Hq, D]
  __nv_bfloat16* out;        // [Tq, Hq, D]
  float* part_o;             // [Tq, Hq, nsplit, D]  (nsplit > 1)
  float* part_lse;           // [Tq, Hq, nsplit]
  const uint8_t* kv_payload; // layer base of the fp8 pool
  const float* kv_scales;
  int64_t stride_block, stride_kv, stride_head, stride_tok;  // payload strides (elements = bytes)
  const int32_t* block_tables;  // [num_seqs, max_blocks]
  int max_blocks;
  const int32_t* q_start;    // [num_seqs + 1] prefix sums of query lengths
  const int32_t* ctx_lens;   // [num_seqs] total length including the new tokens
  int num_seqs, Hq, Hkv, G;
  int nsplit, split_tokens, row_tiles_max;
  float scale_log2;          // softmax scale * log2(e)
  int num_blocks;
  int64_t total_rows;         // total_q * Hq: rows of out / part_o that exist (writes beyond are skipped)
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ uint32_t cvt_e4m3x2_f16x2(uint16_t v) {
  uint32_t r;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(v));
  return r;
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
}  // namespace daser

// tcgen05 / TMEM variant for chunked prefill (attention_tc.cu): one CTA per 128 query rows of a
// KV head and per KV split.  Returns a CUDA error code.
int daser_launch_attention_tc(const daser::AttnParams& p, int max_q_len, cudaStream_t stream);
