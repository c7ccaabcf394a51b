// Paged fp8 attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference project (which has no GPU kernels at
// all); it is an addition of this library.
//
// Who needs it: code that runs where cudaMalloc is off limits - a serving process whose
// device memory was carved up and frozen at start-up so that no later allocation can
// fragment it or fail under load, a latency-critical loop that cannot take the implicit
// device synchronisation an allocation may cause, or a host language runtime that only hands
// raw pointers through a C ABI and owns no device allocator of its own.  The regular entry point, daser_paged_attention_fp8, leaves the
// split-KV scratch (partial outputs and log-sum-exp values, one set per KV split) to the
// caller, and the Python wrapper gets it from torch's allocator.  Here the scratch is a fixed
// array that lives inside the loaded library instead.
//
// Limits and rules:
//  * The scratch holds DASER_NOALLOC_MAX_ROW_SPLITS (query rows x KV splits) entries of
//    128 + 1 floats: about 8.3 MB of device memory on every GPU that loads the library,
//    held until the process exits.  A call with total_q * Hq * nsplit above that limit is
//    refused with DASER_ERR_TOO_LARGE (-3) and launches nothing.
//  * No cudaMalloc, cudaFree or other allocating call is made, and torch is not involved.
//  * The first call on each device looks up the array's device address (one
//    cudaGetSymbolAddress with that device current) and caches it.  Make that first call
//    before any stream capture begins.
//  * Every call on a device shares the one array and finds the previous call's contents in
//    it.  Nothing in it has to start at zero: every entry the merge step reads is written
//    by the same call first.  Two calls whose kernels overlap on the GPU (different streams
//    without an ordering between them) race on the array; order them.
//
// Arguments are those of daser_paged_attention_fp8 minus the two scratch pointers; inputs
// and outputs are still the caller's.  Returns 0, a negative DASER_ERR_* code, or a
// positive cudaError_t.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "kv_paged.h"

#define DASER_NOALLOC_MAX_ROW_SPLITS 16384

#ifdef __cplusplus
extern "C" {
#endif

__attribute__((visibility("default"))) int daser_paged_attention_fp8_noalloc(
    const void* q, void* out, const DaserKVPool* pool, int layer, int rank, const int32_t* block_tables,
    int max_blocks, const int32_t* q_start, const int32_t* ctx_lens, int num_seqs, int total_q, int max_q_len,
    int Hq, int Hkv, int head_dim, int block_tokens, int nsplit, int split_tokens, float softmax_scale,
    cudaStream_t stream);

#ifdef __cplusplus
}
#endif
