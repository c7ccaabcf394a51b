// Host-visible parameter blocks of the restore / save kernels (mirrored with ctypes
// in daser_b200/ops/kv_ops.py; keep field order and types in sync).
#pragma once
#include <stdint.h>

#define DASER_MAX_RANKS 8

// Return codes of every host entry point of the library: 0 = ok, a positive value is a
// cudaError_t, negative values are these.
#ifndef DASER_ERR_BAD_ARG
#define DASER_ERR_BAD_ARG (-1)
#define DASER_ERR_UNSUPPORTED (-2)
#define DASER_ERR_TOO_LARGE (-3)
#endif

// A paged KV pool, one base pointer per tensor-parallel rank.  Addresses of peers are
// peer-mapped device pointers; element (layer, block, kv, tok, head_local, dim) of rank r
// lives at payload[r] + layer*stride_layer + block*stride_block + kv*stride_kv +
// tok*stride_tok + head_local*stride_head + dim (strides in elements, dim contiguous).
// For an fp8 pool the scale tensor has the same shape with the last dimension divided
// by 16, so every scale stride is the payload stride / 16.
typedef struct {
  void* payload[DASER_MAX_RANKS];
  float* scales[DASER_MAX_RANKS];
  int64_t stride_layer;
  int64_t stride_block;
  int64_t stride_kv;
  int64_t stride_tok;
  int64_t stride_head;
  int32_t num_blocks;       // blocks per layer in every rank's pool (bounds check)
  int32_t n_ranks;          // tensor-parallel degree
  int32_t heads_per_rank;   // KV heads each rank keeps (1 when n_ranks > num_kv_heads)
  int32_t pool_is_fp8;      // 1: e4m3 payload + fp32 scales, 0: bf16
} DaserKVPool;

typedef struct {
  const uint64_t* slot_ptr;  // [n_slots] address of each slot image (source for restore,
                             // destination for save); device, peer or host-mapped memory
  const int32_t* block_id;   // [n_slots] pool block of each slot
  const int32_t* delta;      // [n_slots] positions to rotate keys by (restore only; may be null)
  const float* cos_sin;      // [max_pos][head_dim]: cos in [0, D/2), sin in [D/2, D)
  uint32_t* status;          // [2]: {error code, offending slot index}; may be null
  int32_t max_pos;
  int32_t n_slots;
  int32_t num_layers;
  int32_t num_kv_heads;      // heads stored in a slot image (all heads, TP-agnostic)
  int32_t head_dim;
  int32_t block_tokens;
  int32_t image_is_fp8;      // slot image codec: 1 fp8b16, 0 raw bf16
  int32_t rank;              // save only: whose heads this launch writes
  int32_t layer_begin;       // restore only: first layer this launch covers
  int32_t layer_count;       // restore only: how many layers from layer_begin (0 = all of them)
  int32_t lg_heads;          // filled in by the launcher: log2 of num_kv_heads, block_tokens and
  int32_t lg_tokens;         //   head_dim / 16 when all three are powers of two (the kernels then
  int32_t lg_groups;         //   index with shifts), else -1
  int32_t reserved;
} DaserKVJob;
