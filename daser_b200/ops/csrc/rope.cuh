// RoPE + paged KV write of one (token, head, pair of 16-wide groups): shared by the stand-alone
// kernel (elementwise.cu) and the QKV GEMM's fused epilogue (gemm.cu).
//
// x1 holds head dims [16j, 16j + 16), x2 the rotary partners [D/2 + 16j, D/2 + 16j + 16): two fp8
// scale groups, so rotation and quantisation stay thread local.  Query heads go to q_out (bf16,
// [T, Hq, D]); key and value heads go into the paged pool at slot_mapping[t]
// (block * block_tokens + offset; negative = no write), keys rotated, values as they are.
#pragma once
#include "common.cuh"

namespace daser {

struct RopeKvWrite {
  const int32_t* positions;
  const int64_t* slot_mapping;
  const float* cos_sin;  // [max_pos][D]: cos in [0, D/2), sin in [D/2, D)
  int max_pos;
  __nv_bfloat16* q_out;
  int Hq, Hkv, D, block_tokens;
  DaserKVPool pool;
  int layer, rank;
};

template <bool POOL_FP8>
__device__ __forceinline__ void rope_kv_write_item(const RopeKvWrite& r, float (&x1)[16], float (&x2)[16], int t,
                                                   int hd, int j) {
  const int D = r.D, half = D >> 1;
  const bool is_v = hd >= r.Hq + r.Hkv;
  if (!is_v) {
    int pos = r.positions[t];
    pos = pos < 0 ? 0 : (pos >= r.max_pos ? r.max_pos - 1 : pos);
    const float* cs = r.cos_sin + (int64_t)pos * D + j * FP8_GROUP;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float c = cs[i], s = cs[half + i];
      const float a = x1[i], b = x2[i];
      x1[i] = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
      x2[i] = __fadd_rn(__fmul_rn(b, c), __fmul_rn(a, s));
    }
  }
  if (hd < r.Hq) {
    __nv_bfloat16* dst = r.q_out + ((int64_t)t * r.Hq + hd) * D + j * FP8_GROUP;
    store_bf16x16(dst, x1);
    store_bf16x16(dst + half, x2);
    return;
  }
  const int64_t sm = r.slot_mapping[t];
  if (sm < 0) return;
  const int block = (int)(sm / r.block_tokens), tok = (int)(sm % r.block_tokens);
  if (block >= r.pool.num_blocks) return;
  const int kv = is_v ? 1 : 0;
  const int hl = is_v ? hd - r.Hq - r.Hkv : hd - r.Hq;
  const int64_t d1 = (int64_t)r.layer * r.pool.stride_layer + (int64_t)block * r.pool.stride_block +
                     (int64_t)kv * r.pool.stride_kv + (int64_t)tok * r.pool.stride_tok +
                     (int64_t)hl * r.pool.stride_head + j * FP8_GROUP;
  const int64_t d2 = d1 + half;
  if (POOL_FP8) {
    uint4 q1, q2;
    float s1, s2;
    // quantise what a bf16 pool would have held, so both pool kinds see the same values
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      x1[i] = __bfloat162float(__float2bfloat16(x1[i]));
      x2[i] = __bfloat162float(__float2bfloat16(x2[i]));
    }
    quant_group16(x1, q1, s1);
    quant_group16(x2, q2, s2);
    uint8_t* p = reinterpret_cast<uint8_t*>(r.pool.payload[r.rank]);
    *reinterpret_cast<uint4*>(p + d1) = q1;
    *reinterpret_cast<uint4*>(p + d2) = q2;
    r.pool.scales[r.rank][d1 / FP8_GROUP] = s1;
    r.pool.scales[r.rank][d2 / FP8_GROUP] = s2;
  } else {
    __nv_bfloat16* p = reinterpret_cast<__nv_bfloat16*>(r.pool.payload[r.rank]);
    store_bf16x16(p + d1, x1);
    store_bf16x16(p + d2, x2);
  }
}

}  // namespace daser
