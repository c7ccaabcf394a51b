// Paged attention that reads block-scaled fp8 KV directly (decode and chunked prefill).
//
// In the reference's serving stack this is stock vLLM's FlashAttention / FlashInfer paged
// kernel over a bf16 cache; here the cache holds e4m3 payload + one fp32 scale per 16 dims and
// is dequantised on the fly, so a decode step moves 1.25 bytes per KV element instead of 2.
//
// One WARP is one worker: it owns a tile of 16 query rows (rows = query tokens x the G query
// heads that share one KV head, G | 16) and a contiguous range of KV pages (split-KV), streams
// those pages through its private cp.async ring in shared memory, and keeps an online softmax.
// No CTA-wide synchronisation exists in the main loop.  With more than one split the partial
// results (normalised O and log2-sum-exp) go to a scratch buffer and a merge kernel combines
// them.
//
// Tensor-core mapping (mma.sync m16n8k16, f16 inputs, fp32 accumulate; the op is bandwidth
// bound, the MMA only has to keep up with HBM).  The contraction index of an MMA may be
// permuted freely as long as A and B agree, and so may the N index of the output, so each
// thread is given data that is contiguous in memory:
//   S = Q K^T : lane (g = lane/4, t = lane%4) supplies, for key token g (and g+8), the 16 dims
//               of scale group t and the 16 dims of scale group 4+t; k-step kk uses elements
//               2kk, 2kk+1 of each.  Q fragments are loaded with the same permutation.
//   O = P V   : lane (g, t) supplies dims [16g, 16g+16) (one scale group) of tokens
//               2t, 2t+1, 2t+8, 2t+9; MMA n-tile j uses dim 16g + j.  The lane therefore
//               accumulates output dims [32t, 32t+32) of rows g and g+8.
#include <stdlib.h>

#include "attention_params.cuh"

namespace daser {

__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(ATT_WARPS * 32, 2)
paged_attn_fp8_kernel(const AttnParams p) {
  extern __shared__ __align__(16) uint8_t att_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int kvh = blockIdx.x, seq = blockIdx.y;
  const int item = blockIdx.z * ATT_WARPS + warp;
  const int rt = item / p.nsplit, sp = item % p.nsplit;
  pdl_enter();
  if (rt >= p.row_tiles_max) return;

  const int q0 = p.q_start[seq];
  const int q_len = p.q_start[seq + 1] - q0;
  const int ctx = p.ctx_lens[seq];
  const int G = p.G;
  const int toks_per_tile = 16 / G;
  const int tok_first = rt * toks_per_tile;
  if (tok_first >= q_len) return;
  const int tok_last = min(tok_first + toks_per_tile, q_len) - 1;
  // keys visible to the last row of the tile
  const int limit = ctx - q_len + tok_last + 1;
  const int key_begin = sp * p.split_tokens;
  const int key_end = min(key_begin + p.split_tokens, limit);

  // rows of this lane: r0 = g, r1 = g + 8
  const int tq0 = tok_first + g / G, tq1 = tok_first + (g + 8) / G;
  const int hq0 = kvh * G + g % G, hq1 = kvh * G + (g + 8) % G;
  const bool v0 = tq0 < q_len, v1 = tq1 < q_len;
  const int pos0 = ctx - q_len + tq0, pos1 = ctx - q_len + tq1;  // last visible key index per row

  float o[16][4];
#pragma unroll
  for (int j = 0; j < 16; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  if (key_begin < key_end) {
    // ---- Q fragments (scaled, f16), permuted as described above ----
    uint32_t qa[8][4];
    {
      const __nv_bfloat16* q0p = p.q + ((int64_t)(q0 + tq0) * p.Hq + hq0) * ATT_D;
      const __nv_bfloat16* q1p = p.q + ((int64_t)(q0 + tq1) * p.Hq + hq1) * ATT_D;
      float a[16], b[16], c[16], d[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) a[i] = b[i] = c[i] = d[i] = 0.f;
      if (v0) { load_bf16x16(q0p + 16 * t, a); load_bf16x16(q0p + 64 + 16 * t, b); }
      if (v1) { load_bf16x16(q1p + 16 * t, c); load_bf16x16(q1p + 64 + 16 * t, d); }
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        qa[kk][0] = pack_half2(a[2 * kk] * p.scale_log2, a[2 * kk + 1] * p.scale_log2);
        qa[kk][1] = pack_half2(c[2 * kk] * p.scale_log2, c[2 * kk + 1] * p.scale_log2);
        qa[kk][2] = pack_half2(b[2 * kk] * p.scale_log2, b[2 * kk + 1] * p.scale_log2);
        qa[kk][3] = pack_half2(d[2 * kk] * p.scale_log2, d[2 * kk + 1] * p.scale_log2);
      }
    }

    uint8_t* ring = att_smem + warp * (ATT_STAGES * ATT_STAGE_BYTES);
    const uint32_t ring_u32 = static_cast<uint32_t>(__cvta_generic_to_shared(ring));
    const int32_t* table = p.block_tables + (int64_t)seq * p.max_blocks;
    const int page_begin = key_begin / ATT_B;
    const int page_end = (key_end + ATT_B - 1) / ATT_B;
    const int n_pages = page_end - page_begin;

    auto issue = [&](int pi) {
      const int stage = pi % ATT_STAGES;
      const uint32_t sbase = ring_u32 + stage * ATT_STAGE_BYTES;
      int blk = table[min(page_begin + pi, p.max_blocks - 1)];
      blk = blk < 0 ? 0 : (blk >= p.num_blocks ? p.num_blocks - 1 : blk);
      const int64_t base_k = (int64_t)blk * p.stride_block + (int64_t)kvh * p.stride_head;
      const int64_t base_v = base_k + p.stride_kv;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int piece = lane + 32 * i;  // 128 pieces of 16 B per 2 KiB page
        const int tok = piece >> 3, slot = piece & 7;
        const int64_t src = (int64_t)tok * p.stride_tok + slot * 16;
        cp_async16(sbase + tok * 128 + ((slot ^ ((tok & 1) << 2)) << 4), p.kv_payload + base_k + src);
        cp_async16(sbase + 2048 + tok * 128 + ((slot ^ (((tok >> 1) & 3) << 1)) << 4), p.kv_payload + base_v + src);
      }
      {
        // scales: 16 tokens x 8 floats = 512 B per page and per K/V; lane -> (token = lane/2, half = lane%2)
        const int tok = lane >> 1, hf = lane & 1;
        const int64_t soff = (base_k + (int64_t)tok * p.stride_tok) / 16 + hf * 4;
        const int64_t voff = (base_v + (int64_t)tok * p.stride_tok) / 16 + hf * 4;
        cp_async16(sbase + 4096 + lane * 16, p.kv_scales + soff);
        cp_async16(sbase + 4608 + lane * 16, p.kv_scales + voff);
      }
    };

#pragma unroll
    for (int s = 0; s < ATT_STAGES - 1; ++s) {
      if (s < n_pages) issue(s);
      cp_async_commit();
    }

    for (int pi = 0; pi < n_pages; ++pi) {
      cp_async_wait<ATT_STAGES - 2>();
      __syncwarp();
      const uint8_t* st = ring + (pi % ATT_STAGES) * ATT_STAGE_BYTES;
      const float* ksc = reinterpret_cast<const float*>(st + 4096);
      const float* vsc = reinterpret_cast<const float*>(st + 4608);
      const int key0 = (page_begin + pi) * ATT_B;

      // ---- S = Q K^T for the 16 tokens of the page (two n-tiles of 8 tokens) ----
      float s[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
        const int tok = nt * 8 + g;
        const int sw = (tok & 1) << 2;
        const uint4 lo = *reinterpret_cast<const uint4*>(st + tok * 128 + ((t ^ sw) << 4));
        const uint4 hi = *reinterpret_cast<const uint4*>(st + tok * 128 + (((4 + t) ^ sw) << 4));
        const float slo = ksc[tok * 8 + t], shi = ksc[tok * 8 + 4 + t];
        const uint32_t slo2 = pack_half2(slo, slo), shi2 = pack_half2(shi, shi);
        const uint32_t wl[4] = {lo.x, lo.y, lo.z, lo.w}, wh[4] = {hi.x, hi.y, hi.z, hi.w};
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint16_t el = (uint16_t)(wl[kk >> 1] >> ((kk & 1) * 16));
          const uint16_t eh = (uint16_t)(wh[kk >> 1] >> ((kk & 1) * 16));
          const uint32_t b0 = hmul2_u32(cvt_e4m3x2_f16x2(el), slo2);
          const uint32_t b1 = hmul2_u32(cvt_e4m3x2_f16x2(eh), shi2);
          mma_16816(s[nt], qa[kk], b0, b1);
        }
      }
      // ---- mask, online softmax ----
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int key = key0 + nt * 8 + 2 * t + e;
          const bool in = key < key_end && key >= key_begin;
          if (!(in && v0 && key <= pos0)) s[nt][e] = -INFINITY;
          if (!(in && v1 && key <= pos1)) s[nt][2 + e] = -INFINITY;
          mx0 = fmaxf(mx0, s[nt][e]);
          mx1 = fmaxf(mx1, s[nt][2 + e]);
        }
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
      const float base0 = mn0 == -INFINITY ? 0.f : mn0, base1 = mn1 == -INFINITY ? 0.f : mn1;
      const float al0 = exp2f(m0 - base0), al1 = exp2f(m1 - base1);  // m = -inf gives 0
      const bool rescale = (mn0 != m0) || (mn1 != m1);
      m0 = mn0;
      m1 = mn1;
      uint32_t pa[4];
      {
        const float p00 = exp2f(s[0][0] - base0), p01 = exp2f(s[0][1] - base0);
        const float p02 = exp2f(s[0][2] - base1), p03 = exp2f(s[0][3] - base1);
        const float p10 = exp2f(s[1][0] - base0), p11 = exp2f(s[1][1] - base0);
        const float p12 = exp2f(s[1][2] - base1), p13 = exp2f(s[1][3] - base1);
        l0 = l0 * al0 + (p00 + p01 + p10 + p11);
        l1 = l1 * al1 + (p02 + p03 + p12 + p13);
        pa[0] = pack_half2(p00, p01);  // row g,   tokens 2t, 2t+1
        pa[1] = pack_half2(p02, p03);  // row g+8, tokens 2t, 2t+1
        pa[2] = pack_half2(p10, p11);  // row g,   tokens 2t+8, 2t+9
        pa[3] = pack_half2(p12, p13);  // row g+8, tokens 2t+8, 2t+9
      }
      if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          o[j][0] *= al0; o[j][1] *= al0; o[j][2] *= al1; o[j][3] *= al1;
        }
      }
      // ---- O += P V ----
      {
        uint4 vr[4];
        float vs[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int tok = 2 * t + (i & 1) + (i >> 1) * 8;
          vr[i] = *reinterpret_cast<const uint4*>(st + 2048 + tok * 128 + ((g ^ (((tok >> 1) & 3) << 1)) << 4));
          vs[i] = vsc[tok * 8 + g];
        }
        const uint32_t sc01 = pack_half2(vs[0], vs[1]), sc23 = pack_half2(vs[2], vs[3]);
        const uint32_t w0[4] = {vr[0].x, vr[0].y, vr[0].z, vr[0].w}, w1[4] = {vr[1].x, vr[1].y, vr[1].z, vr[1].w};
        const uint32_t w2[4] = {vr[2].x, vr[2].y, vr[2].z, vr[2].w}, w3[4] = {vr[3].x, vr[3].y, vr[3].z, vr[3].w};
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          // byte j of token A in the low byte, byte j of token B in the next one
          const uint32_t sel = (uint32_t)(j & 3) | ((uint32_t)(4 + (j & 3)) << 4);
          const uint32_t e01 = __byte_perm(w0[j >> 2], w1[j >> 2], sel);
          const uint32_t e23 = __byte_perm(w2[j >> 2], w3[j >> 2], sel);
          const uint32_t b0 = hmul2_u32(cvt_e4m3x2_f16x2((uint16_t)e01), sc01);
          const uint32_t b1 = hmul2_u32(cvt_e4m3x2_f16x2((uint16_t)e23), sc23);
          mma_16816(o[j], pa, b0, b1);
        }
      }
      __syncwarp();  // every lane is done with this stage before it is refilled
      if (pi + ATT_STAGES - 1 < n_pages) issue(pi + ATT_STAGES - 1);
      cp_async_commit();
    }
    cp_async_wait<0>();
  }

  // ---- finalise ----
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const bool valid = r ? v1 : v0;
    if (!valid) continue;
    const int tq = r ? tq1 : tq0, hq = r ? hq1 : hq0;
    const float inv = r ? inv1 : inv0;
    float vals[32];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      vals[j] = o[j][2 * r] * inv;
      vals[16 + j] = o[j][2 * r + 1] * inv;
    }
    const int64_t row = (int64_t)(q0 + tq) * p.Hq + hq;
    if (row >= p.total_rows) continue;  // q_start names more rows than the caller's buffers hold
    if (p.nsplit == 1) {
      __nv_bfloat16* dst = p.out + row * ATT_D + 32 * t;
      float lo[16], hi[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) { lo[i] = vals[i]; hi[i] = vals[16 + i]; }
      store_bf16x16(dst, lo);
      store_bf16x16(dst + 16, hi);
    } else {
      float* dst = p.part_o + (row * p.nsplit + sp) * ATT_D + 32 * t;
#pragma unroll
      for (int i = 0; i < 8; ++i)
        *reinterpret_cast<float4*>(dst + 4 * i) = make_float4(vals[4 * i], vals[4 * i + 1], vals[4 * i + 2], vals[4 * i + 3]);
      if (t == 0) {
        const float l = r ? l1 : l0, m = r ? m1 : m0;
        p.part_lse[row * p.nsplit + sp] = l > 0.f ? m + log2f(l) : -INFINITY;
      }
    }
  }
}

// ---- prefill variant: one CTA = four row tiles sharing one dequantised KV stream ----------------
//
// With many query tokens the per-warp kernel above converts the same fp8 page to f16 once per
// row tile.  Here the four warps of a CTA take four consecutive row tiles (64 query rows) of
// the same KV head, the CTA streams the pages once (cp.async ring of raw pages), all 128
// threads dequantise a page into f16 tiles in shared memory (one 16-dim scale group per
// thread), and every warp reads its MMA operands from there with ldmatrix (K as the "col"
// operand directly, V through ldmatrix.trans).  f16 tiles are double buffered: one CTA
// barrier per page.  Rows are in the standard m16n8k16 layout (no permutation tricks needed).
constexpr int PF_STAGES = 4;
constexpr int PF_RAW_BYTES = ATT_STAGE_BYTES;                 // 5120: K, V payload + scales
constexpr int PF_F16_BYTES = 2 * ATT_B * ATT_D * 2;           // 8192: K and V tiles in f16
constexpr int PF_SMEM = PF_STAGES * PF_RAW_BYTES + 2 * PF_F16_BYTES;

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

__global__ void __launch_bounds__(128, 3)
paged_attn_fp8_prefill_kernel(const AttnParams p) {
  extern __shared__ __align__(128) uint8_t pf_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int kvh = blockIdx.x, seq = blockIdx.y;
  const int grp = blockIdx.z / p.nsplit, sp = blockIdx.z % p.nsplit;
  pdl_enter();
  const int q0 = p.q_start[seq];
  const int q_len = p.q_start[seq + 1] - q0;
  const int ctx = p.ctx_lens[seq];
  const int G = p.G;
  const int toks_per_tile = 16 / G;
  const int grp_tok_first = grp * 4 * toks_per_tile;
  if (grp_tok_first >= q_len) return;  // uniform over the CTA
  const int grp_tok_last = min(grp_tok_first + 4 * toks_per_tile, q_len) - 1;
  const int grp_limit = ctx - q_len + grp_tok_last + 1;
  const int key_begin = sp * p.split_tokens;
  const int key_end = min(key_begin + p.split_tokens, grp_limit);

  // this warp's row tile
  const int tok_first = grp_tok_first + warp * toks_per_tile;
  const bool tile_live = tok_first < q_len;
  const int tq0 = tok_first + g / G, tq1 = tok_first + (g + 8) / G;
  const int hq0 = kvh * G + g % G, hq1 = kvh * G + (g + 8) % G;
  const bool v0 = tile_live && tq0 < q_len, v1 = tile_live && tq1 < q_len;
  const int pos0 = ctx - q_len + tq0, pos1 = ctx - q_len + tq1;
  const int my_limit = tile_live ? ctx - q_len + min(tok_first + toks_per_tile, q_len) : 0;  // keys this tile can see

  float o[16][4];
#pragma unroll
  for (int j = 0; j < 16; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  if (key_begin < key_end) {
    // Q fragments, standard layout: [kk][0]=(row g, dims 16kk+2t,+1) [1]=(row g+8) [2]=(row g, +8) [3]=(row g+8, +8)
    uint32_t qa[8][4];
    {
      const __nv_bfloat16* q0p = p.q + ((int64_t)(q0 + tq0) * p.Hq + hq0) * ATT_D;
      const __nv_bfloat16* q1p = p.q + ((int64_t)(q0 + tq1) * p.Hq + hq1) * ATT_D;
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int d = 16 * kk + 8 * h + 2 * t;
          const uint32_t a = v0 ? *reinterpret_cast<const uint32_t*>(q0p + d) : 0u;
          const uint32_t b = v1 ? *reinterpret_cast<const uint32_t*>(q1p + d) : 0u;
          qa[kk][2 * h] = pack_half2(bf16_lo(a) * p.scale_log2, bf16_hi(a) * p.scale_log2);
          qa[kk][2 * h + 1] = pack_half2(bf16_lo(b) * p.scale_log2, bf16_hi(b) * p.scale_log2);
        }
      }
    }
    uint8_t* raw = pf_smem;
    uint8_t* f16 = pf_smem + PF_STAGES * PF_RAW_BYTES;
    const uint32_t raw_u32 = static_cast<uint32_t>(__cvta_generic_to_shared(raw));
    const uint32_t f16_u32 = static_cast<uint32_t>(__cvta_generic_to_shared(f16));
    const int32_t* table = p.block_tables + (int64_t)seq * p.max_blocks;
    const int page_begin = key_begin / ATT_B;
    const int n_pages = (key_end + ATT_B - 1) / ATT_B - page_begin;

    auto issue = [&](int pi) {  // 320 pieces of 16 B per page, 128 threads
      const uint32_t sbase = raw_u32 + (pi % PF_STAGES) * PF_RAW_BYTES;
      int blk = table[min(page_begin + pi, p.max_blocks - 1)];
      blk = blk < 0 ? 0 : (blk >= p.num_blocks ? p.num_blocks - 1 : blk);
      const int64_t base_k = (int64_t)blk * p.stride_block + (int64_t)kvh * p.stride_head;
      const int64_t base_v = base_k + p.stride_kv;
      for (int piece = threadIdx.x; piece < 320; piece += 128) {
        if (piece < 256) {
          const int which = piece >> 7, q = piece & 127, tok = q >> 3, slot = q & 7;
          const int64_t src = (which ? base_v : base_k) + (int64_t)tok * p.stride_tok + slot * 16;
          cp_async16(sbase + which * 2048 + q * 16, p.kv_payload + src);
        } else {
          const int q = piece - 256, which = q >> 5, r = q & 31, tok = r >> 1, hf = r & 1;
          const int64_t soff = ((which ? base_v : base_k) + (int64_t)tok * p.stride_tok) / 16 + hf * 4;
          cp_async16(sbase + 4096 + which * 512 + r * 16, p.kv_scales + soff);
        }
      }
    };
#pragma unroll
    for (int s = 0; s < PF_STAGES - 1; ++s) {
      if (s < n_pages) issue(s);
      cp_async_commit();
    }
    for (int pi = 0; pi < n_pages; ++pi) {
      cp_async_wait<PF_STAGES - 2>();
      __syncthreads();  // raw page pi has landed for everyone; f16 buffer (pi & 1) is free (read at pi - 2)
      {
        // dequantise: thread -> (which = K|V, token, 16-dim chunk); 256 chunks per page, 2 per thread
        const uint8_t* st = raw + (pi % PF_STAGES) * PF_RAW_BYTES;
        uint8_t* dstb = f16 + (pi & 1) * PF_F16_BYTES;
#pragma unroll
        for (int rep = 0; rep < 2; ++rep) {
          const int item = threadIdx.x + rep * 128;
          const int which = item >> 7, q = item & 127, tok = q >> 3, chunk = q & 7;
          const uint4 w = *reinterpret_cast<const uint4*>(st + which * 2048 + q * 16);
          const float sc = reinterpret_cast<const float*>(st + 4096 + which * 512)[tok * 8 + chunk];
          const uint32_t sc2 = pack_half2(sc, sc);
          const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
          uint32_t h[8];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            h[2 * i] = hmul2_u32(cvt_e4m3x2_f16x2((uint16_t)(ww[i] & 0xffffu)), sc2);
            h[2 * i + 1] = hmul2_u32(cvt_e4m3x2_f16x2((uint16_t)(ww[i] >> 16)), sc2);
          }
          uint8_t* row = dstb + which * 4096 + tok * 256;
          *reinterpret_cast<uint4*>(row + (((2 * chunk) ^ (tok & 7)) << 4)) = make_uint4(h[0], h[1], h[2], h[3]);
          *reinterpret_cast<uint4*>(row + (((2 * chunk + 1) ^ (tok & 7)) << 4)) = make_uint4(h[4], h[5], h[6], h[7]);
        }
      }
      // the next raw page may be fetched now (its stage was consumed by the dequant of page pi - 1)
      if (pi + PF_STAGES - 1 < n_pages) issue(pi + PF_STAGES - 1);
      cp_async_commit();
      __syncthreads();  // f16 tiles of page pi are complete
      const int key0 = (page_begin + pi) * ATT_B;
      if (tile_live && key0 < my_limit) {
        const uint32_t kt = f16_u32 + (pi & 1) * PF_F16_BYTES, vt = kt + 4096;
        float s[2][4];
        s[0][0] = s[0][1] = s[0][2] = s[0][3] = s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.f;
        {
          const int mi = lane >> 3, r = lane & 7;
          const int tok = r + 8 * (mi >> 1);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            uint32_t b[4];
            ldmatrix_x4(b, kt + tok * 256 + (((2 * kk + (mi & 1)) ^ (tok & 7)) << 4));
            mma_16816(s[0], qa[kk], b[0], b[1]);
            mma_16816(s[1], qa[kk], b[2], b[3]);
          }
        }
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int key = key0 + nt * 8 + 2 * t + e;
            const bool in = key < key_end;
            if (!(in && v0 && key <= pos0)) s[nt][e] = -INFINITY;
            if (!(in && v1 && key <= pos1)) s[nt][2 + e] = -INFINITY;
            mx0 = fmaxf(mx0, s[nt][e]);
            mx1 = fmaxf(mx1, s[nt][2 + e]);
          }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float base0 = mn0 == -INFINITY ? 0.f : mn0, base1 = mn1 == -INFINITY ? 0.f : mn1;
        const float al0 = exp2f(m0 - base0), al1 = exp2f(m1 - base1);
        const bool rescale = (mn0 != m0) || (mn1 != m1);
        m0 = mn0;
        m1 = mn1;
        uint32_t pa[4];
        {
          const float p00 = exp2f(s[0][0] - base0), p01 = exp2f(s[0][1] - base0);
          const float p02 = exp2f(s[0][2] - base1), p03 = exp2f(s[0][3] - base1);
          const float p10 = exp2f(s[1][0] - base0), p11 = exp2f(s[1][1] - base0);
          const float p12 = exp2f(s[1][2] - base1), p13 = exp2f(s[1][3] - base1);
          l0 = l0 * al0 + (p00 + p01 + p10 + p11);
          l1 = l1 * al1 + (p02 + p03 + p12 + p13);
          pa[0] = pack_half2(p00, p01);
          pa[1] = pack_half2(p02, p03);
          pa[2] = pack_half2(p10, p11);
          pa[3] = pack_half2(p12, p13);
        }
        if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            o[j][0] *= al0; o[j][1] *= al0; o[j][2] *= al1; o[j][3] *= al1;
          }
        }
        {
          const int mi = lane >> 3, r = lane & 7;
          const int tok = r + 8 * (mi & 1);
#pragma unroll
          for (int j2 = 0; j2 < 8; ++j2) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, vt + tok * 256 + (((2 * j2 + (mi >> 1)) ^ (tok & 7)) << 4));
            mma_16816(o[2 * j2], pa, b[0], b[1]);
            mma_16816(o[2 * j2 + 1], pa, b[2], b[3]);
          }
        }
      }
    }
    cp_async_wait<0>();
  }
  if (!tile_live) return;
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    if (!(r ? v1 : v0)) continue;
    const int tq = r ? tq1 : tq0, hq = r ? hq1 : hq0;
    const float inv = r ? inv1 : inv0;
    const int64_t row = (int64_t)(q0 + tq) * p.Hq + hq;
    if (row >= p.total_rows) continue;
    if (p.nsplit == 1) {
      __nv_bfloat16* dst = p.out + row * ATT_D + 2 * t;
#pragma unroll
      for (int j = 0; j < 16; ++j)
        *reinterpret_cast<uint32_t*>(dst + 8 * j) = pack_bf16x2(o[j][2 * r] * inv, o[j][2 * r + 1] * inv);
    } else {
      float* dst = p.part_o + (row * p.nsplit + sp) * ATT_D + 2 * t;
#pragma unroll
      for (int j = 0; j < 16; ++j)
        *reinterpret_cast<float2*>(dst + 8 * j) = make_float2(o[j][2 * r] * inv, o[j][2 * r + 1] * inv);
      if (t == 0) {
        const float l = r ? l1 : l0, m = r ? m1 : m0;
        p.part_lse[row * p.nsplit + sp] = l > 0.f ? m + log2f(l) : -INFINITY;
      }
    }
  }
}

// One warp per (query token, head): out = sum_s w_s O_s / sum_s w_s, w_s = 2^(lse_s - max).
__global__ void __launch_bounds__(128)
attn_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                  __nv_bfloat16* __restrict__ out, int64_t rows, int nsplit) {
  const int64_t row = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  pdl_enter();
  if (row >= rows) return;
  float mx = -INFINITY;
  for (int s = 0; s < nsplit; ++s) mx = fmaxf(mx, part_lse[row * nsplit + s]);
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  float wsum = 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const float lse = part_lse[row * nsplit + s];
    if (lse == -INFINITY) continue;
    const float w = exp2f(lse - mx);
    const float4 v = *reinterpret_cast<const float4*>(part_o + (row * nsplit + s) * ATT_D + lane * 4);
    acc[0] += w * v.x; acc[1] += w * v.y; acc[2] += w * v.z; acc[3] += w * v.w;
    wsum += w;
  }
  const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
  uint2 o;
  o.x = pack_bf16x2(acc[0] * inv, acc[1] * inv);
  o.y = pack_bf16x2(acc[2] * inv, acc[3] * inv);
  *reinterpret_cast<uint2*>(out + row * ATT_D + lane * 4) = o;
}

}  // namespace daser

// Chunked prefill goes to the tcgen05 kernel unless DASER_ATTN_TC=0 (or the setter) says otherwise.
static int g_attn_tc_mode = -1;
static bool attention_tc_enabled() {
  if (g_attn_tc_mode < 0) {
    const char* v = getenv("DASER_ATTN_TC");
    g_attn_tc_mode = (v && v[0] == '0') ? 0 : 1;
  }
  return g_attn_tc_mode != 0;
}
DASER_API void daser_attention_set_tc(int enabled) { g_attn_tc_mode = enabled ? 1 : 0; }

// Paged attention over an fp8b16 pool.  `pool` gives the layout; only this rank's base
// pointers (index `rank`) are used.  part_o / part_lse are scratch of
// Tq*Hq*nsplit*(128+1) floats, needed when nsplit > 1.
DASER_API int daser_paged_attention_fp8(const void* q, void* out, float* part_o, float* part_lse,
                                        const DaserKVPool* pool, int layer, int rank,
                                        const int32_t* block_tables, int max_blocks, const int32_t* q_start,
                                        const int32_t* ctx_lens, int num_seqs, int total_q, int max_q_len,
                                        int Hq, int Hkv, int head_dim, int block_tokens, int nsplit,
                                        int split_tokens, float softmax_scale, cudaStream_t stream) {
  using namespace daser;
  if (!pool || !pool->pool_is_fp8) return DASER_ERR_UNSUPPORTED;
  if (head_dim != ATT_D || block_tokens != ATT_B) return DASER_ERR_UNSUPPORTED;
  if (Hkv <= 0 || Hq % Hkv) return DASER_ERR_BAD_ARG;
  const int G = Hq / Hkv;
  if (G > 16 || 16 % G) return DASER_ERR_UNSUPPORTED;
  if (nsplit < 1 || split_tokens <= 0 || split_tokens % ATT_B) return DASER_ERR_BAD_ARG;
  if (nsplit > 1 && (!part_o || !part_lse)) return DASER_ERR_BAD_ARG;
  if (num_seqs <= 0 || total_q <= 0) return 0;
  if (pool->stride_tok % 16 || pool->stride_head % 16 || pool->stride_kv % 16 || pool->stride_block % 16) return DASER_ERR_UNSUPPORTED;
  AttnParams p;
  p.q = (const __nv_bfloat16*)q;
  p.out = (__nv_bfloat16*)out;
  p.part_o = part_o;
  p.part_lse = part_lse;
  p.kv_payload = (const uint8_t*)pool->payload[rank] + (int64_t)layer * pool->stride_layer;
  p.kv_scales = pool->scales[rank] + (int64_t)layer * pool->stride_layer / 16;
  p.stride_block = pool->stride_block; p.stride_kv = pool->stride_kv;
  p.stride_head = pool->stride_head; p.stride_tok = pool->stride_tok;
  p.block_tables = block_tables; p.max_blocks = max_blocks;
  p.q_start = q_start; p.ctx_lens = ctx_lens;
  p.num_seqs = num_seqs; p.Hq = Hq; p.Hkv = Hkv; p.G = G;
  p.nsplit = nsplit; p.split_tokens = split_tokens;
  p.row_tiles_max = (max_q_len * G + 15) / 16;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.num_blocks = pool->num_blocks;
  p.total_rows = (int64_t)total_q * Hq;
  const int items = p.row_tiles_max * nsplit;
  const dim3 grid(Hkv, num_seqs, (items + ATT_WARPS - 1) / ATT_WARPS);
  const size_t smem = ATT_WARPS * ATT_STAGES * ATT_STAGE_BYTES;
  static bool configured[DASER_MAX_DEVICES] = {false};  // per device: the attribute is the device's
  if (daser_first_use_on_device(configured)) {
    cudaError_t e = cudaFuncSetAttribute(paged_attn_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(paged_attn_fp8_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PF_SMEM);
    if (e != cudaSuccess) return (int)e;
  }
  if (attention_tc_enabled() && max_q_len * G >= 64 && 128 % G == 0) {
    // at least half of a 128-row MMA tile per KV head: the tcgen05 kernel
    const int rc = daser_launch_attention_tc(p, max_q_len, stream);
    if (rc != 0) return rc;
  } else if (p.row_tiles_max > 1) {
    // several row tiles per KV head: the CTA-shared dequantisation pays off
    const int groups = (p.row_tiles_max + 3) / 4;
    const dim3 pgrid(Hkv, num_seqs, groups * nsplit);
    launch_pdl(paged_attn_fp8_prefill_kernel, pgrid, dim3(128), (size_t)PF_SMEM, stream, p);
  } else {
    launch_pdl(paged_attn_fp8_kernel, grid, dim3(ATT_WARPS * 32), smem, stream, p);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  if (nsplit > 1) {
    const int64_t rows = (int64_t)total_q * Hq;
    launch_pdl(attn_merge_kernel, dim3((unsigned)((rows + 3) / 4)), dim3(128), 0, stream, (const float*)part_o,
               (const float*)part_lse, (__nv_bfloat16*)out, rows, nsplit);
    e = cudaGetLastError();
  }
  return (int)e;
}

// ---- allocation-free variant (see attention_noalloc.h) ------------------------------------------
#include "attention_noalloc.h"

namespace daser {
// Split-KV scratch that lives in the library image: partial outputs first, then the
// log-sum-exp values.  In host code this name is only a handle for cudaGetSymbolAddress.
static __device__ __align__(256) float g_noalloc_scratch[(size_t)DASER_NOALLOC_MAX_ROW_SPLITS * (ATT_D + 1)];

constexpr int kNoallocMaxDevices = 64;
static float* g_noalloc_ptr[kNoallocMaxDevices] = {nullptr};
}  // namespace daser

DASER_API int daser_paged_attention_fp8_noalloc(const void* q, void* out, const DaserKVPool* pool, int layer,
                                                int rank, const int32_t* block_tables, int max_blocks,
                                                const int32_t* q_start, const int32_t* ctx_lens, int num_seqs,
                                                int total_q, int max_q_len, int Hq, int Hkv, int head_dim,
                                                int block_tokens, int nsplit, int split_tokens,
                                                float softmax_scale, cudaStream_t stream) {
  using namespace daser;
  if (total_q < 0 || Hq <= 0 || nsplit < 1) return DASER_ERR_BAD_ARG;
  if ((int64_t)total_q * Hq * nsplit > DASER_NOALLOC_MAX_ROW_SPLITS) return DASER_ERR_TOO_LARGE;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kNoallocMaxDevices) return DASER_ERR_UNSUPPORTED;
  if (g_noalloc_ptr[dev] == nullptr) {
    // once per device, with that device current: the array's address on THIS device
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    if (p == nullptr) return DASER_ERR_UNSUPPORTED;
    g_noalloc_ptr[dev] = p;
  }
  float* part_o = g_noalloc_ptr[dev];
  float* part_lse = part_o + (size_t)DASER_NOALLOC_MAX_ROW_SPLITS * ATT_D;
  return daser_paged_attention_fp8(q, out, part_o, part_lse, pool, layer, rank, block_tables, max_blocks, q_start,
                                   ctx_lens, num_seqs, total_q, max_q_len, Hq, Hkv, head_dim, block_tokens, nsplit,
                                   split_tokens, softmax_scale, stream);
}
