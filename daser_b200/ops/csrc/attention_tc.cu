// Chunked-prefill paged attention on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// In the reference's serving stack the prefill of a RAG query over restored chunk KV is stock
// vLLM's FlashAttention kernel over a bf16 cache (vllm/v1/attention/backends/flash_attn.py).
// Here the cache is block-scaled fp8 and the query block is small (tens of tokens) while the
// context is thousands of keys, so the kernel is organised around one 128-row MMA tile:
//
//   * one CTA = 128 query rows of one KV head (128 / G query tokens x the G heads that share
//     the KV head) and one contiguous range of keys (split-KV; partials are merged by
//     attn_merge_kernel);
//   * keys are streamed in tiles of 64 (four 16-token pages): the raw fp8 pages and their
//     scales arrive through a two-stage cp.async ring, all 128 threads dequantise them to f16
//     straight into the 128-byte-swizzled K-major layout the MMA descriptors expect: K as
//     [key][dim], V transposed to [dim][key] so that both MMAs take K-major operands;
//   * S = Q K^T (M 128, N 64, K 128) is issued by one thread as eight tcgen05.mma into TMEM;
//     every thread then owns one row of S (tcgen05.ld 32x32b: lane = row), so the online
//     softmax needs no shuffles; P goes back to shared memory as f16 (over the K tile, which
//     is dead by then) and O_tile = P V (M 128, N 128, K 64) is four more tcgen05.mma;
//   * P = 2^(S - m) is computed two at a time in f16 (ex2.approx.f16x2) and is the MMA operand
//     as is; V^T carries one extra row of ones, so column 128 of the output accumulates the row
//     sums of exactly the P that was multiplied (no separate summation);
//   * the output accumulates in TMEM across tiles.  The running maximum m is only raised when
//     a tile exceeds it by more than 2^8 (the f16 P has the head-room), and only then is the
//     accumulator rescaled (tcgen05.ld / st); most tiles do not touch it.
//
// Two CTAs fit one SM (about 105 KB of shared memory, 256 TMEM columns and 128 threads each),
// which is what overlaps one CTA's softmax with the other's MMAs and copies.
// Every mbarrier wait is bounded; on expiry the CTA records it in a status word, frees its
// TMEM and returns.
#include "attention_params.cuh"
#include "tcgen05.cuh"

namespace daser {
using namespace sm100;

constexpr int TC_NK = 64;                        // keys per tile
constexpr int TC_PAGES = TC_NK / ATT_B;          // 4
constexpr int TC_Q_BYTES = 128 * ATT_D * 2;      // 32768: two sub-tiles [128 rows][64 dims]
constexpr int TC_KP_BYTES = 16384;               // K: two sub-tiles [64 keys][64 dims]; later P: [128 rows][64 keys]
constexpr int TC_ON = ATT_D + 16;                // output columns: 128 dims, the row sum, 15 unused
constexpr int TC_VT_BYTES = TC_ON * 128;         // V^T: [128 dims + 16][64 keys] = 18432
constexpr int TC_RAW_PAYLOAD = TC_PAGES * 4096;  // per page: K 2048 B, V 2048 B
constexpr int TC_RAW_KSCALE = TC_PAGES * 512;
constexpr int TC_RAW_VSCALE = TC_NK * 8 * 4;
constexpr int TC_RAW_BYTES = TC_RAW_PAYLOAD + TC_RAW_KSCALE + TC_RAW_VSCALE;  // 20480
constexpr int TC_SMEM = 1024 + TC_Q_BYTES + TC_KP_BYTES + TC_VT_BYTES + 2 * TC_RAW_BYTES + 64;
constexpr uint32_t TC_TMEM_COLS = 256;           // S in columns [0, 64), O in [64, 208)
constexpr uint32_t TC_O_COL = 64;
constexpr float TC_RESCALE_AT = 8.f;             // raise the running maximum only beyond this (log2)

__device__ uint32_t g_attn_tc_status = 0;        // bit 0: a bounded wait ran out

__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// {2^lo, 2^hi} as packed f16 (lo in the low half).
__device__ __forceinline__ uint32_t ex2_f16x2(float lo, float hi) {
  uint32_t r;
  asm("{\n\t.reg .b32 t;\n\t"
      "cvt.rn.f16x2.f32 t, %2, %1;\n\t"
      "ex2.approx.f16x2 %0, t;\n\t}\n"
      : "=r"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ float ex2_f32(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}

__global__ void __launch_bounds__(128, 2)
paged_attn_fp8_tc_kernel(const AttnParams p) {
  extern __shared__ uint8_t tc_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;
  uint8_t* kp_s = q_s + TC_Q_BYTES;
  uint8_t* vt_s = kp_s + TC_KP_BYTES;
  uint8_t* raw_s = vt_s + TC_VT_BYTES;
  uint64_t* bar_s = reinterpret_cast<uint64_t*>(raw_s + 2 * TC_RAW_BYTES);
  uint64_t* bar_o = bar_s + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_s + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int tid = threadIdx.x, warp = tid >> 5;
  const int kvh = blockIdx.x, seq = blockIdx.y;
  const int grp = blockIdx.z / p.nsplit, sp = blockIdx.z % p.nsplit;
  pdl_wait();  // launched ahead of its predecessor's end: nothing is read before this returns
  const int q0 = p.q_start[seq];
  const int q_len = p.q_start[seq + 1] - q0;
  const int ctx = p.ctx_lens[seq];
  const int G = p.G;
  const int toks_per_cta = 128 / G;
  const int grp_tok_first = grp * toks_per_cta;
  if (grp_tok_first >= q_len) return;  // uniform over the CTA
  const int grp_tok_last = min(grp_tok_first + toks_per_cta, q_len) - 1;
  const int grp_limit = ctx - q_len + grp_tok_last + 1;  // keys visible to the last row
  const int key_begin = sp * p.split_tokens;
  const int key_end = min(key_begin + p.split_tokens, grp_limit);
  const int n_tiles = key_begin < key_end ? (key_end - key_begin + TC_NK - 1) / TC_NK : 0;

  // this thread's row
  const int tq = grp_tok_first + tid / G;
  const int hq = kvh * G + tid % G;
  // rows beyond total_q (a q_start that names more rows than the buffers hold) are computed but never stored
  const bool valid = tq < q_len && ((int64_t)(q0 + tq) * p.Hq + hq) < p.total_rows;
  const int pos = ctx - q_len + tq;  // last key this row may see

  float m = -INFINITY;  // the maximum the accumulated P are relative to
  float l = 0.f;

  if (n_tiles > 0) {
    const uint32_t q_u32 = smem_u32(q_s), kp_u32 = smem_u32(kp_s), vt_u32 = smem_u32(vt_s), raw_u32 = smem_u32(raw_s);
    if (tid == 0) {
      mbar_init(bar_s, 1);
      mbar_init(bar_o, 1);
      *abort_flag = 0u;
      mbar_init_fence();
    }
    if (warp == 0) {
      tmem_alloc(tmem_slot, TC_TMEM_COLS);
      tmem_relinquish();
    }
    const int32_t* table = p.block_tables + (int64_t)seq * p.max_blocks;
    const int page_begin = key_begin / ATT_B;

    // Block ids are fetched one tile ahead of the copies that need them, so that the table
    // read (a dependent global load) is never on the critical path of a tile.
    int blk_next[TC_PAGES];
    auto fetch_blocks = [&](int ti) {
#pragma unroll
      for (int pg = 0; pg < TC_PAGES; ++pg)
        blk_next[pg] = __ldg(table + min(page_begin + ti * TC_PAGES + pg, p.max_blocks - 1));
    };
    auto issue = [&](int ti) {
      const uint32_t st = raw_u32 + (ti & 1) * TC_RAW_BYTES;
      const int key0 = key_begin + ti * TC_NK;
      int64_t base[TC_PAGES];
      bool live[TC_PAGES];
#pragma unroll
      for (int pg = 0; pg < TC_PAGES; ++pg) {
        live[pg] = key0 + pg * ATT_B < key_end;
        int blk = blk_next[pg];
        blk = blk < 0 ? 0 : (blk >= p.num_blocks ? p.num_blocks - 1 : blk);
        base[pg] = (int64_t)blk * p.stride_block + (int64_t)kvh * p.stride_head;
      }
      // payload: 4 pages x (K, V) x 128 pieces of 16 B.  The 16-byte chunk c of a token row is
      // stored at chunk (c ^ tok%8) for K and (c ^ key/8) for V, so that the dequantisation
      // below reads shared memory without bank conflicts.
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const int idx = tid + 128 * it;
        const int pg = idx >> 8, which = (idx >> 7) & 1, tok = (idx >> 3) & 15, c = idx & 7;
        if (!live[pg]) continue;
        const int kt = pg * ATT_B + tok;
        const int at = which ? (c ^ ((kt >> 3) & 7)) : (c ^ (tok & 7));
        const int64_t src = base[pg] + (which ? p.stride_kv : 0) + (int64_t)tok * p.stride_tok + c * 16;
        cp_async16(st + pg * 4096 + which * 2048 + tok * 128 + at * 16, p.kv_payload + src);
      }
      {  // K scales: [page][tok][8] as stored
        const int pg = tid >> 5, r = tid & 31, tok = r >> 1, hf = r & 1;
        int64_t b = base[0];
        bool lv = live[0];
#pragma unroll
        for (int x = 1; x < TC_PAGES; ++x)
          if (x == pg) { b = base[x]; lv = live[x]; }
        if (lv) {
          const int64_t soff = (b + (int64_t)tok * p.stride_tok) / 16 + hf * 4;
          cp_async16(st + TC_RAW_PAYLOAD + pg * 512 + r * 16, p.kv_scales + soff);
        }
      }
      // V scales: one word each, laid out [key % 8][group][key / 8]
#pragma unroll
      for (int it = 0; it < 4; ++it) {
        const int idx = tid + 128 * it;
        const int kt = idx >> 3, c = idx & 7, pg = kt >> 4, tok = kt & 15;
        if (!live[pg]) continue;
        const int64_t soff = (base[pg] + p.stride_kv + (int64_t)tok * p.stride_tok) / 16 + c;
        cp_async4(st + TC_RAW_PAYLOAD + TC_RAW_KSCALE + (((kt & 7) * 64 + c * 8 + (kt >> 3)) << 2), p.kv_scales + soff);
      }
    };
    fetch_blocks(0);
    issue(0);
    cp_async_commit();
    fetch_blocks(1);

    {  // Q row -> f16, pre-multiplied by scale * log2(e), into the swizzled A tile
      const __nv_bfloat16* qp = p.q + ((int64_t)(q0 + tq) * p.Hq + hq) * ATT_D;
#pragma unroll
      for (int ck = 0; ck < 16; ++ck) {
        uint4 w = make_uint4(0u, 0u, 0u, 0u);
        if (valid) w = *reinterpret_cast<const uint4*>(qp + ck * 8);
        uint4 h;
        h.x = pack_half2(bf16_lo(w.x) * p.scale_log2, bf16_hi(w.x) * p.scale_log2);
        h.y = pack_half2(bf16_lo(w.y) * p.scale_log2, bf16_hi(w.y) * p.scale_log2);
        h.z = pack_half2(bf16_lo(w.z) * p.scale_log2, bf16_hi(w.z) * p.scale_log2);
        h.w = pack_half2(bf16_lo(w.w) * p.scale_log2, bf16_hi(w.w) * p.scale_log2);
        *reinterpret_cast<uint4*>(q_s + (ck >> 3) * 16384 + tid * 128 + ((((ck & 7) ^ (tid & 7))) << 4)) = h;
      }
    }
    {  // rows 128..143 of V^T: row 128 all ones (it accumulates the row sums of P), the rest zero
      const uint32_t one2 = 0x3c003c00u;
      const uint32_t v = tid < 8 ? one2 : 0u;
      *reinterpret_cast<uint4*>(vt_s + ATT_D * 128 + tid * 16) = make_uint4(v, v, v, v);
    }
    tc_fence_before();
    __syncthreads();  // barriers initialised, TMEM address published
    tc_fence_after();
    pdl_launch_dependents();  // only now: this CTA holds its tensor memory, a successor cannot take it
    const uint32_t tmem = *tmem_slot;
    const uint32_t tmem_row = tmem + ((uint32_t)(warp * 32) << 16);
    constexpr uint32_t idesc_s = make_idesc_f16(128, TC_NK, 0);
    constexpr uint32_t idesc_o = make_idesc_f16(128, TC_ON, 0);
    int fail = 0;

    for (int ti = 0; ti < n_tiles; ++ti) {
      cp_async_wait<0>();
      if (__syncthreads_or(fail)) break;  // raw tile ti is in; K/P and V^T are free (PV of ti - 1 has completed)
      if (ti + 1 < n_tiles) issue(ti + 1);
      cp_async_commit();
      fetch_blocks(ti + 2);  // clamped to the table; used by the next iteration
      const uint8_t* st = raw_s + (ti & 1) * TC_RAW_BYTES;
      const int key0 = key_begin + ti * TC_NK;

      // ---- K: (key, 16-dim group) items, four per thread ----
#pragma unroll
      for (int rep = 0; rep < 4; ++rep) {
        const int item = tid + 128 * rep;
        const int kt = (item & 7) + 8 * (item >> 6), c = (item >> 3) & 7;
        const int pg = kt >> 4, tok = kt & 15;
        uint32_t h[8];
        if (key0 + kt < key_end) {
          const uint4 w = *reinterpret_cast<const uint4*>(st + pg * 4096 + tok * 128 + ((c ^ (tok & 7)) << 4));
          const float sc = reinterpret_cast<const float*>(st + TC_RAW_PAYLOAD + pg * 512)[tok * 8 + c];
          const uint32_t sc2 = pack_half2(sc, sc);
          const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            h[2 * i] = hmul2_u32(cvt_e4m3x2_f16x2((uint16_t)(ww[i] & 0xffffu)), sc2);
            h[2 * i + 1] = hmul2_u32(cvt_e4m3x2_f16x2((uint16_t)(ww[i] >> 16)), sc2);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) h[i] = 0u;
        }
        uint8_t* row = kp_s + (c >> 2) * 8192 + kt * 128;
        *reinterpret_cast<uint4*>(row + (((2 * (c & 3)) ^ (kt & 7)) << 4)) = make_uint4(h[0], h[1], h[2], h[3]);
        *reinterpret_cast<uint4*>(row + (((2 * (c & 3) + 1) ^ (kt & 7)) << 4)) = make_uint4(h[4], h[5], h[6], h[7]);
      }
      // ---- V^T: (8 keys, 4 dims) items, two per thread ----
#pragma unroll
      for (int rep = 0; rep < 2; ++rep) {
        const int item = tid + 128 * rep;
        const int ko = item & 7, dq = item >> 3, c = dq >> 2;
        const int pg = ko >> 1;
        uint32_t h01[8], h23[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int tok = 8 * (ko & 1) + i;
          if (key0 + 8 * ko + i < key_end) {
            const uint32_t w = *reinterpret_cast<const uint32_t*>(st + pg * 4096 + 2048 + tok * 128 + ((c ^ ko) << 4) + (dq & 3) * 4);
            const float sc = reinterpret_cast<const float*>(st + TC_RAW_PAYLOAD + TC_RAW_KSCALE)[i * 64 + c * 8 + ko];
            const uint32_t sc2 = pack_half2(sc, sc);
            h01[i] = hmul2_u32(cvt_e4m3x2_f16x2((uint16_t)(w & 0xffffu)), sc2);
            h23[i] = hmul2_u32(cvt_e4m3x2_f16x2((uint16_t)(w >> 16)), sc2);
          } else {
            h01[i] = 0u;
            h23[i] = 0u;
          }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t* src = (j < 2) ? h01 : h23;
          const uint32_t sel = (j & 1) ? 0x7632u : 0x5410u;
          const int d = 4 * dq + j;
          uint4 v;
          v.x = prmt(src[0], src[1], sel);
          v.y = prmt(src[2], src[3], sel);
          v.z = prmt(src[4], src[5], sel);
          v.w = prmt(src[6], src[7], sel);
          *reinterpret_cast<uint4*>(vt_s + d * 128 + ((ko ^ (d & 7)) << 4)) = v;
        }
      }
      fence_async_smem();
      tc_fence_before();
      __syncthreads();
      if (tid == 0 && !*abort_flag) {
        tc_fence_after();
#pragma unroll
        for (int sub = 0; sub < 2; ++sub) {
          const uint64_t da = make_desc_k_sw128(q_u32 + sub * 16384);
          const uint64_t db = make_desc_k_sw128(kp_u32 + sub * 8192);
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_f16(tmem, da + 2 * k, db + 2 * k, idesc_s, (sub | k) ? 1u : 0u);
        }
        umma_commit(bar_s);
      }
      if (!mbar_wait(bar_s, ti & 1, abort_flag)) fail = 1;
      __syncwarp();
      tc_fence_after();

      // ---- softmax on this thread's row ----
      {
        uint32_t sr[2][32];
        tmem_ld_32x32(tmem_row, sr[0]);
        tmem_ld_32x32(tmem_row + 32, sr[1]);
        tmem_ld_wait();
        if (!(valid && key0 + TC_NK - 1 <= pos && key0 + TC_NK <= key_end)) {
          // the causal edge or the end of the range runs through this tile
#pragma unroll
          for (int j = 0; j < TC_NK; ++j) {
            const int key = key0 + j;
            if (!(valid && key < key_end && key <= pos)) sr[j >> 5][j & 31] = 0xff800000u;  // -inf
          }
        }
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          mx0 = fmaxf(mx0, __uint_as_float(sr[0][j]));
          mx1 = fmaxf(mx1, __uint_as_float(sr[1][j]));
        }
        const float mx = fmaxf(mx0, mx1);
        // Raise m only when this tile is far above it: P then stays below 2^8, well inside f16.
        const bool raise = mx > m + TC_RESCALE_AT || (m == -INFINITY && mx > -INFINITY);
        if (ti > 0 && __any_sync(0xffffffffu, raise)) {
          // the previous P V has completed (its barrier was waited for before this tile's K was written)
          const float alpha = raise ? ex2_f32(m - mx) : 1.f;
#pragma unroll
          for (int cc = 0; cc < 5; ++cc) {
            uint32_t r[32];
            tmem_ld_32x32(tmem_row + TC_O_COL + 32 * cc, r);
            tmem_ld_wait();
#pragma unroll
            for (int x = 0; x < 32; ++x) r[x] = __float_as_uint(__uint_as_float(r[x]) * alpha);
            tmem_st_32x32(tmem_row + TC_O_COL + 32 * cc, r);
          }
          tmem_st_wait();
        }
        if (raise) m = mx;
        const float base = m == -INFINITY ? 0.f : m;
#pragma unroll
        for (int ck = 0; ck < 8; ++ck) {
          uint32_t h[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int j = ck * 8 + 2 * e;
            h[e] = ex2_f16x2(__uint_as_float(sr[j >> 5][j & 31]) - base, __uint_as_float(sr[(j + 1) >> 5][(j + 1) & 31]) - base);
          }
          *reinterpret_cast<uint4*>(kp_s + tid * 128 + ((ck ^ (tid & 7)) << 4)) = make_uint4(h[0], h[1], h[2], h[3]);
        }
      }
      fence_async_smem();
      tc_fence_before();
      __syncthreads();
      if (tid == 0 && !*abort_flag) {
        tc_fence_after();
        const uint64_t da = make_desc_k_sw128(kp_u32);
        const uint64_t db = make_desc_k_sw128(vt_u32);
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_f16(tmem + TC_O_COL, da + 2 * k, db + 2 * k, idesc_o, (ti | k) ? 1u : 0u);
        umma_commit(bar_o);
      }
      if (!mbar_wait(bar_o, ti & 1, abort_flag)) fail = 1;
      __syncwarp();
      tc_fence_after();
    }
    cp_async_wait<0>();
    const bool aborted = __syncthreads_or(fail) != 0;
    if (!aborted) {
      // ---- epilogue: O / l from TMEM (column 128 holds l).  The TMEM loads are warp-wide
      // (.sync.aligned): every thread executes them, only the global stores depend on `valid`.
      const int64_t row = (int64_t)(q0 + tq) * p.Hq + hq;
      uint32_t r[32];
      __syncwarp();
      tmem_ld_32x32(tmem_row + TC_O_COL + ATT_D, r);
      tmem_ld_wait();
      l = __uint_as_float(r[0]);
      const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        __syncwarp();  // reconverge after the predicated stores of the previous chunk
        tmem_ld_32x32(tmem_row + TC_O_COL + 32 * cc, r);
        tmem_ld_wait();
        if (!valid) continue;
        if (p.nsplit == 1) {
          __nv_bfloat16* dst = p.out + row * ATT_D + 32 * cc;
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(r[8 * x]) * inv, __uint_as_float(r[8 * x + 1]) * inv);
            w.y = pack_bf16x2(__uint_as_float(r[8 * x + 2]) * inv, __uint_as_float(r[8 * x + 3]) * inv);
            w.z = pack_bf16x2(__uint_as_float(r[8 * x + 4]) * inv, __uint_as_float(r[8 * x + 5]) * inv);
            w.w = pack_bf16x2(__uint_as_float(r[8 * x + 6]) * inv, __uint_as_float(r[8 * x + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + 8 * x) = w;
          }
        } else {
          float* dst = p.part_o + (row * p.nsplit + sp) * ATT_D + 32 * cc;
#pragma unroll
          for (int x = 0; x < 8; ++x)
            *reinterpret_cast<float4*>(dst + 4 * x) =
                make_float4(__uint_as_float(r[4 * x]) * inv, __uint_as_float(r[4 * x + 1]) * inv,
                            __uint_as_float(r[4 * x + 2]) * inv, __uint_as_float(r[4 * x + 3]) * inv);
        }
      }
      if (valid && p.nsplit > 1) p.part_lse[row * p.nsplit + sp] = l > 0.f ? m + log2f(l) : -INFINITY;
      __syncwarp();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, TC_TMEM_COLS);
    if (aborted && tid == 0) atomicOr(&g_attn_tc_status, 1u);
  } else if (valid) {
    // no keys in this split: an empty partial
    const int64_t row = (int64_t)(q0 + tq) * p.Hq + hq;
    if (p.nsplit == 1) {
      __nv_bfloat16* dst = p.out + row * ATT_D;
#pragma unroll
      for (int ck = 0; ck < 16; ++ck) *reinterpret_cast<uint4*>(dst + 8 * ck) = make_uint4(0u, 0u, 0u, 0u);
    } else {
      float* dst = p.part_o + (row * p.nsplit + sp) * ATT_D;
#pragma unroll
      for (int ck = 0; ck < 32; ++ck) *reinterpret_cast<float4*>(dst + 4 * ck) = make_float4(0.f, 0.f, 0.f, 0.f);
      p.part_lse[row * p.nsplit + sp] = -INFINITY;
    }
  }
}

}  // namespace daser

int daser_launch_attention_tc(const daser::AttnParams& p, int max_q_len, cudaStream_t stream) {
  using namespace daser;
  static bool configured[DASER_MAX_DEVICES] = {false};  // per device: the attribute is the device's
  if (daser_first_use_on_device(configured)) {
    cudaError_t e = cudaFuncSetAttribute(paged_attn_fp8_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM);
    if (e != cudaSuccess) return (int)e;
  }
  const int groups = (max_q_len * p.G + 127) / 128;
  const dim3 grid(p.Hkv, p.num_seqs, groups * p.nsplit);
  launch_pdl(paged_attn_fp8_tc_kernel, grid, dim3(128), TC_SMEM, stream, p);
  return (int)cudaGetLastError();
}

// Non-zero once any tensor-core attention CTA gave up on a bounded wait (synchronises the device).
DASER_API int daser_attention_tc_status(uint32_t* out) {
  uint32_t v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, daser::g_attn_tc_status, sizeof(v));
  if (out) *out = v;
  return (int)e;
}
