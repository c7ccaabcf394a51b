// tcgen05 GEMM for the serving model: C[M,N] (+)= A[M,K] * B[N,K]^T, bf16 in, fp32 accumulate
// in tensor memory.  A is the activation matrix (row-major), B a Linear weight as PyTorch
// stores it ([out_features, in_features]), so both operands are K-major and go from global
// memory to 128-byte-swizzled shared memory with plain TMA tiled loads (each CTA fetches its own tiles).
//
// In the reference's serving stack these GEMMs are cuBLAS/CUTLASS calls inside stock vLLM
// (vllm/model_executor/layers/linear.py) followed, for the row-parallel layers, by a
// separate all-reduce; here the reduce-scatter is the epilogue of the same kernel.
//
// Work decomposition: grid = (n_tiles, m_tiles, k_splits); one 128 x BN output tile and one
// K range per CTA.  Serving GEMMs have few rows (a decode batch or a prompt tail), so the
// time is set by how fast the weights stream from HBM: split-K keeps all 148 SMs pulling
// even when N / BN is small.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner,
// warps 2..5 = epilogue (TMEM lane quarter = warp % 4).
//
// Epilogues:
//   EPI_STORE_BF16   C is bf16, k_splits must be 1.  With several owners this is the
//                    reduce-scatter's scatter half in bf16: rank s stores its partial rows
//                    into slot s of the owner's receive buffer ([slot][rows_per_owner][N],
//                    dst_row_offset = s * rows_per_owner) with plain 64-byte stores and bumps the
//                    owner's arrival counter; the owner's add + RMSNorm kernel sums the slots.
//                    With `bcast` the rows are not partitioned: every rank receives the whole
//                    partial (one-shot all-reduce; each rank then sums and normalises all rows
//                    itself, so no all-gather follows).  One NVLink hop instead of two, tp - 1
//                    times the bytes: the form for the few rows of a serving step.
//                    Half the NVLink bytes of the fp32 form and no atomics.
//   EPI_REDUCE_F32   C is fp32 and is accumulated with vector red.global.add; rows are
//                    partitioned over n_owners buffers (rows_per_owner each).  With one owner
//                    this is local split-K; with the owners being the tensor-parallel ranks'
//                    peer-mapped buffers it is GEMM -> reduce-scatter: every partial tile goes
//                    straight from TMEM over NVLink into the rank that owns those rows, and a
//                    per-owner arrival counter is bumped (release, system scope) once the
//                    CTA's contributions are out (one bump per CTA and owner).
//
//   EPI_SWIGLU_BF16  the gate/up projection with its activation: the weight rows of every BN-row
//                    tile are BN/2 gate rows followed by the BN/2 up rows of the same outputs
//                    (the loader interleaves them), so one CTA holds both halves in TMEM and
//                    stores silu(gate) * up as bf16 [M, N/2].  With split-K the partials are added
//                    into the fp32 work buffer and the CTA that completes a tile applies the
//                    activation (and hands the buffer back zeroed).
//   EPI_QKV_ROPE     the QKV projection with what follows it: BN = head_dim = 128, so a tile is one
//                    head of up to 128 tokens and an epilogue thread holds one token's head.  Query
//                    heads are rotated and stored as bf16, key heads rotated, value heads as they
//                    are, both quantised into the paged KV pool at the token's slot (rope.cuh: the
//                    same code the stand-alone kernel runs).  Unsplit, the values come straight from
//                    tensor memory; with split-K the partials are added into the fp32 work buffer
//                    and the CTA that completes a tile does the rest (and hands the buffer back zeroed).
//   EPI_SPLITK_SCATTER  split-K and the bf16 scatter in one kernel: every K split adds its
//                    partial tile into a local fp32 work buffer; the CTA that finishes a tile
//                    last (per-tile counter) reads the sum back, hands the work buffer back
//                    zeroed, and does the bf16 slot stores + arrival bumps of EPI_STORE_BF16.
//                    All SMs stream weights, yet only one bf16 copy of the tile crosses NVLink.
//
// Every wait is bounded; on a timeout the kernel records it in `status`, drains, frees its
// TMEM and returns.
#include <cuda.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "rope.cuh"
#include "tcgen05.cuh"

namespace daser {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;  // 64 bf16 = 128 B = one swizzle row
constexpr int GEMM_THREADS = 192;

enum { EPI_STORE_BF16 = 0, EPI_REDUCE_F32 = 1, EPI_SPLITK_SCATTER = 2, EPI_SWIGLU_BF16 = 3, EPI_QKV_ROPE = 4 };

struct GemmParams {
  int M, N, K;
  int k_splits;
  int epilogue;
  int n_owners;
  int rows_per_owner;
  int64_t ldc;
  int64_t dst_row_offset;  // added to the row inside the owner's buffer (bf16 store epilogue)
  int bcast;               // bf16 epilogues.  1: store every row to ALL n_owners buffers (one-shot all-reduce);
                           // 2: store every row to c[0] only (this rank's own buffer, which peers read
                           // through the switch) but still bump all n_owners arrival counters
  void* c[DASER_MAX_RANKS];
  uint32_t* arrive[DASER_MAX_RANKS];  // per-owner arrival counters (may be null)
  uint32_t* status;                   // [0] = timeout flag
  float* work;                        // EPI_SPLITK_SCATTER: local fp32 [M][work_ld], zero between GEMMs
  int64_t work_ld;
  uint32_t* tile_counters;            // EPI_SPLITK_SCATTER: one per output tile, zero between GEMMs
  // all-gather side: A rows [g*gate_rows, (g+1)*gate_rows) may be loaded once
  // gate_flags[g] >= gate_target + *gate_base (null flags = no gating; null base = 0).
  // The base lives in device memory so that a captured CUDA graph can be replayed while the
  // counters keep growing.
  const uint32_t* gate_flags;
  const uint32_t* gate_base;
  uint32_t gate_target;
  int gate_rows;
  RopeKvWrite rope;   // EPI_QKV_ROPE
  int rope_pool_fp8;
};

__device__ __forceinline__ void red_add_f32x4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

template <int BN, int STAGES>
struct GemmSmem {
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
  static constexpr int B_BYTES = BN * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  // full[STAGES], empty[STAGES], tmem_full, then the TMEM base word and the abort flag
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 1) * 8 + 16;
  static constexpr int DYNAMIC = TOTAL + 1024;  // slack to align the tiles to 1024 B
};

// FUSED: compiled with the epilogues that finish another operator's work (EPI_QKV_ROPE, and
// EPI_SWIGLU_BF16 under split-K).  They cost registers, so the plain GEMM is a separate instance.
template <int BN, int STAGES, bool FUSED = false>
__global__ void __launch_bounds__(GEMM_THREADS, (BN <= 128 ? 2 : 1))
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const GemmParams p) {
  using S = GemmSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full_bar = empty_bar + STAGES;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_full_bar + 1);
  volatile uint32_t* abort_flag = tmem_base_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BN;
  const int m0 = blockIdx.y * GEMM_BM;

  const int kb_total = (p.K + GEMM_BK - 1) / GEMM_BK;
  const int kb_per = (kb_total + p.k_splits - 1) / p.k_splits;
  const int kb_begin = blockIdx.z * kb_per;
  const int kb_end = min(kb_begin + kb_per, kb_total);
  const int num_kb = kb_end - kb_begin;
  if (num_kb <= 0) return;  // uniform across the CTA

  constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;  // power of two >= 32

  if (warp == 0 && lane == 0) {
    sm100::prefetch_tmap(&tmap_a);
    sm100::prefetch_tmap(&tmap_b);
    for (int s = 0; s < STAGES; ++s) {
      sm100::mbar_init(&full_bar[s], 1);
      sm100::mbar_init(&empty_bar[s], 1);
    }
    sm100::mbar_init(tmem_full_bar, 1);
    *abort_flag = 0u;
    sm100::mbar_init_fence();
  }
  if (warp == 1) {
    sm100::tmem_alloc(tmem_base_slot, TMEM_COLS);
    sm100::tmem_relinquish();
  }
  sm100::tc_fence_before();
  __syncthreads();
  sm100::tc_fence_after();
  // This CTA holds its tensor memory: the next kernel of the stream may be scheduled (it parks
  // in griddepcontrol.wait until this grid has completed).
  pdl_launch_dependents();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      bool ok = true;
      // Weights do not depend on the previous kernel (nor on the peers): start streaming the
      // first stages' B tiles at once, then wait for whatever produces A.
      const int pre = num_kb < STAGES ? num_kb : STAGES;
      for (int it = 0; it < pre; ++it) {
        uint8_t* b_dst = smem + it * S::STAGE_BYTES + S::A_BYTES;
        sm100::mbar_expect_tx(&full_bar[it], S::STAGE_BYTES);
        sm100::tma_load_2d(b_dst, &tmap_b, &full_bar[it], (kb_begin + it) * GEMM_BK, n0);
      }
      // Programmatic dependent launch: this grid may have started while the previous kernel
      // on the stream was still draining; its results are visible after this returns
      // (a no-op when launched without the attribute).
      asm volatile("griddepcontrol.wait;" ::: "memory");
      if (p.gate_flags != nullptr) {
        // all-gather gating: the rows of this m-tile come from one or more peers' pushes
        const int g0 = m0 / p.gate_rows;
        const int g1 = min(m0 + GEMM_BM - 1, p.M - 1) / p.gate_rows;
        const uint32_t want = p.gate_target + (p.gate_base ? *p.gate_base : 0u);
        for (int g = g0; g <= g1 && ok; ++g) {
          const uint64_t t0 = sm100::global_timer_ns();
          while ((int32_t)(ld_acquire_sys(p.gate_flags + g) - want) < 0) {
            if (*abort_flag || sm100::global_timer_ns() - t0 > DASER_WAIT_NS) { ok = false; *abort_flag = 1u; break; }
            __nanosleep(64);
          }
        }
      }
      int issued = pre;  // their B halves are in flight either way
      for (int it = 0; it < num_kb && ok; ++it) {
        const int s = it % STAGES;
        uint8_t* a_dst = smem + s * S::STAGE_BYTES;
        uint8_t* b_dst = a_dst + S::A_BYTES;
        const int k = (kb_begin + it) * GEMM_BK;
        if (it < pre) {
          sm100::tma_load_2d(a_dst, &tmap_a, &full_bar[s], k, m0);
          continue;
        }
        const uint32_t parity = ((it / STAGES) & 1) ^ 1;
        if (!sm100::mbar_wait(&empty_bar[s], parity, abort_flag)) { ok = false; break; }
        sm100::mbar_expect_tx(&full_bar[s], S::STAGE_BYTES);
        sm100::tma_load_2d(b_dst, &tmap_b, &full_bar[s], k, n0);
        sm100::tma_load_2d(a_dst, &tmap_a, &full_bar[s], k, m0);
        issued = it + 1;
      }
      if (!ok) {
        // Aborting: give the loads already in flight a bounded chance to land before the
        // CTA retires its shared memory.
        const int first = issued > STAGES ? issued - STAGES : 0;
        for (int it = first; it < issued; ++it) {
          const int s = it % STAGES;
          const uint64_t t0 = sm100::global_timer_ns();
          while (!sm100::mbar_try_wait(&full_bar[s], (it / STAGES) & 1))
            if (sm100::global_timer_ns() - t0 > 100000000ull) break;  // 100 ms
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (lane == 0) {
      constexpr uint32_t idesc = sm100::make_idesc_f16(GEMM_BM, BN, 1u);
      bool ok = true;
      for (int it = 0; it < num_kb; ++it) {
        const int s = it % STAGES;
        if (!sm100::mbar_wait(&full_bar[s], (it / STAGES) & 1, abort_flag)) { ok = false; break; }
        sm100::tc_fence_after();
        const uint32_t a_addr = sm100::smem_u32(smem + s * S::STAGE_BYTES);
        const uint32_t b_addr = a_addr + S::A_BYTES;
        const uint64_t da = sm100::make_desc_k_sw128(a_addr);
        const uint64_t db = sm100::make_desc_k_sw128(b_addr);
#pragma unroll
        for (int k = 0; k < GEMM_BK / 16; ++k) {
          // advancing 16 bf16 (32 B) along K inside the swizzle row: +2 in 16-byte units
          sm100::umma_f16(tmem_base, da + 2 * k, db + 2 * k, idesc, (it > 0 || k > 0) ? 1u : 0u);
        }
        sm100::umma_commit(&empty_bar[s]);  // frees the stage once the MMAs have read it
      }
      if (ok) sm100::umma_commit(tmem_full_bar);
    }
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int quarter = warp & 3;
    const bool ok = sm100::mbar_wait(tmem_full_bar, 0, abort_flag);
    sm100::tc_fence_after();
    if (ok) {
      const int row = m0 + quarter * 32 + lane;
      const bool row_ok = row < p.M;
      const int owner = row_ok ? row / p.rows_per_owner : 0;
      const int64_t local_row = row_ok ? row - (int64_t)owner * p.rows_per_owner : 0;
      const bool swiglu_split = FUSED && p.epilogue == EPI_SWIGLU_BF16 && p.k_splits > 1;
      if (p.epilogue == EPI_SWIGLU_BF16 && !swiglu_split) {
        if constexpr (BN >= 64) {
          // columns [0, BN/2) of the tile are gate, [BN/2, BN) the matching up values
#pragma unroll 1
          for (int c = 0; c < BN / 64; ++c) {
            uint32_t g[32], u[32];
            sm100::tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(c * 32), g);
            sm100::tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(BN / 2 + c * 32), u);
            sm100::tmem_ld_wait();
            if (!row_ok) continue;
            const int col0 = (n0 >> 1) + c * 32;  // output column
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.c[0]) + (int64_t)row * p.ldc + col0;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              if (2 * (col0 + v * 8) < p.N) {
                float o[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  const float gv = __uint_as_float(g[v * 8 + i]);
                  o[i] = gv / (1.f + __expf(-gv)) * __uint_as_float(u[v * 8 + i]);
                }
                uint4 w;
                w.x = pack_bf16x2(o[0], o[1]); w.y = pack_bf16x2(o[2], o[3]);
                w.z = pack_bf16x2(o[4], o[5]); w.w = pack_bf16x2(o[6], o[7]);
                *reinterpret_cast<uint4*>(dst + v * 8) = w;
              }
            }
          }
        }
      }
      const bool rope_split = FUSED && p.epilogue == EPI_QKV_ROPE && p.k_splits > 1;
      if (FUSED && p.epilogue == EPI_QKV_ROPE && !rope_split) {
        if constexpr (BN == 128 && FUSED) {
          const int hd = n0 / 128;
#pragma unroll 1
          for (int c = 0; c < 2; ++c) {
            // columns [32c, 32c + 32) and their rotary partners [64 + 32c, 64 + 32c + 32)
            uint32_t ra[32], rb[32];
            sm100::tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(c * 32), ra);
            sm100::tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(64 + c * 32), rb);
            sm100::tmem_ld_wait();
            if (!row_ok) continue;
#pragma unroll
            for (int jj = 0; jj < 2; ++jj) {
              float x1[16], x2[16];
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                x1[i] = __uint_as_float(ra[16 * jj + i]);
                x2[i] = __uint_as_float(rb[16 * jj + i]);
              }
              if (p.rope_pool_fp8) rope_kv_write_item<true>(p.rope, x1, x2, row, hd, 2 * c + jj);
              else rope_kv_write_item<false>(p.rope, x1, x2, row, hd, 2 * c + jj);
            }
          }
        }
      }
      const bool splitk_tail = p.epilogue == EPI_SPLITK_SCATTER || rope_split || swiglu_split;  // partials meet in `work`
      const int n_chunks = ((p.epilogue == EPI_SWIGLU_BF16 && !swiglu_split) || (p.epilogue == EPI_QKV_ROPE && !rope_split))
                               ? 0 : BN / 32;  // (those epilogues are done)
#pragma unroll 1
      for (int c = 0; c < n_chunks; ++c) {
        uint32_t r[32];
        sm100::tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(c * 32), r);
        sm100::tmem_ld_wait();
        if (!row_ok) continue;
        const int col0 = n0 + c * 32;
        if (p.epilogue == EPI_STORE_BF16) {
          uint4 o[4];
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            o[v].x = pack_bf16x2(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1]));
            o[v].y = pack_bf16x2(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]));
            o[v].z = pack_bf16x2(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]));
            o[v].w = pack_bf16x2(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]));
          }
          // one destination (the row's owner), or every rank's copy when broadcasting
          const int n_dst = p.bcast == 1 ? p.n_owners : 1;
          for (int d = 0; d < n_dst; ++d) {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.c[p.bcast == 1 ? d : (p.bcast ? 0 : owner)]) +
                                 ((p.bcast ? (int64_t)row : local_row) + p.dst_row_offset) * p.ldc + col0;
#pragma unroll
            for (int v = 0; v < 4; ++v)
              if (col0 + v * 8 < p.N) *reinterpret_cast<uint4*>(dst + v * 8) = o[v];
          }
        } else {
          float* dst = splitk_tail
                           ? p.work + (int64_t)row * p.work_ld + col0
                           : reinterpret_cast<float*>(p.c[owner]) + local_row * p.ldc + col0;
#pragma unroll
          for (int v = 0; v < 8; ++v) {
            if (col0 + v * 4 < p.N)
              red_add_f32x4(dst + v * 4, __uint_as_float(r[v * 4 + 0]), __uint_as_float(r[v * 4 + 1]),
                            __uint_as_float(r[v * 4 + 2]), __uint_as_float(r[v * 4 + 3]));
          }
        }
      }
      bool signal = p.arrive[0] != nullptr;
      if (splitk_tail) {
        // Which CTA completes this tile?  (uniform over the 128 epilogue threads: a named
        // barrier is safe here because `ok` is true for all of them or for none)
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        uint32_t* s_last = tmem_base_slot + 2;
        if (threadIdx.x == 64) {
          const int live = (kb_total + kb_per - 1) / kb_per;
          uint32_t* ctr = p.tile_counters + blockIdx.y * gridDim.x + blockIdx.x;
          const uint32_t old = atomicAdd(ctr, 1u);
          const bool last = old + 1u == (uint32_t)live;
          if (last) atomicExch(ctr, 0u);
          *s_last = last ? 1u : 0u;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        signal = signal && (*s_last != 0u);
        if (*s_last != 0u && rope_split) {
          __threadfence();
          if constexpr (BN == 128 && FUSED) {
            // the tile's sum is in `work` (L2): any thread may take any row, so the (row, group
            // pair) items are dealt over all 128 epilogue threads, not one row per thread
            const int hd = n0 / 128;
            const int rows_here = min(GEMM_BM, p.M - m0);
            const int et = threadIdx.x - 64;  // 0..127
#pragma unroll 1
            for (int item = et; item < rows_here * 4; item += 128) {
              const int r = m0 + (item >> 2), j = item & 3;
              float* s1 = p.work + (int64_t)r * p.work_ld + n0 + j * FP8_GROUP;
              float* s2 = s1 + 64;
              float x1[16], x2[16];
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                const float4 a = __ldcg(reinterpret_cast<const float4*>(s1 + 4 * v));
                const float4 b = __ldcg(reinterpret_cast<const float4*>(s2 + 4 * v));
                x1[4 * v] = a.x; x1[4 * v + 1] = a.y; x1[4 * v + 2] = a.z; x1[4 * v + 3] = a.w;
                x2[4 * v] = b.x; x2[4 * v + 1] = b.y; x2[4 * v + 2] = b.z; x2[4 * v + 3] = b.w;
              }
#pragma unroll
              for (int v = 0; v < 4; ++v) {  // the work buffer goes back zeroed
                *reinterpret_cast<float4*>(s1 + 4 * v) = make_float4(0.f, 0.f, 0.f, 0.f);
                *reinterpret_cast<float4*>(s2 + 4 * v) = make_float4(0.f, 0.f, 0.f, 0.f);
              }
              if (p.rope_pool_fp8) rope_kv_write_item<true>(p.rope, x1, x2, r, hd, j);
              else rope_kv_write_item<false>(p.rope, x1, x2, r, hd, j);
            }
          }
        } else if (*s_last != 0u && row_ok && swiglu_split) {
          __threadfence();
          if constexpr (BN >= 64 && FUSED) {
#pragma unroll 1
            for (int c = 0; c < BN / 64; ++c) {
              float* gs = p.work + (int64_t)row * p.work_ld + n0 + c * 32;  // gate columns of the tile
              float* us = gs + BN / 2;                                      // the matching up columns
              const int col0 = (n0 >> 1) + c * 32;                          // output column
              __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.c[0]) + (int64_t)row * p.ldc + col0;
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                if (2 * (col0 + v * 8) >= p.N) continue;
                const float4 g0 = __ldcg(reinterpret_cast<const float4*>(gs + v * 8));
                const float4 g1 = __ldcg(reinterpret_cast<const float4*>(gs + v * 8 + 4));
                const float4 u0 = __ldcg(reinterpret_cast<const float4*>(us + v * 8));
                const float4 u1 = __ldcg(reinterpret_cast<const float4*>(us + v * 8 + 4));
                *reinterpret_cast<float4*>(gs + v * 8) = make_float4(0.f, 0.f, 0.f, 0.f);
                *reinterpret_cast<float4*>(gs + v * 8 + 4) = make_float4(0.f, 0.f, 0.f, 0.f);
                *reinterpret_cast<float4*>(us + v * 8) = make_float4(0.f, 0.f, 0.f, 0.f);
                *reinterpret_cast<float4*>(us + v * 8 + 4) = make_float4(0.f, 0.f, 0.f, 0.f);
                const float gv[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
                const float uv[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
                float o[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i] = gv[i] / (1.f + __expf(-gv[i])) * uv[i];
                uint4 w;
                w.x = pack_bf16x2(o[0], o[1]); w.y = pack_bf16x2(o[2], o[3]);
                w.z = pack_bf16x2(o[4], o[5]); w.w = pack_bf16x2(o[6], o[7]);
                *reinterpret_cast<uint4*>(dst + v * 8) = w;
              }
            }
          }
        } else if (*s_last != 0u && row_ok) {
          __threadfence();
#pragma unroll 1
          for (int c = 0; c < BN / 32; ++c) {
            const int col0 = n0 + c * 32;
            float* src = p.work + (int64_t)row * p.work_ld + col0;
            // all loads of the chunk first (one L2 round trip), then the stores
            float4 t[8];
#pragma unroll
            for (int v = 0; v < 8; ++v)
              t[v] = (col0 + v * 4 < p.N) ? __ldcg(reinterpret_cast<const float4*>(src + v * 4))
                                          : make_float4(0.f, 0.f, 0.f, 0.f);
            uint4 o[4];
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              if (col0 + v * 8 < p.N) {
                *reinterpret_cast<float4*>(src + v * 8) = make_float4(0.f, 0.f, 0.f, 0.f);
                *reinterpret_cast<float4*>(src + v * 8 + 4) = make_float4(0.f, 0.f, 0.f, 0.f);
              }
              o[v].x = pack_bf16x2(t[2 * v].x, t[2 * v].y); o[v].y = pack_bf16x2(t[2 * v].z, t[2 * v].w);
              o[v].z = pack_bf16x2(t[2 * v + 1].x, t[2 * v + 1].y); o[v].w = pack_bf16x2(t[2 * v + 1].z, t[2 * v + 1].w);
            }
            const int n_dst = p.bcast == 1 ? p.n_owners : 1;
            for (int d = 0; d < n_dst; ++d) {
              __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.c[p.bcast == 1 ? d : (p.bcast ? 0 : owner)]) +
                                   ((p.bcast ? (int64_t)row : local_row) + p.dst_row_offset) * p.ldc + col0;
#pragma unroll
              for (int v = 0; v < 4; ++v)
                if (col0 + v * 8 < p.N) *reinterpret_cast<uint4*>(dst + v * 8) = o[v];
            }
          }
        }
      }
      if (p.arrive[0] != nullptr) {
        // The CTA's contributions are out: publish them, then bump every owner that the tile's
        // rows touch, once per CTA.  The barrier orders every epilogue thread's stores before
        // thread 64's fence, and a fence is cumulative, so one system-scope fence per CTA is
        // enough.  (The host derives the expected count per owner from the same rule.)
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (threadIdx.x == 64 && signal) {
          __threadfence_system();  // one release fence, then relaxed bumps (a release per bump would pay it again)
          const int o0 = p.bcast ? 0 : m0 / p.rows_per_owner;
          const int o1 = p.bcast ? p.n_owners - 1 : min(m0 + GEMM_BM - 1, p.M - 1) / p.rows_per_owner;
          for (int o = o0; o <= o1; ++o)
            asm volatile("red.relaxed.sys.global.add.u32 [%0], 1;" ::"l"(p.arrive[o]) : "memory");
        }
      }
    }
  }

  sm100::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    sm100::tc_fence_after();
    sm100::tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_flag && p.status != nullptr) atomicExch(p.status, DASER_STATUS_TIMEOUT);
}

// ---- host side -----------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// bf16 [rows, cols] row-major with leading dimension ld (elements): box = [box_rows, 64 cols], 128 B swizzle.
static int make_tmap(CUtensorMap* out, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows) {
  EncodeTiledFn fn = encode_tiled();
  if (!fn) return DASER_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld * 2) % 16) return DASER_ERR_BAD_ARG;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {(cuuint32_t)GEMM_BK, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : DASER_ERR_BAD_ARG;
}

static bool pdl_enabled() { return pdl_allowed(); }

template <int BN, int STAGES, bool FUSED = false>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, cudaStream_t stream) {
  using S = GemmSmem<BN, STAGES>;
  static bool configured[DASER_MAX_DEVICES] = {false};  // per device: the attribute is the device's
  if (daser_first_use_on_device(configured)) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, STAGES, FUSED>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, S::DYNAMIC);
    if (e != cudaSuccess) return (int)e;
  }
  const dim3 grid((p.N + BN - 1) / BN, (p.M + GEMM_BM - 1) / GEMM_BM, p.k_splits);
  // Programmatic dependent launch: CTAs of this grid may be scheduled while the previous
  // kernel's last CTAs drain; every role executes griddepcontrol.wait before it touches
  // anything the previous kernel wrote, and the weight prefetch runs ahead of that wait.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(GEMM_THREADS);
  cfg.dynamicSmemBytes = S::DYNAMIC;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, gemm_tcgen05_kernel<BN, STAGES, FUSED>, ta, tb, p);
}

}  // namespace daser

// C-callable description of one GEMM (mirrored with ctypes in daser_b200/ops/gemm.py).
typedef struct {
  const void* a;  // bf16 [M, K], leading dimension lda
  const void* b;  // bf16 [N, K], leading dimension ldb
  int64_t lda, ldb, ldc;
  int32_t M, N, K;
  int32_t block_n;   // 32, 64, 128 or 256
  int32_t k_splits;  // >= 1
  int32_t epilogue;  // 0 = bf16 store, 1 = fp32 red.add
  int32_t n_owners;  // output row partitions (1 = plain)
  int32_t rows_per_owner;
  int32_t dst_row_offset;
  void* c[DASER_MAX_RANKS];
  uint32_t* arrive[DASER_MAX_RANKS];
  uint32_t* status;
  const uint32_t* gate_flags;
  uint32_t gate_target;
  int32_t gate_rows;
  const uint32_t* gate_base;
  float* work;
  int64_t work_ld;
  uint32_t* tile_counters;
  int32_t bcast;  // 1: the bf16 epilogues store to every c[i] (row + dst_row_offset) and bump every arrive[i];
                  // 2: they store to c[0] only and bump every arrive[i] (the partial stays in this rank's
                  //    memory; peers fetch the sum with multimem.ld_reduce once all counters are up)
  // epilogue 4 (QKV projection + RoPE + paged KV write); N = (rope_hq + 2 * rope_hkv) * 128, block_n = 128
  const int32_t* rope_positions;
  const int64_t* rope_slot_mapping;
  const float* rope_cos_sin;
  void* rope_q_out;
  const DaserKVPool* rope_pool;
  int32_t rope_max_pos, rope_hq, rope_hkv, rope_block_tokens, rope_layer, rope_rank;
} DaserGemm;

DASER_API int daser_gemm(const DaserGemm* g, cudaStream_t stream) {
  using namespace daser;
  if (!g || g->M <= 0 || g->N <= 0 || g->K <= 0 || g->k_splits < 1) return DASER_ERR_BAD_ARG;
  if (g->K % 8 || g->N % 8) return DASER_ERR_UNSUPPORTED;
  if (g->epilogue == EPI_STORE_BF16 && g->k_splits != 1) return DASER_ERR_BAD_ARG;
  if (g->epilogue == EPI_SWIGLU_BF16 &&
      (g->block_n < 64 || g->N % g->block_n || g->n_owners != 1 ||
       (g->k_splits != 1 && (!g->work || !g->tile_counters)))) return DASER_ERR_BAD_ARG;
  if (g->epilogue == EPI_QKV_ROPE) {
    if (g->block_n != 128 || !g->rope_pool || !g->rope_positions || !g->rope_slot_mapping || !g->rope_cos_sin ||
        !g->rope_q_out || g->rope_max_pos <= 0 || g->rope_block_tokens <= 0) return DASER_ERR_BAD_ARG;
    if (g->N != (g->rope_hq + 2 * g->rope_hkv) * 128 || g->rope_rank < 0 || g->rope_rank >= DASER_MAX_RANKS)
      return DASER_ERR_BAD_ARG;
    if (g->k_splits > 1 && (!g->work || !g->tile_counters)) return DASER_ERR_BAD_ARG;
  }
  if (g->n_owners < 1 || g->n_owners > DASER_MAX_RANKS) return DASER_ERR_BAD_ARG;
  if (g->rows_per_owner <= 0 || (int64_t)g->rows_per_owner * g->n_owners < g->M) return DASER_ERR_BAD_ARG;
  if (g->gate_flags && g->gate_rows <= 0) return DASER_ERR_BAD_ARG;
  GemmParams p;
  p.M = g->M; p.N = g->N; p.K = g->K;
  p.k_splits = g->k_splits;
  p.epilogue = g->epilogue;
  p.n_owners = g->n_owners;
  p.rows_per_owner = g->rows_per_owner;
  p.ldc = g->ldc;
  p.dst_row_offset = g->dst_row_offset;
  p.bcast = g->bcast < 0 || g->bcast > 2 ? 1 : g->bcast;
  if (p.bcast && g->epilogue == EPI_REDUCE_F32) return DASER_ERR_BAD_ARG;
  for (int i = 0; i < DASER_MAX_RANKS; ++i) { p.c[i] = g->c[i]; p.arrive[i] = g->arrive[i]; }
  p.status = g->status;
  p.work = g->work;
  p.work_ld = g->work_ld;
  p.tile_counters = g->tile_counters;
  if (g->epilogue == EPI_SPLITK_SCATTER && (!g->work || !g->tile_counters)) return DASER_ERR_BAD_ARG;
  p.gate_flags = g->gate_flags;
  p.gate_target = g->gate_target;
  p.gate_base = g->gate_base;
  p.gate_rows = g->gate_rows > 0 ? g->gate_rows : 1;
  memset(&p.rope, 0, sizeof(p.rope));
  p.rope_pool_fp8 = 0;
  if (g->epilogue == EPI_QKV_ROPE) {
    p.rope.positions = g->rope_positions; p.rope.slot_mapping = g->rope_slot_mapping;
    p.rope.cos_sin = g->rope_cos_sin; p.rope.max_pos = g->rope_max_pos;
    p.rope.q_out = (__nv_bfloat16*)g->rope_q_out;
    p.rope.Hq = g->rope_hq; p.rope.Hkv = g->rope_hkv; p.rope.D = 128; p.rope.block_tokens = g->rope_block_tokens;
    p.rope.pool = *g->rope_pool; p.rope.layer = g->rope_layer; p.rope.rank = g->rope_rank;
    p.rope_pool_fp8 = g->rope_pool->pool_is_fp8;
  }
  CUtensorMap ta, tb;
  if (int e = make_tmap(&ta, g->a, g->M, g->K, g->lda, GEMM_BM)) return e;
  if (int e = make_tmap(&tb, g->b, g->N, g->K, g->ldb, g->block_n)) return e;
  const bool fused = g->epilogue == EPI_QKV_ROPE || (g->epilogue == EPI_SWIGLU_BF16 && g->k_splits > 1);
  if (fused) {
    if (g->block_n != 128) return DASER_ERR_UNSUPPORTED;
    return launch<128, 3, true>(ta, tb, p, stream);
  }
  switch (g->block_n) {
    // stage counts keep two CTAs resident per SM for BN <= 128 (<= ~100 KB each)
    case 32: return launch<32, 5>(ta, tb, p, stream);
    case 64: return launch<64, 4>(ta, tb, p, stream);
    case 128: return launch<128, 3>(ta, tb, p, stream);
    case 256: return launch<256, 4>(ta, tb, p, stream);
    default: return DASER_ERR_UNSUPPORTED;
  }
}
