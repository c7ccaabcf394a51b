// Bandwidth-bound serving-model kernels: fused residual-add + RMSNorm, RoPE fused with
// the paged KV-cache write (bf16 or block-scaled fp8 pool), SwiGLU, embedding gather
// and greedy sampling.  In the reference these all come from stock vLLM (its _C fused
// add+rmsnorm, rotary and cache-write kernels); the reference itself has no GPU code.
//
// Inputs that come from a split-K / reduce-scatter GEMM are fp32 accumulators: the
// consumer reads them and, when asked, writes zeros back so the next GEMM can
// accumulate into the same buffer without a separate memset.
#include <string.h>

#include <stdlib.h>

#include "common.cuh"
#include "rope.cuh"
#include "kv_paged.h"

namespace daser {

template <typename T> struct Loader;
template <> struct Loader<__nv_bfloat16> {
  static __device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8], bool) {
    const uint4 a = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { v[2 * i] = bf16_lo(w[i]); v[2 * i + 1] = bf16_hi(w[i]); }
  }
};
template <> struct Loader<float> {
  static __device__ __forceinline__ void load8(float* p, float (&v)[8], bool zero_after) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    if (zero_after) {
      *reinterpret_cast<float4*>(p) = make_float4(0.f, 0.f, 0.f, 0.f);
      *reinterpret_cast<float4*>(p + 4) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
};

__device__ __forceinline__ void store8_bf16(__nv_bfloat16* p, const float (&v)[8]) {
  *reinterpret_cast<uint4*>(p) = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]),
                                            pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
}

struct OutList {
  __nv_bfloat16* ptr[DASER_MAX_RANKS];  // normalised rows go to each of these (peers for the all-gather push)
  int n;
};

// Cross-rank ordering of the sequence-parallel add + RMSNorm (all pointers may be null):
//   wait_counter / wait_target : arrivals of the reduce-scattered partials this rank must see
//                                before it reads its accumulator rows (bumped by the GEMM epilogues
//                                of every rank);
//   done_counter / done_target : local count of finished CTAs; the CTA that completes it
//   signal[0..n_signal)        : bumps each rank's "rows of rank r have landed" flag, which gates
//                                the TMA loads of the next column-parallel GEMM there.
struct TpSync {
  const uint32_t* wait_counter;
  uint32_t wait_target;   // plus *wait_base when that is set
  uint32_t* done_counter;
  uint32_t done_target;   // plus *done_base when that is set
  const uint32_t* wait_base;
  const uint32_t* done_base;
  uint32_t* signal[DASER_MAX_RANKS];
  int n_signal;
  uint32_t* status;
  // NVLink multicast alias of x (bf16 only, may be null): when set, the row's values are the SUM
  // over every rank's buffer at the same offset, fetched with multimem.ld_reduce (the switch
  // adds the ranks' partials in flight); x itself is not read and n_partials is ignored
  const __nv_bfloat16* mc_x;
};

// Sum over all ranks of the 8 bf16 values at the same offset of a multicast-bound buffer, added in
// fp32 inside the switch.  Only after the arrival counter said that every rank's partial is in its
// own memory (acquire by thread 0, then the CTA barrier).
__device__ __forceinline__ void multimem_sum8(const __nv_bfloat16* mc, float (&v)[8]) {
  uint32_t w[4];
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3])
               : "l"(mc)
               : "memory");
#pragma unroll
  for (int i = 0; i < 4; ++i) { v[2 * i] = bf16_lo(w[i]); v[2 * i + 1] = bf16_hi(w[i]); }
}

__device__ __forceinline__ uint64_t ew_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint32_t ew_ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
#ifndef DASER_WAIT_NS
#define DASER_WAIT_NS 2000000000ull
#endif

// out = rmsnorm(x [+ residual]) * weight ; residual <- x + residual.
// One CTA per row; each thread keeps ITERS fragments of 8 values in registers
// (hidden <= 8 * ITERS * blockDim), so the row is read from memory once.  Two shapes: 256
// threads with several fragments each when there are rows enough to fill the GPU (bandwidth
// bound), and up to 1024 threads with one fragment each when there are only a few rows (a
// token block of a serving step: latency bound, so every load of the row is in flight at once).
// MC: the row is read as the in-switch sum over ranks (sync.mc_x) instead of from x.
template <typename TIn, int ITERS, int MAXT, bool MC = false>
__global__ void __launch_bounds__(MAXT)
add_rmsnorm_kernel(TIn* __restrict__ x, __nv_bfloat16* __restrict__ residual,
                   const __nv_bfloat16* __restrict__ weight, OutList out, int64_t out_row_offset,
                   int hidden, float eps, int zero_after, TpSync sync, int n_partials, int64_t partial_stride) {
  __shared__ float s_part[32];
  __shared__ int s_ok;
  pdl_enter();
  const int64_t row = blockIdx.x;
  if (sync.wait_counter != nullptr) {
    // bounded wait for the other ranks' partial sums (a second or two, never for ever)
    if (threadIdx.x == 0) {
      int ok = 1;
      const uint64_t t0 = ew_timer_ns();
      const uint32_t want = sync.wait_target + (sync.wait_base ? *sync.wait_base : 0u);
      while ((int32_t)(ew_ld_acquire_sys(sync.wait_counter) - want) < 0) {
        if (ew_timer_ns() - t0 > DASER_WAIT_NS) { ok = 0; break; }
        __nanosleep(32);
      }
      if (!ok && sync.status) atomicExch(sync.status, DASER_STATUS_TIMEOUT);
      s_ok = ok;
    }
    __syncthreads();
    // on a timeout the rows are still processed (from whatever arrived) so that peers are
    // signalled and nobody downstream waits on this rank; the status word marks the step invalid
  }
  TIn* xr = x + row * hidden;
  __nv_bfloat16* rr = residual ? residual + row * hidden : nullptr;
  float v[ITERS][8];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int c = (it * blockDim.x + threadIdx.x) * 8;
    if (c < hidden) {
      if (MC) multimem_sum8(sync.mc_x + row * hidden + c, v[it]);
      else Loader<TIn>::load8(const_cast<TIn*>(xr) + c, v[it], zero_after != 0);
      // reduce-scatter, bf16 form: x holds one slot of partial rows per source rank
      for (int pt = 1; pt < (MC ? 1 : n_partials); ++pt) {
        float t[8];
        Loader<TIn>::load8(const_cast<TIn*>(xr) + pt * partial_stride + c, t, false);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[it][i] += t[i];
      }
      if (rr) {
        float r[8];
        Loader<__nv_bfloat16>::load8(rr + c, r, false);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[it][i] += r[i];
        // the residual stream is kept in bf16: normalise what the next layer will read
        store8_bf16(rr + c, v[it]);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[it][i] = __bfloat162float(__float2bfloat16(v[it][i]));
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += v[it][i] * v[it][i];
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? s_part[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) s_part[0] = rsqrtf(t / (float)hidden + eps);
  }
  __syncthreads();
  const float inv = s_part[0];
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int c = (it * blockDim.x + threadIdx.x) * 8;
    if (c < hidden) {
      float w[8], o[8];
      Loader<__nv_bfloat16>::load8(weight + c, w, false);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = v[it][i] * inv * w[i];
      for (int k = 0; k < out.n; ++k) store8_bf16(out.ptr[k] + (out_row_offset + row) * hidden + c, o);
    }
  }
  if (sync.done_counter != nullptr) {
    __threadfence_system();  // this CTA's pushes are visible system-wide before it is counted
    __syncthreads();
    if (threadIdx.x == 0) {
      const uint32_t prev = atomicAdd(sync.done_counter, 1u);
      if (prev + 1u == sync.done_target + (sync.done_base ? *sync.done_base : 0u)) {
        __threadfence_system();  // acquire side of the CTA count, release side of the signals
        for (int k = 0; k < sync.n_signal; ++k)
          asm volatile("red.relaxed.sys.global.add.u32 [%0], 1;" ::"l"(sync.signal[k]) : "memory");
      }
    }
  }
}

// epochs[i] += delta[i]: run at the end of a tensor-parallel forward so that the next
// forward (or the next replay of the same captured graph) waits for fresh arrivals.
__global__ void advance_epochs_kernel(uint32_t* epochs, uint32_t d0, uint32_t d1, uint32_t d2) {
  pdl_enter();
  epochs[0] += d0;
  epochs[1] += d1;
  epochs[2] += d2;
}

// Bounded wait until every flags[i] >= target (one thread); records a timeout in status.
__global__ void wait_flags_kernel(const uint32_t* flags, int n, uint32_t target, const uint32_t* base,
                                  uint32_t* status) {
  const uint64_t t0 = ew_timer_ns();
  const uint32_t want = target + (base ? *base : 0u);
  for (int i = 0; i < n; ++i) {
    while ((int32_t)(ew_ld_acquire_sys(flags + i) - want) < 0) {
      if (ew_timer_ns() - t0 > DASER_WAIT_NS) {
        if (status) atomicExch(status, DASER_STATUS_TIMEOUT);
        return;
      }
      __nanosleep(64);
    }
  }
}

// One thread per target: make everything this stream wrote before (peer memory included) visible
// system-wide, then publish `value` in the target's flag.  The flags of one writer only ever grow.
struct SignalTargets {
  uint32_t* flag[DASER_MAX_RANKS];
};
__global__ void signal_flags_kernel(SignalTargets targets, int n, uint32_t value) {
  const int i = threadIdx.x;
  if (i >= n || targets.flag[i] == nullptr) return;
  __threadfence_system();
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(targets.flag[i]), "r"(value) : "memory");
}

// Tensor-parallel sampling in one kernel.  Every rank holds, per row, the best (value, global
// vocabulary index) of its shard; the sample is the best over the ranks.  This rank's candidates
// go into every rank's table by peer stores, an arrival is published in every rank's counter, the
// kernel waits (bounded) until its own counter shows all `tp` arrivals of this exchange and picks.
// Table of a rank: [2 rounds][tp sources][2: value, index bits][cap] floats; rounds alternate so
// that a fast rank's next push cannot land on candidates a slow rank has not read yet.  `epoch`
// (device word, local) counts the arrivals consumed so far: the kernel can be replayed.
struct CandTargets {
  float* table[DASER_MAX_RANKS];
  uint32_t* counter[DASER_MAX_RANKS];
};
__global__ void __launch_bounds__(256)
tp_pick_token_kernel(const float* best_val, const int32_t* best_idx, int n, int rank,
                     int tp, int cap, CandTargets tg, uint32_t* epoch, uint32_t* status, int32_t* out_idx) {
  __shared__ uint32_t base_s;
  __shared__ int ok_s;
  if (threadIdx.x == 0) { base_s = *epoch; ok_s = 1; }
  __syncthreads();
  const uint32_t base = base_s;
  const int round = (base / (uint32_t)tp) & 1;
  for (int i = threadIdx.x; i < n * tp; i += blockDim.x) {
    const int r = i / n, j = i - r * n;
    float* dst = tg.table[r] + (size_t)(round * tp + rank) * 2 * cap;
    dst[j] = best_val[j];
    dst[cap + j] = __int_as_float(best_idx[j]);
  }
  __threadfence_system();
  __syncthreads();
  if ((int)threadIdx.x < tp)
    asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(tg.counter[threadIdx.x]) : "memory");
  if (threadIdx.x == 0) {
    const uint64_t t0 = ew_timer_ns();
    const uint32_t want = base + (uint32_t)tp;
    while ((int32_t)(ew_ld_acquire_sys(tg.counter[rank]) - want) < 0) {
      if (ew_timer_ns() - t0 > DASER_WAIT_NS) {
        if (status) atomicExch(status, DASER_STATUS_TIMEOUT);
        ok_s = 0;
        break;
      }
      __nanosleep(64);
    }
  }
  __syncthreads();
  if (ok_s) {
    for (int j = threadIdx.x; j < n; j += blockDim.x) {
      float best = 0.f;
      int idx = 0;
      for (int r = 0; r < tp; ++r) {
        const float* src = tg.table[rank] + (size_t)(round * tp + r) * 2 * cap;
        float v, ib;
        asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(src + j) : "memory");
        asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(ib) : "l"(src + cap + j) : "memory");
        if (r == 0 || v > best) { best = v; idx = __float_as_int(ib); }  // ties: the lowest rank
      }
      out_idx[j] = idx;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) *epoch = base + (uint32_t)tp;
}

// RoPE on q and k, then k/v into the paged pool.  qkv row = [Hq*D | Hkv*D | Hkv*D].
// slot_mapping[t] = block * block_tokens + offset inside the block, or < 0 to skip the write.
// QKNORM (Qwen3 family): every query and key head is RMS-normalised over head_dim and scaled by
// q_norm_w / k_norm_w before the rotation.  A head's `segs` items sit on consecutive lanes of one
// warp (segs is a power of two <= 32, the item stride is a multiple of the block size), so the sum
// of squares is a butterfly over those lanes only; all of them are inside the loop together.
template <typename TIn, bool POOL_FP8, bool QKNORM = false>
__global__ void __launch_bounds__(128)
rope_kv_write_kernel(TIn* __restrict__ qkv, int64_t qkv_stride, const int32_t* __restrict__ positions,
                     const int64_t* __restrict__ slot_mapping, const float* __restrict__ cos_sin,
                     int max_pos, __nv_bfloat16* __restrict__ q_out, int T, int Hq, int Hkv, int D,
                     int block_tokens, DaserKVPool pool, int layer, int rank, int zero_after,
                     const __nv_bfloat16* __restrict__ q_norm_w = nullptr,
                     const __nv_bfloat16* __restrict__ k_norm_w = nullptr, float norm_eps = 0.f) {
  pdl_enter();
  const int half = D >> 1;
  const int segs = half / FP8_GROUP;
  const int heads = Hq + 2 * Hkv;
  const int64_t total = (int64_t)T * heads * segs;
  for (int64_t item = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; item < total;
       item += (int64_t)gridDim.x * blockDim.x) {
    const int j = item % segs;
    const int hd = (item / segs) % heads;
    const int t = item / ((int64_t)segs * heads);
    TIn* src = qkv + (int64_t)t * qkv_stride + (int64_t)hd * D + j * FP8_GROUP;
    float x1[16], x2[16];
    {
      float a[8], b[8];
      Loader<TIn>::load8(src, a, zero_after != 0);
      Loader<TIn>::load8(src + 8, b, zero_after != 0);
#pragma unroll
      for (int i = 0; i < 8; ++i) { x1[i] = a[i]; x1[8 + i] = b[i]; }
      Loader<TIn>::load8(src + half, a, zero_after != 0);
      Loader<TIn>::load8(src + half + 8, b, zero_after != 0);
#pragma unroll
      for (int i = 0; i < 8; ++i) { x2[i] = a[i]; x2[8 + i] = b[i]; }
    }
    const bool is_v = hd >= Hq + Hkv;
    if (QKNORM && !is_v) {
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) ss += x1[i] * x1[i] + x2[i] * x2[i];
      const unsigned lane = threadIdx.x & 31u;
      const unsigned group = (segs >= 32 ? 0xFFFFFFFFu : ((1u << segs) - 1u) << (lane & ~(unsigned)(segs - 1)));
      for (int m = segs >> 1; m > 0; m >>= 1) ss += __shfl_xor_sync(group, ss, m);
      const float inv = rsqrtf(ss / (float)D + norm_eps);
      const __nv_bfloat16* w = (hd < Hq ? q_norm_w : k_norm_w) + j * FP8_GROUP;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        // the normalised head is a bf16 tensor in the models this follows: round before rotating
        x1[i] = __bfloat162float(__float2bfloat16(x1[i] * inv * __bfloat162float(w[i])));
        x2[i] = __bfloat162float(__float2bfloat16(x2[i] * inv * __bfloat162float(w[half + i])));
      }
    }
    RopeKvWrite r;
    r.positions = positions; r.slot_mapping = slot_mapping; r.cos_sin = cos_sin; r.max_pos = max_pos;
    r.q_out = q_out; r.Hq = Hq; r.Hkv = Hkv; r.D = D; r.block_tokens = block_tokens;
    r.pool = pool; r.layer = layer; r.rank = rank;
    rope_kv_write_item<POOL_FP8>(r, x1, x2, t, hd, j);
  }
}

// y[t, i] = silu(gate[t, i]) * up[t, i].  x rows are [gate | up] (block = 0), or blocks of `block`
// gate values followed by the matching up values (the row order the fused GEMM epilogue uses).
template <typename TIn>
__global__ void __launch_bounds__(256)
swiglu_kernel(TIn* __restrict__ x, __nv_bfloat16* __restrict__ y, int64_t T, int inter, int zero_after, int block) {
  pdl_enter();
  const int64_t total = T * (inter / 8);
  for (int64_t item = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; item < total;
       item += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = item / (inter / 8);
    const int c = (int)(item % (inter / 8)) * 8;
    float g[8], u[8], o[8];
    const int gcol = block ? (c / block) * 2 * block + c % block : c;
    const int ucol = block ? gcol + block : inter + c;
    Loader<TIn>::load8(x + t * 2 * inter + gcol, g, zero_after != 0);
    Loader<TIn>::load8(x + t * 2 * inter + ucol, u, zero_after != 0);
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = g[i] / (1.f + __expf(-g[i])) * u[i];
    store8_bf16(y + t * inter + c, o);
  }
}

__global__ void __launch_bounds__(256)
embedding_kernel(const int32_t* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                 __nv_bfloat16* __restrict__ out, int64_t T, int hidden, int vocab_begin, int vocab_count) {
  pdl_enter();
  const int64_t total = T * (hidden / 8);
  for (int64_t item = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; item < total;
       item += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = item / (hidden / 8);
    const int c = (int)(item % (hidden / 8)) * 8;
    const int id = ids[t] - vocab_begin;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (id >= 0 && id < vocab_count) v = *reinterpret_cast<const uint4*>(table + (int64_t)id * hidden + c);
    *reinterpret_cast<uint4*>(out + t * hidden + c) = v;
  }
}

// Standard Gumbel noise from a counter-based hash of (seed, vocabulary index): the same index gets
// the same noise on whichever rank holds it, and no generator state is kept.
__device__ __forceinline__ float gumbel_noise(uint64_t seed, uint32_t index) {
  uint64_t z = seed + 0x9E3779B97F4A7C15ull * ((uint64_t)index + 1ull);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  // 23 random bits + 0.5: every value is exact in fp32 and strictly inside (0, 1), so both logs are finite
  const float u = ((float)(uint32_t)(z >> 41) + 0.5f) * (1.0f / 8388608.0f);
  return -__logf(-__logf(u));
}

// Greedy sampling: argmax over a row of logits; packs (value, index) so ties pick the lowest index.
// GUMBEL: temperature sampling by the Gumbel-max rule.  argmax_i(logit_i / T + g_i) with independent
// standard Gumbel g_i is a draw from softmax(logits / T), and a maximum composes across vocabulary
// shards, so tensor-parallel ranks sample exactly by exchanging their (value, index) candidates as
// they do for greedy.  inv_temp[row] == 0 leaves that row greedy.
template <typename TIn, bool GUMBEL = false>
__global__ void __launch_bounds__(1024)
argmax_kernel(TIn* __restrict__ logits, int64_t stride, int n, int index_offset,
              float* __restrict__ best_val, int32_t* __restrict__ best_idx, int zero_after,
              const float* __restrict__ inv_temp = nullptr, const uint64_t* __restrict__ seeds = nullptr) {
  __shared__ float s_v[32];
  __shared__ int s_i[32];
  TIn* row = logits + blockIdx.x * stride;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  const float it = GUMBEL ? inv_temp[blockIdx.x] : 0.f;
  const uint64_t seed = GUMBEL ? seeds[blockIdx.x] : 0ull;
  for (int c = threadIdx.x * 8; c < n; c += blockDim.x * 8) {
    float v[8];
    Loader<TIn>::load8(row + c, v, zero_after != 0);
    if (GUMBEL && it > 0.f) {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = v[i] * it + gumbel_noise(seed, (uint32_t)(c + i + index_offset));
    }
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (c + i < n && (v[i] > bv)) { bv = v[i]; bi = c + i; }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { s_v[threadIdx.x >> 5] = bv; s_i[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int nw = blockDim.x >> 5;
    bv = threadIdx.x < nw ? s_v[threadIdx.x] : -INFINITY;
    bi = threadIdx.x < nw ? s_i[threadIdx.x] : 0x7fffffff;
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (threadIdx.x == 0) { best_val[blockIdx.x] = bv; best_idx[blockIdx.x] = bi + index_offset; }
  }
}

static int ew_grid(int64_t items, int threads) {
  int64_t b = (items + threads - 1) / threads;
  const int64_t cap = 148 * 16;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace daser

// Mirrored with ctypes (ops/elementwise.py).
typedef struct {
  const uint32_t* wait_counter;
  uint32_t wait_target;
  uint32_t* done_counter;
  uint32_t done_target;
  uint32_t* signal[DASER_MAX_RANKS];
  int32_t n_signal;
  uint32_t* status;
  const uint32_t* wait_base;
  const uint32_t* done_base;
  const void* mc_x;  // multicast alias of x: rows are read as the sum over ranks (bf16 x only)
} DaserTpSync;

DASER_API int daser_add_rmsnorm_tp(void* x, int x_is_fp32, void* residual, const void* weight,
                                   void* const* out_ptrs, int n_out, int64_t out_row_offset,
                                   int64_t rows, int hidden, float eps, int zero_after,
                                   const DaserTpSync* tp, int n_partials, int64_t partial_stride,
                                   cudaStream_t stream) {
  using namespace daser;
  if (rows < 0 || hidden <= 0 || hidden % 8 || n_out < 1 || n_out > DASER_MAX_RANKS) return DASER_ERR_BAD_ARG;
  if (rows == 0) return 0;
  int threads = ((hidden / 8 + 31) / 32) * 32;
  // measured kernel time, hidden 8192, fp32 input: 64 rows 10.7 us wide / 13.3 us narrow,
  // 128 rows 12.4 / 19.4, 512 rows 47 / 40: wide while one wave of CTAs covers the rows
  const bool few_rows = rows <= 148;
  const int max_threads = few_rows ? 1024 : 256;
  if (threads > max_threads) threads = max_threads;
  const int iters = (hidden / 8 + threads - 1) / threads;
  if (iters > 16) return DASER_ERR_TOO_LARGE;
  OutList out;
  out.n = n_out;
  for (int i = 0; i < n_out; ++i) out.ptr[i] = (__nv_bfloat16*)out_ptrs[i];
  TpSync sync;
  memset(&sync, 0, sizeof(sync));
  if (tp != nullptr) {
    if (tp->n_signal < 0 || tp->n_signal > DASER_MAX_RANKS) return DASER_ERR_BAD_ARG;
    sync.wait_counter = tp->wait_counter; sync.wait_target = tp->wait_target;
    sync.done_counter = tp->done_counter; sync.done_target = tp->done_target;
    sync.n_signal = tp->n_signal; sync.status = tp->status;
    sync.wait_base = tp->wait_base; sync.done_base = tp->done_base;
    if (tp->mc_x != nullptr && (x_is_fp32 || ((uintptr_t)tp->mc_x & 15))) return DASER_ERR_BAD_ARG;
    sync.mc_x = (const __nv_bfloat16*)tp->mc_x;
    for (int i = 0; i < tp->n_signal; ++i) sync.signal[i] = tp->signal[i];
  }
#define NORM_LAUNCH(TIN, IT, MAXT)                                                                    \
  launch_pdl(add_rmsnorm_kernel<TIN, IT, MAXT>, dim3((unsigned)rows), dim3(threads), 0, stream,         \
      (TIN*)x, (__nv_bfloat16*)residual, (const __nv_bfloat16*)weight, out, out_row_offset, hidden, eps, \
      x_is_fp32 ? zero_after : 0, sync, n_partials < 1 ? 1 : n_partials, partial_stride)
#define NORM_DISPATCH(TIN)                                                  \
  if (few_rows && iters <= 1) NORM_LAUNCH(TIN, 1, 1024);                    \
  else if (few_rows && iters <= 2) NORM_LAUNCH(TIN, 2, 1024);               \
  else if (iters <= 1) NORM_LAUNCH(TIN, 1, 256);                            \
  else if (iters <= 2) NORM_LAUNCH(TIN, 2, 256);                            \
  else if (iters <= 4) NORM_LAUNCH(TIN, 4, 256);                            \
  else if (iters <= 8) NORM_LAUNCH(TIN, 8, 256);                            \
  else NORM_LAUNCH(TIN, 16, 256)
  if (sync.mc_x != nullptr) {
    // in-switch sum: bf16 only, and only the shapes a serving step has (rows of up to 16k values)
    if (iters > 2) return DASER_ERR_TOO_LARGE;
#define NORM_LAUNCH_MC(IT, MAXT)                                                                             \
  launch_pdl(add_rmsnorm_kernel<__nv_bfloat16, IT, MAXT, true>, dim3((unsigned)rows), dim3(threads), 0, stream, \
      (__nv_bfloat16*)x, (__nv_bfloat16*)residual, (const __nv_bfloat16*)weight, out, out_row_offset, hidden, \
      eps, 0, sync, 1, (int64_t)0)
    if (few_rows && iters <= 1) NORM_LAUNCH_MC(1, 1024);
    else if (few_rows) NORM_LAUNCH_MC(2, 1024);
    else if (iters <= 1) NORM_LAUNCH_MC(1, 256);
    else NORM_LAUNCH_MC(2, 256);
#undef NORM_LAUNCH_MC
  } else if (x_is_fp32) { NORM_DISPATCH(float); } else { NORM_DISPATCH(__nv_bfloat16); }
#undef NORM_DISPATCH
#undef NORM_LAUNCH
  return (int)cudaGetLastError();
}

// x: bf16 (x_is_fp32 = 0) or fp32 accumulators (x_is_fp32 = 1, zeroed after the read when
// zero_after != 0).  out_ptrs[0..n_out) each receive the normalised rows at row offset
// out_row_offset (the all-gather push when they are peers' buffers).
DASER_API int daser_add_rmsnorm(void* x, int x_is_fp32, void* residual, const void* weight,
                                void* const* out_ptrs, int n_out, int64_t out_row_offset,
                                int64_t rows, int hidden, float eps, int zero_after,
                                cudaStream_t stream) {
  return daser_add_rmsnorm_tp(x, x_is_fp32, residual, weight, out_ptrs, n_out, out_row_offset, rows, hidden, eps,
                              zero_after, nullptr, 1, 0, stream);
}

DASER_API int daser_wait_flags(const uint32_t* flags, int n, uint32_t target, const uint32_t* base,
                               uint32_t* status, cudaStream_t stream) {
  if (!flags || n <= 0) return DASER_ERR_BAD_ARG;
  daser::wait_flags_kernel<<<1, 1, 0, stream>>>(flags, n, target, base, status);
  return (int)cudaGetLastError();
}

// flags[i] <- value for i < n (each possibly in a peer's memory), ordered after all earlier work
// of the stream: "what I wrote for you has landed".
DASER_API int daser_signal_flags(const uint64_t* flag_ptrs, int n, uint32_t value, cudaStream_t stream) {
  if (!flag_ptrs || n <= 0 || n > DASER_MAX_RANKS) return DASER_ERR_BAD_ARG;
  daser::SignalTargets t;
  for (int i = 0; i < DASER_MAX_RANKS; ++i) t.flag[i] = i < n ? reinterpret_cast<uint32_t*>(flag_ptrs[i]) : nullptr;
  daser::signal_flags_kernel<<<1, 32, 0, stream>>>(t, n, value);
  return (int)cudaGetLastError();
}

// table_ptrs[r], counter_ptrs[r]: rank r's candidate table and arrival counter (peer memory for
// r != rank).  best_val / best_idx: this rank's per-row candidates (n <= cap rows).
DASER_API int daser_tp_pick_token(const float* best_val, const int32_t* best_idx, int n, int rank, int tp, int cap,
                                  const uint64_t* table_ptrs, const uint64_t* counter_ptrs, uint32_t* epoch,
                                  uint32_t* status, int32_t* out_idx, cudaStream_t stream) {
  if (!best_val || !best_idx || !table_ptrs || !counter_ptrs || !epoch || !out_idx) return DASER_ERR_BAD_ARG;
  if (tp < 1 || tp > DASER_MAX_RANKS || rank < 0 || rank >= tp || n < 0 || n > cap) return DASER_ERR_BAD_ARG;
  if (n == 0) return 0;
  daser::CandTargets tg;
  for (int r = 0; r < DASER_MAX_RANKS; ++r) {
    tg.table[r] = r < tp ? reinterpret_cast<float*>(table_ptrs[r]) : nullptr;
    tg.counter[r] = r < tp ? reinterpret_cast<uint32_t*>(counter_ptrs[r]) : nullptr;
    if (r < tp && (!tg.table[r] || !tg.counter[r])) return DASER_ERR_BAD_ARG;
  }
  daser::tp_pick_token_kernel<<<1, 256, 0, stream>>>(best_val, best_idx, n, rank, tp, cap, tg, epoch, status, out_idx);
  return (int)cudaGetLastError();
}

DASER_API int daser_advance_epochs(uint32_t* epochs, uint32_t d0, uint32_t d1, uint32_t d2, cudaStream_t stream) {
  if (!epochs) return DASER_ERR_BAD_ARG;
  return (int)daser::launch_pdl(daser::advance_epochs_kernel, dim3(1), dim3(1), 0, stream, epochs, d0, d1, d2);
}

// The same with RMSNorm over head_dim on every query and key head before the rotation
// (q_norm_w, k_norm_w: bf16 [D]).
DASER_API int daser_rope_kv_write_qknorm(void* qkv, int qkv_is_fp32, int64_t qkv_stride, const int32_t* positions,
                                         const int64_t* slot_mapping, const float* cos_sin, int max_pos,
                                         void* q_out, int T, int Hq, int Hkv, int D, int block_tokens,
                                         const DaserKVPool* pool, int layer, int rank, int zero_after,
                                         const void* q_norm_w, const void* k_norm_w, float eps,
                                         cudaStream_t stream) {
  using namespace daser;
  if (!pool || !q_norm_w || !k_norm_w || T < 0 || D <= 0 || D % 32 || max_pos <= 0) return DASER_ERR_BAD_ARG;
  const int segs = D / 32;
  if (segs > 32 || (segs & (segs - 1))) return DASER_ERR_UNSUPPORTED;  // the lane butterfly needs a power of two
  if (rank < 0 || rank >= DASER_MAX_RANKS) return DASER_ERR_BAD_ARG;
  if (T == 0) return 0;
  const int64_t items = (int64_t)T * (Hq + 2 * Hkv) * segs;
  const int grid = ew_grid(items, 128);
#define LAUNCH_QK(TIN, FP8)                                                                        \
  launch_pdl(rope_kv_write_kernel<TIN, FP8, true>, dim3(grid), dim3(128), 0, stream,               \
      (TIN*)qkv, qkv_stride, positions, slot_mapping, cos_sin, max_pos, (__nv_bfloat16*)q_out, T,  \
      Hq, Hkv, D, block_tokens, *pool, layer, rank, zero_after, (const __nv_bfloat16*)q_norm_w,    \
      (const __nv_bfloat16*)k_norm_w, eps)
  if (qkv_is_fp32) { if (pool->pool_is_fp8) LAUNCH_QK(float, true); else LAUNCH_QK(float, false); }
  else { if (pool->pool_is_fp8) LAUNCH_QK(__nv_bfloat16, true); else LAUNCH_QK(__nv_bfloat16, false); }
#undef LAUNCH_QK
  return (int)cudaGetLastError();
}

DASER_API int daser_rope_kv_write(void* qkv, int qkv_is_fp32, int64_t qkv_stride, const int32_t* positions,
                                  const int64_t* slot_mapping, const float* cos_sin, int max_pos,
                                  void* q_out, int T, int Hq, int Hkv, int D, int block_tokens,
                                  const DaserKVPool* pool, int layer, int rank, int zero_after,
                                  cudaStream_t stream) {
  using namespace daser;
  if (!pool || T < 0 || D <= 0 || D % 32 || max_pos <= 0) return DASER_ERR_BAD_ARG;
  if (rank < 0 || rank >= DASER_MAX_RANKS) return DASER_ERR_BAD_ARG;
  if (T == 0) return 0;
  const int64_t items = (int64_t)T * (Hq + 2 * Hkv) * (D / 32);
  const int grid = ew_grid(items, 128);
#define LAUNCH(TIN, FP8)                                                                         \
  launch_pdl(rope_kv_write_kernel<TIN, FP8>, dim3(grid), dim3(128), 0, stream,                   \
      (TIN*)qkv, qkv_stride, positions, slot_mapping, cos_sin, max_pos, (__nv_bfloat16*)q_out, T, \
      Hq, Hkv, D, block_tokens, *pool, layer, rank, zero_after, (const __nv_bfloat16*)nullptr,    \
      (const __nv_bfloat16*)nullptr, 0.f)
  if (qkv_is_fp32) { if (pool->pool_is_fp8) LAUNCH(float, true); else LAUNCH(float, false); }
  else { if (pool->pool_is_fp8) LAUNCH(__nv_bfloat16, true); else LAUNCH(__nv_bfloat16, false); }
#undef LAUNCH
  return (int)cudaGetLastError();
}

DASER_API int daser_swiglu(void* x, int x_is_fp32, void* y, int64_t T, int inter, int zero_after,
                           int block, cudaStream_t stream) {
  using namespace daser;
  if (T < 0 || inter <= 0 || inter % 8) return DASER_ERR_BAD_ARG;
  if (block < 0 || (block && (block % 8 || inter % block))) return DASER_ERR_BAD_ARG;
  if (T == 0) return 0;
  const int grid = ew_grid(T * (inter / 8), 256);
  if (x_is_fp32)
    return (int)launch_pdl(swiglu_kernel<float>, dim3(grid), dim3(256), 0, stream, (float*)x, (__nv_bfloat16*)y, T, inter,
                           zero_after, block);
  return (int)launch_pdl(swiglu_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, stream, (__nv_bfloat16*)x,
                         (__nv_bfloat16*)y, T, inter, 0, block);
}

DASER_API int daser_embedding(const int32_t* ids, const void* table, void* out, int64_t T, int hidden,
                              int vocab_begin, int vocab_count, cudaStream_t stream) {
  using namespace daser;
  if (T < 0 || hidden <= 0 || hidden % 8) return DASER_ERR_BAD_ARG;
  if (T == 0) return 0;
  return (int)launch_pdl(embedding_kernel, dim3(ew_grid(T * (hidden / 8), 256)), dim3(256), 0, stream, ids,
                         (const __nv_bfloat16*)table, (__nv_bfloat16*)out, T, hidden, vocab_begin, vocab_count);
}

// Temperature sampling (Gumbel-max): inv_temp[rows] = 1 / temperature (0 = greedy for that row),
// seeds[rows] = one 64-bit seed per row and step.
DASER_API int daser_argmax_sample(void* logits, int is_fp32, int64_t stride, int rows, int n, int index_offset,
                                  float* best_val, int32_t* best_idx, int zero_after, const float* inv_temp,
                                  const uint64_t* seeds, cudaStream_t stream) {
  using namespace daser;
  if (rows < 0 || n <= 0 || stride % 8 || !inv_temp || !seeds) return DASER_ERR_BAD_ARG;
  if (rows == 0) return 0;
  if (is_fp32) argmax_kernel<float, true><<<rows, 1024, 0, stream>>>((float*)logits, stride, n, index_offset, best_val, best_idx, zero_after, inv_temp, seeds);
  else argmax_kernel<__nv_bfloat16, true><<<rows, 1024, 0, stream>>>((__nv_bfloat16*)logits, stride, n, index_offset, best_val, best_idx, 0, inv_temp, seeds);
  return (int)cudaGetLastError();
}

DASER_API int daser_argmax(void* logits, int is_fp32, int64_t stride, int rows, int n, int index_offset,
                           float* best_val, int32_t* best_idx, int zero_after, cudaStream_t stream) {
  using namespace daser;
  if (rows < 0 || n <= 0 || stride % 8) return DASER_ERR_BAD_ARG;
  if (rows == 0) return 0;
  if (is_fp32) argmax_kernel<float><<<rows, 1024, 0, stream>>>((float*)logits, stride, n, index_offset, best_val, best_idx, zero_after);
  else argmax_kernel<__nv_bfloat16><<<rows, 1024, 0, stream>>>((__nv_bfloat16*)logits, stride, n, index_offset, best_val, best_idx, 0);
  return (int)cudaGetLastError();
}
