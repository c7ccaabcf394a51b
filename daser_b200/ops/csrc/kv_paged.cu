// Fused chunk-KV restore and save between slot images and paged KV pools.
//
// Restore replaces the reference's host-driven loop of one strided ATen copy per
// (request, slot, layer) (daser/connector/daser_connector.py:537-551): one launch
// covers every slot and layer of the step, dequantises block-scaled fp8, rotates
// keys by the chunk's position delta, optionally requantises for an fp8 pool, and
// stores each head slice straight into the paged pool of the tensor-parallel rank
// that owns it (plain 16-byte stores to peer-mapped pointers over NVLink).
//
// Save replaces daser_connector.py:625-632 (two kernels and an allocation per
// (slot, layer)): each rank gathers its own blocks, compresses them and writes its
// head slice into the slot image, which may live in the IO owner's memory.
//
// One CTA handles one (slot, layer) tile.  A work item is one (K|V, token, head)
// row segment made of dims [16j, 16j+16) and the rotary partner [D/2+16j, D/2+16j+16),
// i.e. exactly two fp8 scale groups, so rotation and requantisation stay thread local.
#include "common.cuh"
#include "kv_paged.h"

namespace daser {

#define KV_ERR_BLOCK_RANGE 2u
#define KV_ERR_DELTA_RANGE 3u
#define KV_ERR_NULL_SLOT 4u

__device__ __forceinline__ void report(uint32_t* status, uint32_t code, uint32_t slot) {
  if (status != nullptr && atomicCAS(status, 0u, code) == 0u) status[1] = slot;
}

// Where element (kv, tok, head, dim0) of a layer goes: the owning rank and the element offset in
// that rank's pool.  With more ranks than KV heads a head is replicated on `replicas` ranks.
struct RestoreDst {
  int rank0;
  int64_t off;
};
__device__ __forceinline__ RestoreDst restore_dst(const DaserKVPool& pool, int H, int replicas, int layer, int block,
                                                  int kv, int tok, int head, int dim0) {
  RestoreDst d;
  const bool wide = pool.n_ranks > H;
  d.rank0 = wide ? head * replicas : head / pool.heads_per_rank;
  const int head_local = wide ? 0 : head % pool.heads_per_rank;
  d.off = (int64_t)layer * pool.stride_layer + (int64_t)block * pool.stride_block + (int64_t)kv * pool.stride_kv +
          (int64_t)tok * pool.stride_tok + (int64_t)head_local * pool.stride_head + dim0;
  return d;
}

// row -> (kv, tok, head) of the image order [K|V][tok][head]; shifts when the sizes are powers of two.
__device__ __forceinline__ void split_row(const DaserKVJob& job, int row, int& kv, int& tok, int& head) {
  if (job.lg_heads >= 0) {
    head = row & ((1 << job.lg_heads) - 1);
    tok = (row >> job.lg_heads) & ((1 << job.lg_tokens) - 1);
    kv = row >> (job.lg_heads + job.lg_tokens);
  } else {
    const int H = job.num_kv_heads, B = job.block_tokens;
    head = row % H;
    tok = (row / H) % B;
    kv = row / (H * B);
  }
}

// One CTA per (slot, layer) of the launch's layer range.
//
// fp8 image into an fp8 pool, the serving path, is mostly a relayout: values rows and the key
// rows of a chunk that keeps its position (delta 0) are copied as they are, 16 payload bytes (one
// scale group) and 16 scale bytes (four groups) per access, four accesses in flight per thread.
// Only key rows that move are dequantised, rotated and requantised, thread-local on the two
// scale groups that rotate into one another.  Every other codec / pool combination goes through
// the general per-item path.
template <bool IMG_FP8, bool POOL_FP8>
__global__ void __launch_bounds__(256)
kv_restore_kernel(const DaserKVJob job, const DaserKVPool pool) {
  extern __shared__ __align__(16) float s_cs[];  // cos[D/2] then sin[D/2] for this slot's delta
  const int n_layers = job.layer_count > 0 ? job.layer_count : job.num_layers;
  const int slot = blockIdx.x / n_layers;
  const int layer = job.layer_begin + blockIdx.x % n_layers;
  const int D = job.head_dim, H = job.num_kv_heads, B = job.block_tokens;
  const int half = D >> 1;
  const int block = job.block_id[slot];
  const uint64_t img = job.slot_ptr[slot];
  int delta = job.delta ? job.delta[slot] : 0;
  if (block < 0 || block >= pool.num_blocks) {
    if (threadIdx.x == 0) report(job.status, KV_ERR_BLOCK_RANGE, slot);
    return;
  }
  if (img == 0) {
    if (threadIdx.x == 0) report(job.status, KV_ERR_NULL_SLOT, slot);
    return;
  }
  const int adelta = delta < 0 ? -delta : delta;
  if (adelta >= job.max_pos && delta != 0) {
    if (threadIdx.x == 0) report(job.status, KV_ERR_DELTA_RANGE, slot);
    return;
  }
  if (delta != 0) {
    const float* row = job.cos_sin + (int64_t)adelta * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
      float v = row[i];
      s_cs[i] = (i >= half && delta < 0) ? -v : v;  // sin(-x) = -sin(x)
    }
    __syncthreads();
  }

  const int64_t elems_kv = (int64_t)B * H * D;
  const int64_t layer_bytes = IMG_FP8 ? (2 * elems_kv + 2 * elems_kv / FP8_GROUP * 4) : 4 * elems_kv;
  const uint8_t* base = reinterpret_cast<const uint8_t*>(img) + (int64_t)layer * layer_bytes;
  const float* img_scales = reinterpret_cast<const float*>(base + 2 * elems_kv);
  const int replicas = pool.n_ranks > H ? pool.n_ranks / H : 1;
  const int rows = 2 * B * H;

  if (IMG_FP8 && POOL_FP8) {
    // ---- copy path: rows [kv_first * B * H, 2 * B * H) keep their bytes ----
    const int kv_first = delta != 0 ? 1 : 0;
    const int vec_per_row = D / FP8_GROUP;           // 16-byte payload vectors per row
    const int n_vec = (2 - kv_first) * B * H * vec_per_row;
    const int v0 = kv_first * B * H * vec_per_row;
    for (int it = threadIdx.x; it < n_vec; it += 4 * blockDim.x) {
      uint4 q[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int v = it + u * blockDim.x;
        if (v < n_vec) q[u] = *reinterpret_cast<const uint4*>(base + (int64_t)(v0 + v) * FP8_GROUP);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int v = it + u * blockDim.x;
        if (v >= n_vec) continue;
        const int g = v0 + v;
        const int row = job.lg_groups >= 0 ? g >> job.lg_groups : g / vec_per_row;
        const int j = g - row * vec_per_row;
        int head, tok, kv;
        split_row(job, row, kv, tok, head);
        const RestoreDst d = restore_dst(pool, H, replicas, layer, block, kv, tok, head, j * FP8_GROUP);
        for (int rep = 0; rep < replicas; ++rep)
          *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(pool.payload[d.rank0 + rep]) + d.off) = q[u];
      }
    }
    // scales of the same rows: D / 16 floats per row, moved four at a time
    const int sv_per_row = vec_per_row / 4;
    const bool wide_scales = sv_per_row * 4 == vec_per_row &&
                             ((pool.stride_layer | pool.stride_block | pool.stride_kv | pool.stride_tok |
                               pool.stride_head) % (4 * FP8_GROUP)) == 0;  // 16-byte aligned scale quads
    if (wide_scales) {
      const int n_sv = (2 - kv_first) * B * H * sv_per_row;
      const int s0 = kv_first * B * H * sv_per_row;
      for (int v = threadIdx.x; v < n_sv; v += blockDim.x) {
        const int g = s0 + v;
        const float4 sc = *reinterpret_cast<const float4*>(img_scales + (int64_t)g * 4);
        const int row = g / sv_per_row, j4 = g - row * sv_per_row;
        int head, tok, kv;
        split_row(job, row, kv, tok, head);
        const RestoreDst d = restore_dst(pool, H, replicas, layer, block, kv, tok, head, j4 * 4 * FP8_GROUP);
        for (int rep = 0; rep < replicas; ++rep)
          *reinterpret_cast<float4*>(pool.scales[d.rank0 + rep] + d.off / FP8_GROUP) = sc;
      }
    } else {
      const int n_s = (2 - kv_first) * B * H * vec_per_row;
      const int s0 = kv_first * B * H * vec_per_row;
      for (int v = threadIdx.x; v < n_s; v += blockDim.x) {
        const int g = s0 + v;
        const int row = g / vec_per_row, j = g - row * vec_per_row;
        int head, tok, kv;
        split_row(job, row, kv, tok, head);
        const RestoreDst d = restore_dst(pool, H, replicas, layer, block, kv, tok, head, j * FP8_GROUP);
        for (int rep = 0; rep < replicas; ++rep) pool.scales[d.rank0 + rep][d.off / FP8_GROUP] = img_scales[g];
      }
    }
    if (delta == 0) return;
    // key rows (kv = 0) still to do, through the item path below
  }

  // ---- item path: one (row, pair of scale groups) per item ----
  const int segs = half / FP8_GROUP;  // items per row
  const int item_rows = (IMG_FP8 && POOL_FP8) ? B * H : rows;  // copy path took the value rows
  for (int item = threadIdx.x; item < item_rows * segs; item += blockDim.x) {
    const int j = item % segs;
    const int row = item / segs;
    int head, tok, kv;
    split_row(job, row, kv, tok, head);
    const int64_t e1 = (int64_t)row * D + j * FP8_GROUP;  // element offset inside the layer
    const int64_t e2 = e1 + half;
    float x1[16], x2[16];
    uint4 q1, q2;
    float sc1 = 1.f, sc2 = 1.f;
    if (IMG_FP8) {
      q1 = *reinterpret_cast<const uint4*>(base + e1);
      q2 = *reinterpret_cast<const uint4*>(base + e2);
      sc1 = img_scales[e1 / FP8_GROUP];
      sc2 = img_scales[e2 / FP8_GROUP];
    } else {
      load_bf16x16(reinterpret_cast<const __nv_bfloat16*>(base) + e1, x1);
      load_bf16x16(reinterpret_cast<const __nv_bfloat16*>(base) + e2, x2);
    }
    const bool rotate = (kv == 0) && (delta != 0);
    const bool passthrough = IMG_FP8 && POOL_FP8 && !rotate;
    if (!passthrough) {
      if (IMG_FP8) {
        dequant_group16(q1, sc1, x1);
        dequant_group16(q2, sc2, x2);
      }
      if (rotate) {
        float c[16], sn[16];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float4 cv = *reinterpret_cast<const float4*>(&s_cs[j * FP8_GROUP + 4 * i]);
          const float4 sv = *reinterpret_cast<const float4*>(&s_cs[half + j * FP8_GROUP + 4 * i]);
          c[4 * i] = cv.x; c[4 * i + 1] = cv.y; c[4 * i + 2] = cv.z; c[4 * i + 3] = cv.w;
          sn[4 * i] = sv.x; sn[4 * i + 1] = sv.y; sn[4 * i + 2] = sv.z; sn[4 * i + 3] = sv.w;
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float a = x1[i], b = x2[i];
          x1[i] = __fsub_rn(__fmul_rn(a, c[i]), __fmul_rn(b, sn[i]));
          x2[i] = __fadd_rn(__fmul_rn(b, c[i]), __fmul_rn(a, sn[i]));
        }
      }
      if (POOL_FP8) {
        quant_group16(x1, q1, sc1);
        quant_group16(x2, q2, sc2);
      }
    }
    const RestoreDst dst = restore_dst(pool, H, replicas, layer, block, kv, tok, head, j * FP8_GROUP);
    const int64_t d1 = dst.off;
    const int64_t d2 = d1 + half;
    for (int rep = 0; rep < replicas; ++rep) {
      const int r = dst.rank0 + rep;
      if (POOL_FP8) {
        uint8_t* p = reinterpret_cast<uint8_t*>(pool.payload[r]);
        *reinterpret_cast<uint4*>(p + d1) = q1;
        *reinterpret_cast<uint4*>(p + d2) = q2;
        pool.scales[r][d1 / FP8_GROUP] = sc1;
        pool.scales[r][d2 / FP8_GROUP] = sc2;
      } else {
        __nv_bfloat16* p = reinterpret_cast<__nv_bfloat16*>(pool.payload[r]);
        store_bf16x16(p + d1, x1);
        store_bf16x16(p + d2, x2);
      }
    }
  }
}

template <bool IMG_FP8, bool POOL_FP8>
__global__ void __launch_bounds__(256)
kv_save_kernel(const DaserKVJob job, const DaserKVPool pool) {
  const int slot = blockIdx.x / job.num_layers;
  const int layer = blockIdx.x % job.num_layers;
  const int D = job.head_dim, H = job.num_kv_heads, B = job.block_tokens;
  const int block = job.block_id[slot];
  const uint64_t img = job.slot_ptr[slot];
  if (block < 0 || block >= pool.num_blocks) {
    if (threadIdx.x == 0) report(job.status, KV_ERR_BLOCK_RANGE, slot);
    return;
  }
  if (img == 0) {
    if (threadIdx.x == 0) report(job.status, KV_ERR_NULL_SLOT, slot);
    return;
  }
  // Heads of this rank inside the full-head slot image.
  int head0, nheads;
  if (pool.n_ranks > H) {
    const int replicas = pool.n_ranks / H;
    if (job.rank % replicas) return;  // only the first replica of a head writes it
    head0 = job.rank / replicas;
    nheads = 1;
  } else {
    head0 = job.rank * pool.heads_per_rank;
    nheads = pool.heads_per_rank;
  }
  const int64_t elems_kv = (int64_t)B * H * D;
  const int64_t layer_bytes = IMG_FP8 ? (2 * elems_kv + 2 * elems_kv / FP8_GROUP * 4) : 4 * elems_kv;
  uint8_t* base = reinterpret_cast<uint8_t*>(img) + (int64_t)layer * layer_bytes;
  float* img_scales = reinterpret_cast<float*>(base + 2 * elems_kv);
  const uint8_t* pool_q = reinterpret_cast<const uint8_t*>(pool.payload[job.rank]);
  const __nv_bfloat16* pool_h = reinterpret_cast<const __nv_bfloat16*>(pool.payload[job.rank]);
  const float* pool_s = pool.scales[job.rank];

  const int segs = D / FP8_GROUP;
  const int rows = 2 * B * nheads;
  for (int item = threadIdx.x; item < rows * segs; item += blockDim.x) {
    const int j = item % segs;
    const int row = item / segs;
    const int hl = row % nheads;
    const int tok = (row / nheads) % B;
    const int kv = row / (nheads * B);
    const int64_t s = (int64_t)layer * pool.stride_layer + (int64_t)block * pool.stride_block +
                      (int64_t)kv * pool.stride_kv + (int64_t)tok * pool.stride_tok +
                      (int64_t)hl * pool.stride_head + j * FP8_GROUP;
    const int64_t e = (((int64_t)kv * B + tok) * H + head0 + hl) * D + j * FP8_GROUP;
    float x[16];
    uint4 q;
    float sc = 1.f;
    if (POOL_FP8) {
      q = *reinterpret_cast<const uint4*>(pool_q + s);
      sc = pool_s[s / FP8_GROUP];
      if (!IMG_FP8) dequant_group16(q, sc, x);
    } else {
      load_bf16x16(pool_h + s, x);
      if (IMG_FP8) quant_group16(x, q, sc);
    }
    if (IMG_FP8) {
      *reinterpret_cast<uint4*>(base + e) = q;
      img_scales[e / FP8_GROUP] = sc;
    } else {
      store_bf16x16(reinterpret_cast<__nv_bfloat16*>(base) + e, x);
    }
  }
}

static int check(const DaserKVJob& j, const DaserKVPool& p) {
  if (j.n_slots < 0 || j.num_layers <= 0 || j.num_kv_heads <= 0 || j.block_tokens <= 0) return DASER_ERR_BAD_ARG;
  if (j.head_dim <= 0 || j.head_dim % 32) return DASER_ERR_UNSUPPORTED;
  if (p.n_ranks < 1 || p.n_ranks > DASER_MAX_RANKS) return DASER_ERR_BAD_ARG;
  if (p.n_ranks <= j.num_kv_heads) {
    if (j.num_kv_heads % p.n_ranks || p.heads_per_rank != j.num_kv_heads / p.n_ranks) return DASER_ERR_BAD_ARG;
  } else if (p.n_ranks % j.num_kv_heads || p.heads_per_rank != 1) {
    return DASER_ERR_BAD_ARG;
  }
  if ((p.stride_layer | p.stride_block | p.stride_kv | p.stride_tok | p.stride_head) % 16) return DASER_ERR_UNSUPPORTED;
  return 0;
}

}  // namespace daser

DASER_API int daser_kv_restore(const DaserKVJob* job, const DaserKVPool* pool, cudaStream_t stream) {
  using namespace daser;
  if (!job || !pool) return DASER_ERR_BAD_ARG;
  if (int e = check(*job, *pool)) return e;
  if (job->n_slots == 0) return 0;
  if (job->delta && (!job->cos_sin || job->max_pos <= 0)) return DASER_ERR_BAD_ARG;
  if (job->layer_begin < 0 || job->layer_count < 0 || job->layer_begin + job->layer_count > job->num_layers)
    return DASER_ERR_BAD_ARG;
  const int n_layers = job->layer_count > 0 ? job->layer_count : job->num_layers - job->layer_begin;
  if (n_layers <= 0) return 0;
  DaserKVJob ranged = *job;
  ranged.layer_count = n_layers;
  auto lg = [](int v) { int l = 0; while ((1 << l) < v) ++l; return (1 << l) == v ? l : -1; };
  ranged.lg_heads = lg(job->num_kv_heads);
  ranged.lg_tokens = lg(job->block_tokens);
  ranged.lg_groups = lg(job->head_dim / FP8_GROUP);
  if (ranged.lg_heads < 0 || ranged.lg_tokens < 0 || ranged.lg_groups < 0) ranged.lg_heads = ranged.lg_tokens = ranged.lg_groups = -1;
  job = &ranged;
  const dim3 grid((unsigned)(job->n_slots * n_layers));
  const size_t smem = job->head_dim * sizeof(float);
  const bool a = job->image_is_fp8, b = pool->pool_is_fp8;
  if (a && b) kv_restore_kernel<true, true><<<grid, 256, smem, stream>>>(*job, *pool);
  else if (a && !b) kv_restore_kernel<true, false><<<grid, 256, smem, stream>>>(*job, *pool);
  else if (!a && b) kv_restore_kernel<false, true><<<grid, 256, smem, stream>>>(*job, *pool);
  else kv_restore_kernel<false, false><<<grid, 256, smem, stream>>>(*job, *pool);
  return (int)cudaGetLastError();
}

DASER_API int daser_kv_save(const DaserKVJob* job, const DaserKVPool* pool, cudaStream_t stream) {
  using namespace daser;
  if (!job || !pool) return DASER_ERR_BAD_ARG;
  if (int e = check(*job, *pool)) return e;
  if (job->rank < 0 || job->rank >= pool->n_ranks) return DASER_ERR_BAD_ARG;
  if (job->n_slots == 0) return 0;
  const dim3 grid((unsigned)(job->n_slots * job->num_layers));
  const bool a = job->image_is_fp8, b = pool->pool_is_fp8;
  if (a && b) kv_save_kernel<true, true><<<grid, 256, 0, stream>>>(*job, *pool);
  else if (a && !b) kv_save_kernel<true, false><<<grid, 256, 0, stream>>>(*job, *pool);
  else if (!a && b) kv_save_kernel<false, true><<<grid, 256, 0, stream>>>(*job, *pool);
  else kv_save_kernel<false, false><<<grid, 256, 0, stream>>>(*job, *pool);
  return (int)cudaGetLastError();
}

// `rows` runs of `width` bytes, `pitch` bytes apart on both sides, moved by the copy engine
// (cudaMemcpy2DAsync, direction inferred from the pointers).  Used to bring some layers of every
// slot image of a chunk from the pinned host tier into the HBM tier without a kernel.
DASER_API int daser_copy_rows(void* dst, const void* src, int64_t pitch, int64_t width, int64_t rows,
                              cudaStream_t stream) {
  if (!dst || !src || width <= 0 || rows <= 0 || pitch < width) return DASER_ERR_BAD_ARG;
  if (rows == 1 || pitch == width)
    return (int)cudaMemcpyAsync(dst, src, (size_t)(width * rows), cudaMemcpyDefault, stream);
  return (int)cudaMemcpy2DAsync(dst, (size_t)pitch, src, (size_t)pitch, (size_t)width, (size_t)rows,
                                cudaMemcpyDefault, stream);
}
