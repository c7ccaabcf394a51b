// Shared device helpers for the sm_100a kernels of daser_b200.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#define DASER_API extern "C" __attribute__((visibility("default")))

#include "kv_paged.h"  // DASER_ERR_* return codes and the host-visible parameter blocks

// True the first time it is called for the current device with this `flags` array: attributes
// set with cudaFuncSetAttribute belong to a device, so a process that drives several GPUs has to
// set them once on each.
#define DASER_MAX_DEVICES 64
static inline bool daser_first_use_on_device(bool (&flags)[DASER_MAX_DEVICES]) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= DASER_MAX_DEVICES) return true;
  if (flags[dev]) return false;
  flags[dev] = true;
  return true;
}

// Status words written by kernels whose waits ran out (see signals.cuh).
#define DASER_STATUS_OK 0u
#define DASER_STATUS_TIMEOUT 1u

#define FP8_GROUP 16
#define E4M3_MAX 448.0f

namespace daser {

// ---- programmatic dependent launch ----------------------------------------------------------
// A serving step is a few hundred short kernels in one stream.  Launched the plain way, each
// starts only after its predecessor has drained and the launch latency of every one of them is
// exposed.  Kernels launched with `launch_pdl` may instead be scheduled while the predecessor
// still runs: they run their set-up, call `pdl_wait()` (which returns once the predecessor has
// completed and its writes are visible) and only then touch memory.  `pdl_launch_dependents()`
// tells the scheduler that the NEXT kernel may be brought in; a kernel that holds tensor memory
// calls it only after its own allocation, so that a successor can never take the columns a
// not-yet-started CTA of this kernel still needs.
// Every kernel that is launched with `launch_pdl` must execute `pdl_wait()` before its first
// global-memory access.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_enter() {
  pdl_launch_dependents();
  pdl_wait();
}

inline bool pdl_allowed() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("DASER_PDL");
    v = (e == nullptr || e[0] != '0') ? 1 : 0;
  }
  return v == 1;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_allowed() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&p);
}

// Two e4m3 bytes (low 16 bits of v) -> two floats.
__device__ __forceinline__ float2 e4m3x2_to_float2(uint16_t v) {
  __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)v, __NV_E4M3);
  return __half22float2(*reinterpret_cast<__half2*>(&h));
}

__device__ __forceinline__ uint16_t float2_to_e4m3x2(float lo, float hi) {
  return (uint16_t)__nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, __NV_E4M3);
}

// 16 floats -> 16 e4m3 bytes with one shared scale (absmax / 448; 1 for an all-zero group).
// inv = 448 / absmax and the product x * inv are single IEEE fp32 operations so the
// CPU oracle (kv/codec.py) reproduces the payload bit for bit.
__device__ __forceinline__ void quant_group16(const float (&x)[16], uint4& payload, float& scale) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(x[i]));
  float inv = 1.f;
  scale = 1.f;
  if (amax > 0.f) {
    inv = __fdiv_rn(E4M3_MAX, amax);
    scale = __fdiv_rn(amax, E4M3_MAX);
  }
  // cvt.rn.satfinite saturates at +-448, which is what a clamp of x * inv would give
  // (|x * inv| exceeds 448 by rounding at most), so no explicit clamp is needed.
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    w[i] = (uint32_t)float2_to_e4m3x2(__fmul_rn(x[4 * i + 0], inv), __fmul_rn(x[4 * i + 1], inv)) |
           ((uint32_t)float2_to_e4m3x2(__fmul_rn(x[4 * i + 2], inv), __fmul_rn(x[4 * i + 3], inv)) << 16);
  }
  payload = make_uint4(w[0], w[1], w[2], w[3]);
}

__device__ __forceinline__ void dequant_group16(const uint4& payload, float scale, float (&x)[16]) {
  const uint32_t w[4] = {payload.x, payload.y, payload.z, payload.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 a = e4m3x2_to_float2((uint16_t)(w[i] & 0xffffu));
    float2 b = e4m3x2_to_float2((uint16_t)(w[i] >> 16));
    x[4 * i + 0] = __fmul_rn(a.x, scale);
    x[4 * i + 1] = __fmul_rn(a.y, scale);
    x[4 * i + 2] = __fmul_rn(b.x, scale);
    x[4 * i + 3] = __fmul_rn(b.y, scale);
  }
}

__device__ __forceinline__ void load_bf16x16(const __nv_bfloat16* p, float (&x)[16]) {
  const uint4 a = *reinterpret_cast<const uint4*>(p);
  const uint4 b = *reinterpret_cast<const uint4*>(p + 8);
  const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    x[2 * i] = bf16_lo(w[i]);
    x[2 * i + 1] = bf16_hi(w[i]);
  }
}

__device__ __forceinline__ void store_bf16x16(__nv_bfloat16* p, const float (&x)[16]) {
  uint32_t w[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) w[i] = pack_bf16x2(x[2 * i], x[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  *reinterpret_cast<uint4*>(p + 8) = make_uint4(w[4], w[5], w[6], w[7]);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace daser
