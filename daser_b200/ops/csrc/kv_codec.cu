// Block-scaled fp8 (e4m3, one fp32 scale per 16 elements) quantise / dequantise.
//
// Stand-alone form of the codec that the save and restore kernels apply inline;
// used by the HBM tier when it admits bf16 KV and by the tests.  The reference
// stores KV raw and has no codec (daser/connector/daser_connector.py:625-632).
// One thread owns one 16-element group: 32 B in, 16 B + 4 B out, so a warp
// moves 1 KiB of contiguous bf16 per instruction pair.
#include "common.cuh"

namespace daser {

__global__ void __launch_bounds__(256)
quant_fp8b16_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ payload,
                    float* __restrict__ scales, int64_t n_groups) {
  for (int64_t g = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; g < n_groups;
       g += (int64_t)gridDim.x * blockDim.x) {
    float v[16];
    load_bf16x16(x + g * 16, v);
    uint4 q;
    float s;
    quant_group16(v, q, s);
    *reinterpret_cast<uint4*>(payload + g * 16) = q;
    scales[g] = s;
  }
}

__global__ void __launch_bounds__(256)
dequant_fp8b16_kernel(const uint8_t* __restrict__ payload, const float* __restrict__ scales,
                      __nv_bfloat16* __restrict__ y, int64_t n_groups) {
  for (int64_t g = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; g < n_groups;
       g += (int64_t)gridDim.x * blockDim.x) {
    float v[16];
    dequant_group16(*reinterpret_cast<const uint4*>(payload + g * 16), scales[g], v);
    store_bf16x16(y + g * 16, v);
  }
}

static int grid_for(int64_t n_groups) {
  int64_t blocks = (n_groups + 255) / 256;
  const int64_t cap = 148 * 8;
  return (int)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

}  // namespace daser

DASER_API int daser_quant_fp8b16(const void* x, void* payload, void* scales, int64_t n_elems,
                                 cudaStream_t stream) {
  if (n_elems < 0 || n_elems % 16) return DASER_ERR_BAD_ARG;
  if (n_elems == 0) return 0;
  const int64_t g = n_elems / 16;
  daser::quant_fp8b16_kernel<<<daser::grid_for(g), 256, 0, stream>>>(
      (const __nv_bfloat16*)x, (uint8_t*)payload, (float*)scales, g);
  return (int)cudaGetLastError();
}

DASER_API int daser_dequant_fp8b16(const void* payload, const void* scales, void* y,
                                   int64_t n_elems, cudaStream_t stream) {
  if (n_elems < 0 || n_elems % 16) return DASER_ERR_BAD_ARG;
  if (n_elems == 0) return 0;
  const int64_t g = n_elems / 16;
  daser::dequant_fp8b16_kernel<<<daser::grid_for(g), 256, 0, stream>>>(
      (const uint8_t*)payload, (const float*)scales, (__nv_bfloat16*)y, g);
  return (int)cudaGetLastError();
}
