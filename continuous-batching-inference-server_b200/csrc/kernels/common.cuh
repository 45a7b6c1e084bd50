// Shared helpers of the sm_100a kernels: status codes, dtype codes, loads that
// convert to 32-bit, and block reductions that work for any multiple of 32 threads
// (the reference's tree reduction, kernels/elementwise.cu:41-48, needs a power of two).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

// Status codes returned by every launcher (0 = launched; CUDA errors are returned as they are, > 0).
#define CBIS_OK 0
#define CBIS_ERR_BAD_DTYPE (-1)
#define CBIS_ERR_BAD_SIZE (-2)       // a size the kernel does not take (the message names it on the Python side)
#define CBIS_ERR_ALIGNMENT (-3)
#define CBIS_ERR_TOO_LARGE (-4)

#define CBIS_F32 0
#define CBIS_BF16 1

#define CBIS_ACT_NONE 0
#define CBIS_ACT_GELU_ERF 1
#define CBIS_ACT_GELU_TANH 2

#define CBIS_EXPORT extern "C" __attribute__((visibility("default")))

namespace cbis {

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ void from_f32(float& dst, float v) { dst = v; }
__device__ __forceinline__ void from_f32(__nv_bfloat16& dst, float v) { dst = __float2bfloat16_rn(v); }

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

// Sum over the block; every thread gets the result.  `red` holds >= 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // protects `red` from a previous use
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarp ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

// GELU in 32-bit.  erf form: kernels/elementwise.cu:59-66 of the reference; tanh form: GPT-2's gelu_new.
__device__ __forceinline__ float activate(float v, int act) {
  if (act == CBIS_ACT_GELU_ERF) return 0.5f * v * (1.0f + erff(v * 0.70710678118654752440f));
  if (act == CBIS_ACT_GELU_TANH) {
    const float c = 0.7978845608028654f;  // sqrt(2/pi)
    return 0.5f * v * (1.0f + tanhf(c * (v + 0.044715f * v * v * v)));
  }
  return v;
}

}  // namespace cbis
