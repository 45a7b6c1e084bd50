// Shared helpers of the sm_100a kernels: status codes, dtype codes, loads that
// convert to 32-bit, and block reductions that work for any multiple of 32 threads
// (the reference's tree reduction, kernels/elementwise.cu:41-48, needs a power of two).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

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

// Programmatic dependent launch: a kernel launched with launch_pdl may start while the kernel
// before it in the stream still runs.  It first lets ITS successor start (pdl_trigger), may
// fetch what no earlier kernel writes (weights), and calls pdl_wait before it touches anything
// an earlier kernel produces: pdl_wait returns when the preceding kernels have finished and
// their writes are visible.  Without the launch attribute both calls do nothing.
// Pointers to anything an earlier kernel of the step may have written are NOT declared
// `const __restrict__`: that lets the compiler read them through the non-coherent path
// (ld.global.nc), whose cached lines may predate the writes when kernels overlap, and lets it
// move the loads above the wait.  Only weights, biases and norm parameters are read that way.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// 0 switches the launch attribute off (environment CBIS_PDL=0): kernels then run strictly one after the other.
inline int pdl_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("CBIS_PDL");
    on = (e && e[0] == '0') ? 0 : 1;
  }
  return on;
}

// `after_kernel`: the operation before this launch in the stream is a kernel.  A kernel that
// follows a copy or a graph launch (the first kernel of a step, the sampling kernel after a
// replayed step) is launched without the attribute: it then starts only when everything before
// it has finished.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_after(bool after_kernel, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = after_kernel ? pdl_enabled() : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args... args) {
  return launch_after(true, kernel, grid, block, smem, st, args...);
}

// Asks the memory system to bring [p, p + bytes) into L2 (bytes a multiple of 16, p 16-byte aligned);
// nothing waits for it.  Used to have the NEXT kernel's weights on their way while this one runs.
__device__ __forceinline__ void prefetch_l2(const void* p, unsigned int bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

// This block's share of a prefetch of `bytes` bytes at `p`, spread evenly over the grid, in pieces of 16 KB.
__device__ __forceinline__ void prefetch_share(const void* p, unsigned long long bytes, unsigned int block,
                                               unsigned int n_blocks) {
  if (p == nullptr || bytes == 0) return;
  unsigned long long chunk = ((bytes + n_blocks - 1) / n_blocks + 15ull) & ~15ull;
  unsigned long long off = (unsigned long long)block * chunk;
  if (off >= bytes) return;
  unsigned long long end = off + chunk < bytes ? off + chunk : (bytes & ~15ull);
  for (; off < end; off += 16384ull) {
    const unsigned long long n = end - off < 16384ull ? end - off : 16384ull;
    prefetch_l2(static_cast<const char*>(p) + off, (unsigned int)n);
  }
}

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
