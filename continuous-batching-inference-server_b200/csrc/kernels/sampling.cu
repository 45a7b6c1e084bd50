// Next-token choice on the device: greedy argmax (first maximum wins, as the host scan of
// the reference does, src/server_demo.cpp:70-74) and temperature sampling by the Gumbel-max
// rule, argmax_i(logit_i / temperature + g_i), g_i = -log(-log u_i).  u_i comes from a counter
// generator keyed per (request, output index) by the host, so a draw depends neither on the
// batch nor on how the prompt was cut.
#include "common.cuh"
#include <math.h>

namespace cbis {

__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

// Best (score, index) of a thread's candidates, reduced over the block; valid in thread 0.
__device__ __forceinline__ void block_best(float& best, int& bi, float* sval, int* sidx) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if (lane == 0) { sval[warp] = best; sidx[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    best = lane < nwarp ? sval[lane] : -INFINITY;
    bi = lane < nwarp ? sidx[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
  }
}

// grid (chunks, R): block (c, r) scans its part of row r; the block of a row that finishes last
// (a counter per row, which it sets back to zero) reduces the chunks' results.  part_val/part_idx:
// [R][chunks]; counters: [R], zero before the first launch.
__global__ void sample_kernel(const float* logits, int ld, const float* temperature,
                              const unsigned long long* keys, int* __restrict__ out, int V,
                              float* part_val, int* part_idx, unsigned int* counters) {
  __shared__ float sval[32];
  __shared__ int sidx[32];
  __shared__ bool last;
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.y, chunks = gridDim.x;
  const float* row = logits + (size_t)r * ld;
  const float temp = temperature ? temperature[r] : 0.f;
  const unsigned long long key = keys ? keys[r] : 0ull;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < V; i += chunks * blockDim.x) {
    float v = row[i];
    if (temp > 0.f) {
      const unsigned long long z = mix64(key + (unsigned long long)(i + 1) * 0x9E3779B97F4A7C15ull);
      const float u = ((float)(z >> 41) + 0.5f) * (1.0f / 8388608.0f);  // (0,1), exact in 24 bits
      v = v / temp - logf(-logf(u));
    }
    if (v != v) v = -INFINITY;  // NaN never wins over a number
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
  }
  block_best(best, bi, sval, sidx);
  if (chunks == 1) {
    if (threadIdx.x == 0) out[r] = bi < V ? bi : 0;
    return;
  }
  if (threadIdx.x == 0) {
    part_val[(size_t)r * chunks + blockIdx.x] = best;
    part_idx[(size_t)r * chunks + blockIdx.x] = bi;
    __threadfence();
    last = atomicAdd(&counters[r], 1u) == (unsigned)chunks - 1;
  }
  __syncthreads();
  if (!last) return;
  __threadfence();
  best = -INFINITY;
  bi = 0x7fffffff;
  for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
    const float v = part_val[(size_t)r * chunks + c];
    const int i = part_idx[(size_t)r * chunks + c];
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
  }
  __syncthreads();
  block_best(best, bi, sval, sidx);
  if (threadIdx.x == 0) {
    out[r] = bi < V ? bi : 0;
    counters[r] = 0;
  }
}

}  // namespace cbis

using namespace cbis;

// Chunks a row of V entries is cut into, and the scratch this needs: chunks*R floats, chunks*R ints, R counters.
#define CBIS_SAMPLE_MAX_CHUNKS 64
CBIS_EXPORT int cbis_sample_chunks(int V) {
  int c = (V + 4095) / 4096;
  return c < 1 ? 1 : (c > CBIS_SAMPLE_MAX_CHUNKS ? CBIS_SAMPLE_MAX_CHUNKS : c);
}

// logits [R, ld >= V] 32-bit; temperature[R] (<= 0: greedy) and keys[R] may be null (greedy).
// part_val/part_idx [R * chunks], counters [R] (zeroed once by the caller; the kernel leaves them zero).
CBIS_EXPORT int cbis_sample(const float* logits, int ld, const float* temperature, const unsigned long long* keys,
                            int* out, int R, int V, float* part_val, int* part_idx, unsigned int* counters,
                            void* stream) {
  if (R <= 0) return CBIS_OK;
  if (V <= 0 || ld < V) return CBIS_ERR_BAD_SIZE;
  const int chunks = cbis_sample_chunks(V);
  if (chunks > 1 && (!part_val || !part_idx || !counters)) return CBIS_ERR_BAD_SIZE;
  const int threads = V >= 1024 ? 256 : 64;
  dim3 grid(chunks, R);
  return (int)launch_after(false, sample_kernel, grid, dim3(threads), 0, (cudaStream_t)stream, logits, ld, temperature, keys, out,
                         V, part_val, part_idx, counters);
}

// ---------------------------------------------------------------------------------------------
// The same sampling with the library's own scratch: see sample_no_alloc.h.
// ---------------------------------------------------------------------------------------------
#include "sample_no_alloc.h"
#include <mutex>

namespace {

constexpr int NA_MAX_CHUNKS = CBIS_SAMPLE_MAX_CHUNKS;  // the bound that cbis_sample_chunks() itself clamps to
constexpr int NA_WORDS = CBIS_SAMPLE_NO_ALLOC_MAX_ROWS * NA_MAX_CHUNKS * 2 + CBIS_SAMPLE_NO_ALLOC_MAX_ROWS;

// chunk maxima (floats), their indices (ints), one counter per row: 33,024 words = 132,096 bytes.
// In host code this name is only a handle for the runtime, never a device address.
static __device__ __align__(256) unsigned int na_scratch[NA_WORDS];

constexpr int NA_MAX_DEVICES = 64;
static unsigned int* na_device_ptr[NA_MAX_DEVICES];
static std::mutex na_mutex;

// Device address of na_scratch on the current device; looked up once per device.
static int na_scratch_address(unsigned int** ptr) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= NA_MAX_DEVICES) return CBIS_ERR_BAD_SIZE;
  std::lock_guard<std::mutex> lock(na_mutex);
  if (na_device_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, na_scratch);
    if (e != cudaSuccess) return (int)e;
    na_device_ptr[dev] = static_cast<unsigned int*>(p);
  }
  *ptr = na_device_ptr[dev];
  return CBIS_OK;
}

}  // namespace

CBIS_EXPORT int cbis_sample_no_alloc(const float* logits, int ld, const float* temperature,
                                     const unsigned long long* keys, int* out, int R, int V, void* stream) {
  if (R <= 0) return CBIS_OK;
  if (V <= 0 || ld < V) return CBIS_ERR_BAD_SIZE;
  if (R > CBIS_SAMPLE_NO_ALLOC_MAX_ROWS) return CBIS_ERR_TOO_LARGE;
  unsigned int* base = nullptr;
  const int st = na_scratch_address(&base);
  if (st != CBIS_OK) return st;
  float* part_val = reinterpret_cast<float*>(base);
  int* part_idx = reinterpret_cast<int*>(base + CBIS_SAMPLE_NO_ALLOC_MAX_ROWS * NA_MAX_CHUNKS);
  unsigned int* counters = base + CBIS_SAMPLE_NO_ALLOC_MAX_ROWS * NA_MAX_CHUNKS * 2;
  // The counters must be zero when the kernel starts; whatever an earlier call left (it may have been cut short) goes.
  cudaError_t e = cudaMemsetAsync(counters, 0, (size_t)R * sizeof(unsigned int), (cudaStream_t)stream);
  if (e != cudaSuccess) return (int)e;
  const int chunks = cbis_sample_chunks(V);
  if (chunks > NA_MAX_CHUNKS) return CBIS_ERR_TOO_LARGE;   // the fixed array is laid out for NA_MAX_CHUNKS per row
  const int threads = V >= 1024 ? 256 : 64;
  dim3 grid(chunks, R);
  return (int)launch_after(false, sample_kernel, grid, dim3(threads), 0, (cudaStream_t)stream, logits, ld, temperature,
                           keys, out, V, part_val, part_idx, counters);
}
