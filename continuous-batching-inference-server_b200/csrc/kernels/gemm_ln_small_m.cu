// LayerNorm and the matrix product that follows it, for up to 8 rows (decoding), in one kernel:
//   C[M,N] = act(LN(x)[M,K] * W^T + bias),   x the 32-bit residual rows, W stored [N,K] (K contiguous)
// A separate norm kernel normalises a few rows in a microsecond or two; most of what it costs in a decode step is the
// boundary between two dependent kernels.  Here every block normalises the M rows itself, two warps to a row
// (statistics in 32-bit, mean first and then the centred squares, as kernels/elementwise.cu of this package does; the
// reference: kernels/elementwise.cu:21-57), into shared memory as bfloat16, and then runs the weight-streaming product
// of gemm_small_m.cu on them.  A block is two groups of 8 warps; a group owns 16 output columns over the whole of K,
// its warps take the 32-wide K blocks in turn, every lane fetches 16 bytes of a weight row per block (ld.global.nc;
// the K order is permuted alike for both operands, so that one 16-byte load is two mma.sync m16n8k16 fragments), the
// warps' partial sums meet in shared memory, bias and activation are applied to the 32-bit sum before the one store.
// Two groups to a block halve what the redundant normalising reads from L2 (M*K*4 bytes per block).
#include "common.cuh"

namespace cbis {
namespace gln {

constexpr int GROUPS = 2, GROUP_WARPS = 8, WARPS = GROUPS * GROUP_WARPS, THREADS = WARPS * 32;
constexpr int NT = 2, UNROLL = 4, COLS = NT * 8, RS = COLS + 1;
constexpr int ROWS = 8;                    // rows of the one tensor-core row tile that are used
constexpr int REG_VEC = 8;                 // float4 of a row that a lane holds: rows up to 2 * 32 * 8 * 4 = 2,048 wide stay in registers

__device__ __forceinline__ void mma_bf16_16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void group_sync(int group) {   // a named barrier per group; the ids are literals so that only these are reserved
  if (group == 0) asm volatile("bar.sync 1, %0;" ::"n"(GROUP_WARPS * 32) : "memory");
  else asm volatile("bar.sync 2, %0;" ::"n"(GROUP_WARPS * 32) : "memory");
}
__device__ __forceinline__ void store_normalised(__nv_bfloat16* dst, const float4& v, float mean, float inv, const float4& gm,
                                                 const float4& bt) {
  __nv_bfloat162 lo = __floats2bfloat162_rn((v.x - mean) * inv * gm.x + bt.x, (v.y - mean) * inv * gm.y + bt.y);
  __nv_bfloat162 hi = __floats2bfloat162_rn((v.z - mean) * inv * gm.z + bt.z, (v.w - mean) * inv * gm.w + bt.w);
  uint2 r;
  r.x = *reinterpret_cast<unsigned*>(&lo);
  r.y = *reinterpret_cast<unsigned*>(&hi);
  *reinterpret_cast<uint2*>(dst) = r;
}

// The M rows of x -> h (bfloat16, row pitch `pitch`), columns K .. kpad-1 zero.  Warps 2r and 2r+1 share row r: its
// float4 number c belongs to lane (c % 64) of the pair.  Called by all threads of the block.
template <bool IN_REGISTERS>
__device__ __forceinline__ void normalise_rows(const float* x, int ldx, const float* __restrict__ gamma,
                                               const float* __restrict__ beta, float eps, int M, int K, int kpad, int pitch,
                                               __nv_bfloat16* h, float* stat) {   // gamma, beta: the block's copies in shared memory
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int r = warp >> 1, first = (warp & 1) * 32 + lane;
  const int nvec = K >> 2;
  const bool live = r < M;
  const float4* xv = reinterpret_cast<const float4*>(x + (size_t)(live ? r : 0) * ldx);
  float4 v[IN_REGISTERS ? REG_VEC : 1];
  float sum = 0.f;
  if (live) {
    if constexpr (IN_REGISTERS) {
#pragma unroll
      for (int i = 0; i < REG_VEC; ++i) {
        const int c = first + 64 * i;
        v[i] = c < nvec ? __ldcg(xv + c) : make_float4(0.f, 0.f, 0.f, 0.f);
        sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
      }
    } else {
      for (int c = first; c < nvec; c += 64) {
        const float4 t = __ldcg(xv + c);
        sum += (t.x + t.y) + (t.z + t.w);
      }
    }
    sum = warp_sum(sum);
    if (lane == 0) stat[warp] = sum;
  }
  __syncthreads();
  float mean = 0.f, sq = 0.f;
  if (live) {
    mean = (stat[2 * r] + stat[2 * r + 1]) / (float)K;
    if constexpr (IN_REGISTERS) {
#pragma unroll
      for (int i = 0; i < REG_VEC; ++i) {
        if (first + 64 * i < nvec) {
          const float a = v[i].x - mean, b = v[i].y - mean, c2 = v[i].z - mean, e = v[i].w - mean;
          sq += (a * a + b * b) + (c2 * c2 + e * e);
        }
      }
    } else {
      for (int c = first; c < nvec; c += 64) {
        const float4 t = __ldcg(xv + c);
        const float a = t.x - mean, b = t.y - mean, c2 = t.z - mean, e = t.w - mean;
        sq += (a * a + b * b) + (c2 * c2 + e * e);
      }
    }
    sq = warp_sum(sq);
    if (lane == 0) stat[WARPS + warp] = sq;
  }
  __syncthreads();
  __nv_bfloat16* dst = h + (size_t)r * pitch;
  if (live) {
    const float inv = rsqrtf((stat[WARPS + 2 * r] + stat[WARPS + 2 * r + 1]) / (float)K + eps);
    const float4* gv = reinterpret_cast<const float4*>(gamma);
    const float4* bv = reinterpret_cast<const float4*>(beta);
    if constexpr (IN_REGISTERS) {
#pragma unroll
      for (int i = 0; i < REG_VEC; ++i) {
        const int c = first + 64 * i;
        if (c < nvec) store_normalised(dst + 4 * c, v[i], mean, inv, gv[c], bv[c]);
      }
    } else {
      for (int c = first; c < nvec; c += 64) store_normalised(dst + 4 * c, __ldcg(xv + c), mean, inv, gv[c], bv[c]);
    }
    for (int c = K + first; c < kpad; c += 64) dst[c] = __float2bfloat16_rn(0.f);
  } else if (r < ROWS) {   // rows past M: zeros, so that the tensor-core tile holds nothing undefined
    for (int c = first; c < (kpad >> 2); c += 64) *reinterpret_cast<uint2*>(dst + 4 * c) = make_uint2(0u, 0u);
  }
  __syncthreads();
}

template <typename TO>
__global__ void __launch_bounds__(THREADS, 2)
gemm_ln_small_m_kernel(const float* x, int ldx, const float* __restrict__ gamma, const float* __restrict__ beta, float eps,
                       const __nv_bfloat16* __restrict__ W, const float* __restrict__ bias, TO* __restrict__ C, int ldc, int M,
                       int N, int K, int act, const void* next_w, unsigned long long next_bytes) {
  extern __shared__ __align__(16) unsigned char smem[];
  const int kpad = (K + 31) & ~31, pitch = kpad + 8;   // 16 bytes of padding keep the eight rows' fragment loads off each other's banks
  __nv_bfloat16* h = reinterpret_cast<__nv_bfloat16*>(smem);
  float* red = reinterpret_cast<float*>(smem + (size_t)ROWS * pitch * 2);   // [WARPS][ROWS][RS]
  float* stat = red + (size_t)WARPS * ROWS * RS;                            // [2][WARPS]
  float* gb = stat + 2 * WARPS;                                             // gamma [K], beta [K]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int group = warp / GROUP_WARPS, gw = warp % GROUP_WARPS, gtid = threadIdx.x % (GROUP_WARPS * 32);
  const int g = lane >> 2, t = lane & 3;
  const int n0 = ((int)blockIdx.x * GROUPS + group) * COLS;
  const bool has_columns = n0 < N;
  const int nkb = (K + 31) / 32;

  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  const __nv_bfloat16* wrow[NT];
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    const int n = min(n0 + j * 8 + g, N - 1);  // rows past N are clamped; their columns are never stored
    wrow[j] = W + (size_t)n * K + t * 8;
  }
  pdl_trigger();
  // The weights of the product that runs after this one start towards L2 now, and so does the first round of this
  // group's own weights: they are on their way while the kernels ahead finish and the rows are normalised.
  if (threadIdx.x == 0) prefetch_share(next_w, next_bytes, blockIdx.x, gridDim.x);
  if (has_columns && gtid < COLS && n0 + gtid < N) prefetch_l2(W + (size_t)(n0 + gtid) * K, (unsigned)K * 2u);
  // the norm's weight and bias come into shared memory meanwhile
  for (int c = threadIdx.x; c < (K >> 2); c += THREADS) {
    reinterpret_cast<float4*>(gb)[c] = __ldg(reinterpret_cast<const float4*>(gamma) + c);
    reinterpret_cast<float4*>(gb + K)[c] = __ldg(reinterpret_cast<const float4*>(beta) + c);
  }
  float bias0 = 0.f;
  {
    const int n = n0 + gtid % COLS;
    if (bias && n < N) bias0 = bias[n];
  }
  pdl_wait();   // x comes from the kernels before
  if ((K >> 2) <= 64 * REG_VEC) normalise_rows<true>(x, ldx, gb, gb + K, eps, M, K, kpad, pitch, h, stat);
  else normalise_rows<false>(x, ldx, gb, gb + K, eps, M, K, kpad, pitch, h, stat);
  if (!has_columns) return;   // the block's second group when the columns run out; no barrier of the whole block follows

  const __nv_bfloat16* arow = h + (size_t)g * pitch + t * 8;
  for (int kb0 = gw; kb0 < nkb; kb0 += GROUP_WARPS * UNROLL) {
    uint4 wv[UNROLL][NT];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int kb = kb0 + u * GROUP_WARPS;
      const bool kin = kb < nkb && kb * 32 + t * 8 < K;
#pragma unroll
      for (int j = 0; j < NT; ++j) wv[u][j] = kin ? ldg_stream(wrow[j] + kb * 32) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int kb = kb0 + u * GROUP_WARPS;
      const uint4 av = kb < nkb ? *reinterpret_cast<const uint4*>(arow + kb * 32) : make_uint4(0, 0, 0, 0);
      // physical k = t*8 + s*4 + {0,1} plays the fragment's k = 2t + {0,1}; + {2,3} plays 2t + 8 + {0,1};
      // the tile's rows 8..15 (a1, a3) are zeros
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        mma_bf16_16816(acc[j], av.x, 0u, av.y, 0u, wv[u][j].x, wv[u][j].y);
        mma_bf16_16816(acc[j], av.z, 0u, av.w, 0u, wv[u][j].z, wv[u][j].w);
      }
    }
  }
  // partial sums of the group's warps -> shared memory; c0, c1: row g, columns 2t, 2t+1
  float* mine = red + (size_t)warp * ROWS * RS;
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    mine[g * RS + j * 8 + 2 * t] = acc[j][0];
    mine[g * RS + j * 8 + 2 * t + 1] = acc[j][1];
  }
  group_sync(group);
  // a group's 256 threads are a multiple of COLS, so a thread meets the same column at every idx it takes
  const float* sums = red + (size_t)group * GROUP_WARPS * ROWS * RS;
  for (int idx = gtid; idx < M * COLS; idx += GROUP_WARPS * 32) {
    const int m = idx / COLS, c = idx % COLS;
    const int n = n0 + c;
    if (n >= N) continue;
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < GROUP_WARPS; ++w) v += sums[((size_t)w * ROWS + m) * RS + c];
    from_f32(C[(size_t)m * ldc + n], activate(v + bias0, act));
  }
}

template <typename TO>
static int launch(const float* x, int ldx, const float* gamma, const float* beta, float eps, const void* W, const float* bias,
                  void* C, int ldc, int M, int N, int K, int act, const void* next_w, unsigned long long next_bytes,
                  cudaStream_t st) {
  const int kpad = (K + 31) & ~31;
  const size_t smem = (size_t)ROWS * (kpad + 8) * 2 + ((size_t)WARPS * ROWS * RS + 2 * WARPS + 2 * (size_t)K) * sizeof(float);
  auto kern = gemm_ln_small_m_kernel<TO>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int units = (N + COLS - 1) / COLS, blocks = (units + GROUPS - 1) / GROUPS;
  return (int)launch_pdl(kern, dim3(blocks), dim3(THREADS), smem, st, x, ldx, gamma, beta, eps, (const __nv_bfloat16*)W, bias,
                         (TO*)C, ldc, M, N, K, act, next_w, next_bytes);
}

}  // namespace gln
}  // namespace cbis

using namespace cbis;

// The widest row taken: its normalised copy (16 bytes of shared memory per element of K, for the 8 rows) and the
// norm's weight and bias (8 bytes) have to fit beside the sums in a block's shared memory.
CBIS_EXPORT int cbis_gemm_ln_small_m_max_k() { return 8192; }

// x [M, ldx>=K] float, gamma/beta [K] float, W [N, K] bfloat16, bias [N] float or null, C [M, ldc>=N] bfloat16 or float.
// Takes M <= 8, K a multiple of 8 up to cbis_gemm_ln_small_m_max_k(), 16-byte aligned operands; refuses anything else.
CBIS_EXPORT int cbis_gemm_ln_small_m(const float* x, int ldx, const float* gamma, const float* beta, float eps, const void* W,
                                     const float* bias, void* C, int ldc, int M, int N, int K, int act, int out_dtype,
                                     const void* next_w, unsigned long long next_bytes, void* stream) {
  if (M <= 0 || N <= 0) return CBIS_OK;
  if (M > gln::ROWS || K <= 0 || K % 8 || K > cbis_gemm_ln_small_m_max_k() || ldx < K || ldx % 4 || ldc < N) return CBIS_ERR_BAD_SIZE;
  if (((uintptr_t)x & 15) || ((uintptr_t)W & 15) || ((uintptr_t)gamma & 15) || ((uintptr_t)beta & 15) || ((uintptr_t)next_w & 15))
    return CBIS_ERR_ALIGNMENT;
  cudaStream_t st = (cudaStream_t)stream;
  if (out_dtype == CBIS_BF16)
    return gln::launch<__nv_bfloat16>(x, ldx, gamma, beta, eps, W, bias, C, ldc, M, N, K, act, next_w, next_bytes, st);
  if (out_dtype == CBIS_F32)
    return gln::launch<float>(x, ldx, gamma, beta, eps, W, bias, C, ldc, M, N, K, act, next_w, next_bytes, st);
  return CBIS_ERR_BAD_DTYPE;
}
