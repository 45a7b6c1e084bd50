// Matrix product for few rows (decoding: M <= 64) in bfloat16 with 32-bit accumulation:
//   C[M,N] = act(A[M,K] * W^T + bias),   W stored [N,K] (K contiguous), A [M,K]
// At these sizes the product is bound by reading W once from HBM, so the kernel is built
// around the weight stream: a block owns 8*NT output columns over the whole of K; its 8 warps
// take the 32-wide K blocks in turn (warp w: blocks w, w+8, ...), so together they read each
// weight row in long contiguous runs; every lane fetches 16 bytes of a weight row per block and
// feeds them to the tensor cores as they come (mma.sync m16n8k16, the K order permuted alike
// for both operands so that one 16-byte load is two fragments); the few rows of A come from
// L1/L2.  The warps' partial sums are added in shared memory and bias and activation are
// applied to the 32-bit sum before the one store.  The reference calls cublasSgemm and adds
// the bias in a second kernel and the GELU in a third (kernels/linear.cu:15-34,
// kernels/elementwise.cu:59-66).
#include "common.cuh"

namespace cbis {

constexpr int SM_WARPS = 8;

__device__ __forceinline__ void mma_bf16_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ unsigned cluster_ctarank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// The address, in the cluster's shared-memory window, of `p` (a shared-memory address of this block) in the block `rank`.
__device__ __forceinline__ unsigned in_cluster_block(const void* p, unsigned rank) {
  unsigned r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"((unsigned)__cvta_generic_to_shared(p)), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_cluster_f32(unsigned addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// MT: 16-row tiles of A (M <= 16*MT); NT: 8-column tiles of W per block; UNROLL: K blocks in flight per warp.
// LOW8: M <= 8, so rows 8..15 of the one row tile do not exist: their fragments are zeros and are never loaded
// (fewer registers: four blocks fit on an SM instead of three).
// CLUSTER: the kernel is launched in clusters of `ksplit` blocks that share a block's columns and split K.  (A kernel that
// holds cluster instructions is launched through the cluster scheduler even when it never runs them, which was measured
// to cost the plain form a third of its speed: the two forms are separate kernels.)
template <int MT, int NT, int UNROLL, bool LOW8, typename TO, bool CLUSTER = false>
__device__ __forceinline__ void gemm_small_m_body(const __nv_bfloat16* A, int lda, const __nv_bfloat16* __restrict__ W,
                                                  const float* __restrict__ bias, TO* __restrict__ C, int ldc, int M,
                                                  int N, int K, int act, const void* next_w,
                                                  unsigned long long next_bytes, int ksplit, int accumulate) {
  extern __shared__ float red[];  // [SM_WARPS][MT*16][NT*8 + 1], then [ksplit - 1][MT*16 * NT*8] for the other blocks' sums
  constexpr int RS = NT * 8 + 1;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  // ksplit > 1: a cluster of ksplit blocks shares the block's columns; each takes a run of the 32-wide K blocks
  int rank = 0;
  if constexpr (CLUSTER) rank = (int)cluster_ctarank();
  else ksplit = 1;
  const int n0 = (blockIdx.x / ksplit) * (NT * 8);
  const int nkb_all = (K + 31) / 32;
  const int per_rank = (nkb_all + ksplit - 1) / ksplit;
  const int kb_first = rank * per_rank;
  const int nkb = min(nkb_all, kb_first + per_rank);

  float acc[MT][NT][4];
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[i][j][c] = 0.f;

  const __nv_bfloat16* wrow[NT];
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    const int n = min(n0 + j * 8 + g, N - 1);  // rows past N are clamped; their columns are never stored
    wrow[j] = W + (size_t)n * K + t * 8;
  }
  const __nv_bfloat16* arow[MT][2];
  bool avalid[MT][2];
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int hlf = 0; hlf < 2; ++hlf) {
      const int m = i * 16 + hlf * 8 + g;
      avalid[i][hlf] = m < M;
      arow[i][hlf] = A + (size_t)min(m, M - 1) * lda + t * 8;
    }

  pdl_trigger();
  // The weights of the product that runs after this one start towards L2 now: by the time that kernel
  // starts it reads them from L2, and HBM keeps streaming while the short kernels in between run.
  if (threadIdx.x == 0) prefetch_share(next_w, next_bytes, blockIdx.x, gridDim.x);
  // the bias of this thread's first output column is fetched now (the epilogue maps idx -> column idx % (NT*8))
  float bias0 = 0.f;
  {
    const int n = n0 + (int)(threadIdx.x % (NT * 8));
    if (bias && n < N) bias0 = bias[n];
  }
  bool waited = false;
  for (int kb0 = kb_first + warp; kb0 < nkb; kb0 += SM_WARPS * UNROLL) {
    uint4 wv[UNROLL][NT], av[UNROLL][MT][LOW8 ? 1 : 2];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int kb = kb0 + u * SM_WARPS;
      const bool kin = kb < nkb && kb * 32 + t * 8 < K;
#pragma unroll
      for (int j = 0; j < NT; ++j) wv[u][j] = kin ? ldg_stream(wrow[j] + kb * 32) : make_uint4(0, 0, 0, 0);
    }
    if (!waited) {  // the first batch of weights is on its way before the kernels ahead have finished
      pdl_wait();
      waited = true;
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int kb = kb0 + u * SM_WARPS;
      const bool kin = kb < nkb && kb * 32 + t * 8 < K;
#pragma unroll
      for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int hlf = 0; hlf < (LOW8 ? 1 : 2); ++hlf)
          av[u][i][hlf] = (kin && avalid[i][hlf]) ? __ldcg(reinterpret_cast<const uint4*>(arow[i][hlf] + kb * 32))
                                                   : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
#pragma unroll
      for (int i = 0; i < MT; ++i) {
        // physical k = t*8 + s*4 + {0,1} plays the fragment's k = 2t + {0,1}; + {2,3} plays 2t + 8 + {0,1}
        const uint4 lo = av[u][i][0];
        const uint4 hi = LOW8 ? make_uint4(0, 0, 0, 0) : av[u][i][LOW8 ? 0 : 1];
        const uint32_t a_s0[4] = {lo.x, hi.x, lo.y, hi.y};
        const uint32_t a_s1[4] = {lo.z, hi.z, lo.w, hi.w};
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          mma_bf16_16816(acc[i][j], a_s0, wv[u][j].x, wv[u][j].y);
          mma_bf16_16816(acc[i][j], a_s1, wv[u][j].z, wv[u][j].w);
        }
      }
    }
  }

  if (!waited) pdl_wait();
  // partial sums of the warps -> shared memory; c0,c1: row g, cols 2t,2t+1; c2,c3: row g+8
  float* mine = red + (size_t)warp * (MT * 16) * RS;
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      mine[(i * 16 + g) * RS + j * 8 + 2 * t] = acc[i][j][0];
      mine[(i * 16 + g) * RS + j * 8 + 2 * t + 1] = acc[i][j][1];
      mine[(i * 16 + g + 8) * RS + j * 8 + 2 * t] = acc[i][j][2];
      mine[(i * 16 + g + 8) * RS + j * 8 + 2 * t + 1] = acc[i][j][3];
    }
  __syncthreads();
  float* others = red + (size_t)SM_WARPS * (MT * 16) * RS;   // [ksplit - 1][MT*16 * NT*8], in the cluster's first block
  if constexpr (CLUSTER) {
   if (rank > 0) {
    // this block's sums go into the first block's shared memory; it adds them after the cluster has met
    const unsigned base = in_cluster_block(others + (size_t)(rank - 1) * (MT * 16) * (NT * 8), 0);
    for (int idx = threadIdx.x; idx < M * (NT * 8); idx += blockDim.x) {
      const int m = idx / (NT * 8), c = idx % (NT * 8);
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < SM_WARPS; ++w) v += red[((size_t)w * (MT * 16) + m) * RS + c];
      st_cluster_f32(base + (unsigned)idx * 4u, v);
    }
   }
   cluster_sync();
   if (rank > 0) return;
  }
  // blockDim (256) is a multiple of NT*8, so a thread meets the same column at every idx it takes
  for (int idx = threadIdx.x; idx < M * (NT * 8); idx += blockDim.x) {
    const int m = idx / (NT * 8), c = idx % (NT * 8);
    const int n = n0 + c;
    if (n >= N) continue;
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < SM_WARPS; ++w) v += red[((size_t)w * (MT * 16) + m) * RS + c];
    if constexpr (CLUSTER)
      for (int r = 1; r < ksplit; ++r) v += others[(size_t)(r - 1) * (MT * 16) * (NT * 8) + idx];
    v += bias0;
    v = activate(v, act);
    if (accumulate) v += to_f32(C[(size_t)m * ldc + n]);   // C is the residual stream: written by earlier kernels, all behind the wait
    from_f32(C[(size_t)m * ldc + n], v);
  }
}

// Two entry points over the same body: the compiler's own register choice for the general form (80 registers,
// three blocks per SM), and a cap of 64 registers for the M <= 8 form so that four blocks fit.
template <int MT, int NT, int UNROLL, typename TO>
__global__ void __launch_bounds__(SM_WARPS * 32)
gemm_small_m_kernel(const __nv_bfloat16* A, int lda, const __nv_bfloat16* __restrict__ W,
                    const float* __restrict__ bias, TO* __restrict__ C, int ldc, int M, int N, int K, int act,
                    const void* next_w, unsigned long long next_bytes, int ksplit, int accumulate) {
  gemm_small_m_body<MT, NT, UNROLL, false, TO>(A, lda, W, bias, C, ldc, M, N, K, act, next_w, next_bytes, ksplit, accumulate);
}
template <int MT, int NT, int UNROLL, typename TO>
__global__ void __launch_bounds__(SM_WARPS * 32, 4)
gemm_small_m_low8_kernel(const __nv_bfloat16* A, int lda, const __nv_bfloat16* __restrict__ W,
                         const float* __restrict__ bias, TO* __restrict__ C, int ldc, int M, int N, int K, int act,
                         const void* next_w, unsigned long long next_bytes, int ksplit, int accumulate) {
  gemm_small_m_body<MT, NT, UNROLL, true, TO>(A, lda, W, bias, C, ldc, M, N, K, act, next_w, next_bytes, ksplit, accumulate);
}
template <int MT, int NT, int UNROLL, typename TO>
__global__ void __launch_bounds__(SM_WARPS * 32, 4)
gemm_small_m_low8_ksplit_kernel(const __nv_bfloat16* A, int lda, const __nv_bfloat16* __restrict__ W,
                                const float* __restrict__ bias, TO* __restrict__ C, int ldc, int M, int N, int K, int act,
                                const void* next_w, unsigned long long next_bytes, int ksplit, int accumulate) {
  gemm_small_m_body<MT, NT, UNROLL, true, TO, true>(A, lda, W, bias, C, ldc, M, N, K, act, next_w, next_bytes, ksplit, accumulate);
}

template <int MT, int NT, int UNROLL, bool LOW8, typename TO>
static int launch_small_m(const void* A, int lda, const void* W, const float* bias, void* C, int ldc, int M, int N,
                          int K, int act, const void* next_w, unsigned long long next_bytes, cudaStream_t st, int accumulate,
                          int ksplit = 1) {
  const size_t smem = ((size_t)SM_WARPS * MT * 16 * (NT * 8 + 1) + (size_t)(ksplit - 1) * MT * 16 * NT * 8) * sizeof(float);
  void (*kern)(const __nv_bfloat16*, int, const __nv_bfloat16*, const float*, TO*, int, int, int, int, int, const void*,
               unsigned long long, int, int);
  if constexpr (LOW8) kern = ksplit > 1 ? gemm_small_m_low8_ksplit_kernel<MT, NT, UNROLL, TO> : gemm_small_m_low8_kernel<MT, NT, UNROLL, TO>;
  else kern = gemm_small_m_kernel<MT, NT, UNROLL, TO>;
  if (!LOW8 && ksplit > 1) return CBIS_ERR_BAD_SIZE;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int blocks = (N + NT * 8 - 1) / (NT * 8) * ksplit;
  if (ksplit == 1)
    return (int)launch_pdl(kern, dim3(blocks), dim3(SM_WARPS * 32), smem, st, (const __nv_bfloat16*)A, lda,
                           (const __nv_bfloat16*)W, bias, (TO*)C, ldc, M, N, K, act, next_w, next_bytes, 1, accumulate);
  // clusters of ksplit blocks along x, launched like the others (programmatic dependent launch)
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(blocks);
  cfg.blockDim = dim3(SM_WARPS * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled();
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = ksplit;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return (int)cudaLaunchKernelEx(&cfg, kern, (const __nv_bfloat16*)A, lda, (const __nv_bfloat16*)W, bias, (TO*)C, ldc, M, N, K,
                                 act, next_w, next_bytes, ksplit, accumulate);
}

// CBIS_SMALL_M_KSPLIT=0: K is never split over the blocks of a cluster.
static int ksplit_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("CBIS_SMALL_M_KSPLIT");
    on = (e && e[0] == '0') ? 0 : 1;
  }
  return on;
}

template <typename TO>
static int dispatch_small_m(const void* A, int lda, const void* W, const float* bias, void* C, int ldc, int M, int N,
                            int K, int act, const void* next_w, unsigned long long next_bytes, cudaStream_t st, int accumulate) {
  // Few columns and a long K (the feed-forward's second product: 2,048 x 8,192): 8 columns per block would leave
  // each warp 32 K blocks to walk in four dependent rounds.  Then 16 columns per block and K over the 2 or 4 blocks of
  // a cluster, whose sums meet in the first block's shared memory: one round per warp, as many blocks as before.
  if (M <= 8 && ksplit_enabled() && N < 148 * 2 * 16 && N >= 64) {
    const int tiles16 = (N + 15) / 16, nkb = (K + 31) / 32;
    int ks = 1;
    while (ks < 4 && tiles16 * ks * 2 <= 4 * 148 && nkb >= SM_WARPS * 4 * ks * 2) ks *= 2;
    if (ks > 1)
      return launch_small_m<1, 2, 4, true, TO>(A, lda, W, bias, C, ldc, M, N, K, act, next_w, next_bytes, st, accumulate, ks);
  }
  // Columns per block: 16 when that still gives the 148 SMs about two blocks each, else 8.
  const bool wide = N >= 148 * 2 * 16;
  // M <= 8 and more 16-column blocks than fit at three per SM (444): the 64-register form runs them in one round
  if (M <= 8 && wide && (N + 15) / 16 > 3 * 148 && (N + 15) / 16 <= 4 * 148)
    return launch_small_m<1, 2, 4, true, TO>(A, lda, W, bias, C, ldc, M, N, K, act, next_w, next_bytes, st, accumulate);
  if (M <= 16) {
    if (wide) return launch_small_m<1, 2, 4, false, TO>(A, lda, W, bias, C, ldc, M, N, K, act, next_w, next_bytes, st, accumulate);
    return launch_small_m<1, 1, 8, false, TO>(A, lda, W, bias, C, ldc, M, N, K, act, next_w, next_bytes, st, accumulate);
  }
  if (M <= 32) {
    if (wide) return launch_small_m<2, 2, 2, false, TO>(A, lda, W, bias, C, ldc, M, N, K, act, next_w, next_bytes, st, accumulate);
    return launch_small_m<2, 1, 4, false, TO>(A, lda, W, bias, C, ldc, M, N, K, act, next_w, next_bytes, st, accumulate);
  }
  if (wide) return launch_small_m<4, 2, 2, false, TO>(A, lda, W, bias, C, ldc, M, N, K, act, next_w, next_bytes, st, accumulate);
  return launch_small_m<4, 1, 2, false, TO>(A, lda, W, bias, C, ldc, M, N, K, act, next_w, next_bytes, st, accumulate);
}

}  // namespace cbis

using namespace cbis;

// A [M, lda>=K] bfloat16, W [N, K] bfloat16, bias [N] float or null, C [M, ldc>=N] bfloat16 or float.
// Takes M <= 64 and K a multiple of 8 with 16-byte aligned operands; refuses anything else.
// next_w / next_bytes: weights of the product that will run after this one (16-byte aligned), or null:
// they are prefetched into L2 while this kernel runs.  accumulate (32-bit C only): C += act(A W^T + bias).
CBIS_EXPORT int cbis_gemm_small_m_bf16(const void* A, int lda, const void* W, const float* bias, void* C, int ldc,
                                       int M, int N, int K, int act, int out_dtype, const void* next_w,
                                       unsigned long long next_bytes, int accumulate, void* stream) {
  if (M <= 0 || N <= 0) return CBIS_OK;
  if (M > 64 || K <= 0 || K % 8 || lda < K || ldc < N) return CBIS_ERR_BAD_SIZE;
  if (lda % 8 || ((uintptr_t)A & 15) || ((uintptr_t)W & 15) || ((uintptr_t)next_w & 15)) return CBIS_ERR_ALIGNMENT;
  cudaStream_t st = (cudaStream_t)stream;
  if (accumulate && out_dtype != CBIS_F32) return CBIS_ERR_BAD_DTYPE;   // sums are added into a 32-bit matrix only
  if (out_dtype == CBIS_BF16) return dispatch_small_m<__nv_bfloat16>(A, lda, W, bias, C, ldc, M, N, K, act, next_w, next_bytes, st, 0);
  if (out_dtype == CBIS_F32) return dispatch_small_m<float>(A, lda, W, bias, C, ldc, M, N, K, act, next_w, next_bytes, st, accumulate);
  return CBIS_ERR_BAD_DTYPE;
}
