// Matrix product for few rows (decoding) on the 5th-generation tensor cores, with the operands swapped:
//   C[M,N] = act(A[M,K] * W^T + bias),   W [N,K] bfloat16 (K contiguous), A [M,K] bfloat16, M <= 64
// At these sizes the product is bound by reading W once from HBM.  A block owns 128 rows of W (128 output
// columns) over a share of K; the 128 rows of W are the M side of tcgen05.mma (128 x NT x 16, NT = 16, 32 or 64
// padded rows of A as its N side), so that the weights stream through shared memory by TMA in pieces of 16 KB,
// four or five of them in flight per block and two blocks per SM: over 100 KB per SM on their way with no
// register spent on them, where the mma.sync kernel (gemm_small_m.cu) keeps 32 KB per block in registers and
// pays a round trip to HBM for each batch.  The weights of the first stages are requested BEFORE the kernel
// waits for its predecessor (they depend on nothing), so they are in shared memory when A arrives.
//
// K is split over the blocks of a cluster (1, 2, 4 or 8) so that even a product with few output columns puts
// enough blocks on the machine; the blocks of a cluster hand their 128 x NT partial sums to the first through
// distributed shared memory (into its weight stages, once it says they are free), and the first adds them up,
// adds the bias, applies the activation to the 32-bit sums, rounds once and stores.
// The reference calls cublasSgemm and adds the bias in a second kernel and the GELU in a third
// (kernels/linear.cu:15-34, kernels/elementwise.cu:59-66).
//
// Every wait on an mbarrier is bounded; when one runs out the block sets *error and goes on to the end.
#include "common.cuh"

#include <cuda.h>
#include <mutex>

namespace cbis {
namespace fr {

constexpr int BW = 128, BK = 64;
constexpr int W_BYTES = BW * BK * 2;                 // 16 KB of weights per stage
constexpr int THREADS = 192;                         // warp 0: TMA, warp 1: MMA + tensor memory, warps 2..5: epilogue
constexpr unsigned SPIN_LIMIT = 1u << 21;            // tries of up to 1 us each

template <int NT> struct Shape {
  static constexpr int A_BYTES = NT * BK * 2;
  static constexpr int STAGE_BYTES = W_BYTES + A_BYTES;
  static constexpr int STAGES = NT == 64 ? 4 : 5;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;   // + alignment slack + barriers
};

__device__ __forceinline__ unsigned s32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void bar_init(void* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(bar)), "r"(count));
}
__device__ __forceinline__ void bar_expect(void* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool bar_wait(void* bar, unsigned parity) {
  const unsigned a = s32(bar);
  for (unsigned it = 0; it < SPIN_LIMIT; ++it) {
    unsigned ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\nselp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(a), "r"(parity), "r"(1000u) : "memory");
    if (ok) return true;
  }
  return false;
}
__device__ __forceinline__ void tma_2d(void* smem, const CUtensorMap* map, int x, int y, void* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(s32(smem)), "l"(map), "r"(x), "r"(y), "r"(s32(bar)) : "memory");
}
// K-major operand: rows of 128 bytes, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ unsigned long long desc_kmajor(const void* smem) {
  unsigned long long d = 0;
  d |= (unsigned long long)((s32(smem) & 0x3FFFF) >> 4);
  d |= (unsigned long long)1 << 16;
  d |= (unsigned long long)(1024 >> 4) << 32;
  d |= (unsigned long long)1 << 46;
  d |= (unsigned long long)2 << 61;
  return d;
}
// D = F32, A = B = BF16, both K-major, M = 128, N = n.
__host__ __device__ constexpr unsigned idesc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(BW >> 4) << 24);
}
__device__ __forceinline__ void mma(unsigned tmem_d, unsigned long long da, unsigned long long db, unsigned id, unsigned accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.u32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
               ::"r"(tmem_d), "l"(da), "l"(db), "r"(id), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void commit(void* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld16(unsigned taddr, float* v) {
  unsigned r[16];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                 "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// grid: (N tiles of 128) * ksplit blocks, clusters of ksplit along x.  Thread t of an epilogue warp owns output
// column n0 + 32 * (warp % 4) + lane: lane t of that quarter of tensor memory holds its NT sums, one per row of A.
template <int NT, typename TO>
__global__ void __launch_bounds__(THREADS, 2)
gemm_few_rows_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
                     const float* __restrict__ bias, TO* C, int ldc, int M, int N, int K, int act, int ksplit,
                     const void* next_w, unsigned long long next_bytes, int* error) {
  using S = Shape<NT>;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned long long* full = reinterpret_cast<unsigned long long*>(tiles + S::STAGES * S::STAGE_BYTES);
  unsigned long long* empty = full + S::STAGES;
  unsigned long long* acc_full = empty + S::STAGES;
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(acc_full + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  unsigned rank = 0;
  if (ksplit > 1) asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  const int n0 = ((int)blockIdx.x / ksplit) * BW;
  const int nk = (K + BK - 1) / BK;
  const int k_first = (int)((long long)nk * rank / ksplit), k_end = (int)((long long)nk * (rank + 1) / ksplit);
  const int steps = k_end - k_first;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S::STAGES; ++s) {
      bar_init(&full[s], 1);
      bar_init(&empty[s], 1);
    }
    bar_init(acc_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    // the weights of the product that runs after this one start towards L2 now
    prefetch_share(next_w, next_bytes, blockIdx.x, gridDim.x);
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(tmem_slot)), "r"(NT < 32 ? 32 : NT) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_d = *tmem_slot;
  pdl_trigger();   // only now that the block holds its tensor memory

  if (warp == 0) {
    if (lane == 0) {
      // the first stages' weights depend on no earlier kernel: they are on their way before the wait
      const int ahead = min(steps, S::STAGES);
      for (int i = 0; i < ahead; ++i) {
        bar_expect(&full[i], S::STAGE_BYTES);
        tma_2d(tiles + i * S::STAGE_BYTES, &map_w, (k_first + i) * BK, n0, &full[i]);
      }
      pdl_wait();   // A comes from the kernel before
      for (int i = 0; i < ahead; ++i)
        tma_2d(tiles + i * S::STAGE_BYTES + W_BYTES, &map_a, (k_first + i) * BK, 0, &full[i]);
      for (int i = ahead; i < steps; ++i) {
        const int s = i % S::STAGES;
        if (!bar_wait(&empty[s], ((i / S::STAGES) - 1) & 1)) { atomicExch(error, 41); break; }
        bar_expect(&full[s], S::STAGE_BYTES);
        tma_2d(tiles + s * S::STAGE_BYTES, &map_w, (k_first + i) * BK, n0, &full[s]);
        tma_2d(tiles + s * S::STAGE_BYTES + W_BYTES, &map_a, (k_first + i) * BK, 0, &full[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const unsigned long long dw = desc_kmajor(tiles), da = desc_kmajor(tiles + W_BYTES);
      bool ok = true;
      for (int i = 0; i < steps; ++i) {
        const int s = i % S::STAGES;
        if (!bar_wait(&full[s], (i / S::STAGES) & 1)) { atomicExch(error, 42); ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned off = (unsigned)((s * S::STAGE_BYTES) >> 4);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k)   // 16 elements = 32 bytes further along K inside the swizzled row
          mma(tmem_d, dw + off + (unsigned)(k * 2), da + off + (unsigned)(k * 2), idesc(NT), (i > 0 || k > 0) ? 1u : 0u);
        commit(&empty[s]);
      }
      if (ok) commit(acc_full);   // arrives when every product issued so far has finished
    }
  }
  // ---- the sums: from tensor memory, through the first block of the cluster, to C ---------------------------
  const bool epi = warp >= 2;
  const int quarter = warp & 3;                      // warps 2..5 read quarters 2, 3, 0, 1 of tensor memory
  const int col = quarter * 32 + lane;               // this thread's output column within the tile
  float v[NT];
#pragma unroll
  for (int i = 0; i < NT; ++i) v[i] = 0.f;
  if (epi && steps > 0) {
    if (!bar_wait(acc_full, 0)) {
      atomicExch(error, 43);
    } else {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
      for (int c0 = 0; c0 < NT; c0 += 16) tmem_ld16(tmem_d + ((unsigned)(quarter * 32) << 16) + (unsigned)c0, v + c0);
    }
  }
  if (!epi && warp == 0 && steps == 0) pdl_wait();   // (a block without a share of K still honours the order)
  if (ksplit > 1) {
    // The first block's weight stages take the others' sums: [sender][NT / 4][128 columns][4 floats], so that a
    // thread writes and reads 16 bytes next to its neighbours'.  They are free once the first block's products
    // have all finished, which its epilogue threads know when they get here.
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    cluster_sync_all();
    if (epi && rank != 0) {
      unsigned remote;
      asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(remote) : "r"(s32(tiles)));
      remote += (rank - 1) * (unsigned)(BW * NT * 4);
#pragma unroll
      for (int i = 0; i < NT; i += 4)
        asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};"
                     ::"r"(remote + (unsigned)(((i >> 2) * BW + col) * 16)), "f"(v[i]), "f"(v[i + 1]), "f"(v[i + 2]), "f"(v[i + 3])
                     : "memory");
    }
    cluster_sync_all();
    if (epi && rank == 0) {
      for (int r = 1; r < ksplit; ++r) {
        const float4* src = reinterpret_cast<const float4*>(tiles + (size_t)(r - 1) * (BW * NT * 4));
#pragma unroll
        for (int i = 0; i < NT; i += 4) {
          const float4 t = src[(i >> 2) * BW + col];
          v[i] += t.x; v[i + 1] += t.y; v[i + 2] += t.z; v[i + 3] += t.w;
        }
      }
    }
  }
  if (epi && rank == 0) {
    const int n = n0 + col;
    if (n < N) {
      const float b = bias ? bias[n] : 0.f;
#pragma unroll
      for (int m = 0; m < NT; ++m)
        if (m < M) from_f32(C[(size_t)m * ldc + n], activate(v[m] + b, act));
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(NT < 32 ? 32 : NT) : "memory");
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encoder() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}
// [rows, K] bfloat16 with row pitch ld elements; boxes of 64 columns x box_rows rows, 128-byte swizzle; what lies
// outside the matrix reads as zero.
static int make_map(CUtensorMap* map, const void* ptr, int rows, int K, int ld, int box_rows) {
  EncodeTiledFn fn = encoder();
  if (!fn) return CBIS_ERR_BAD_SIZE;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? CBIS_OK : CBIS_ERR_BAD_SIZE;
}

template <int NT, typename TO>
static int launch(const CUtensorMap& map_w, const CUtensorMap& map_a, const float* bias, void* C, int ldc, int M, int N, int K,
                  int act, int ksplit, const void* next_w, unsigned long long next_bytes, int* error, cudaStream_t st) {
  auto kern = gemm_few_rows_kernel<NT, TO>;
  const size_t smem = Shape<NT>::SMEM_BYTES;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
  if (e != cudaSuccess) return (int)e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(((N + BW - 1) / BW) * ksplit));
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled();
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = (unsigned)ksplit;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return (int)cudaLaunchKernelEx(&cfg, kern, map_w, map_a, bias, (TO*)C, ldc, M, N, K, act, ksplit, next_w, next_bytes, error);
}

}  // namespace fr
}  // namespace cbis

using namespace cbis;

// A [M, lda>=K] and W [N, K] bfloat16 (K contiguous, K and lda multiples of 8, 16-byte aligned), bias [N] float or
// null, C [M, ldc>=N] bfloat16 or float, M <= 64.  ksplit: 1, 2, 4 or 8 blocks share K (0: chosen here).
// next_w / next_bytes: weights of the product that will run after this one, prefetched into L2, or null.
// error: int on the device, set non-zero if a wait inside the kernel ran out.
CBIS_EXPORT int cbis_gemm_few_rows_tc5(const void* A, int lda, const void* W, const float* bias, void* C, int ldc, int M,
                                       int N, int K, int act, int out_dtype, int ksplit, const void* next_w,
                                       unsigned long long next_bytes, int* error, void* stream) {
  if (M <= 0 || N <= 0) return CBIS_OK;
  if (M > 64 || K <= 0 || K % 8 || lda % 8 || lda < K || ldc < N) return CBIS_ERR_BAD_SIZE;
  if (((uintptr_t)A & 15) || ((uintptr_t)W & 15) || ((uintptr_t)next_w & 15) || error == nullptr) return CBIS_ERR_ALIGNMENT;
  const int nt = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
  const int nk = (K + fr::BK - 1) / fr::BK, tiles = (N + fr::BW - 1) / fr::BW;
  // the sums of the other blocks must fit into the first block's weight stages
  const int stages = nt == 64 ? 4 : 5;
  const int most = 1 + (stages * (fr::W_BYTES + nt * fr::BK * 2)) / (fr::BW * nt * 4);
  if (ksplit <= 0) {
    // enough blocks for two on every SM, every block with at least four steps of K
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    ksplit = 1;
    while (ksplit < 8 && tiles * ksplit * 2 <= 2 * sms && nk / (ksplit * 2) >= 4 && ksplit * 2 <= most) ksplit *= 2;
  }
  if ((ksplit != 1 && ksplit != 2 && ksplit != 4 && ksplit != 8) || ksplit > most || ksplit > nk) return CBIS_ERR_BAD_SIZE;
  CUtensorMap map_w, map_a;
  int st = fr::make_map(&map_w, W, N, K, K, fr::BW);
  if (st != CBIS_OK) return st;
  st = fr::make_map(&map_a, A, M, K, lda, nt);
  if (st != CBIS_OK) return st;
  cudaStream_t s = (cudaStream_t)stream;
#define CBIS_FR(NT_)                                                                                                  \
  if (nt == NT_) {                                                                                                    \
    if (out_dtype == CBIS_BF16)                                                                                       \
      return fr::launch<NT_, __nv_bfloat16>(map_w, map_a, bias, C, ldc, M, N, K, act, ksplit, next_w, next_bytes, error, s); \
    if (out_dtype == CBIS_F32)                                                                                        \
      return fr::launch<NT_, float>(map_w, map_a, bias, C, ldc, M, N, K, act, ksplit, next_w, next_bytes, error, s);  \
    return CBIS_ERR_BAD_DTYPE;                                                                                        \
  }
  CBIS_FR(16)
  CBIS_FR(32)
  CBIS_FR(64)
#undef CBIS_FR
  return CBIS_ERR_BAD_SIZE;
}
