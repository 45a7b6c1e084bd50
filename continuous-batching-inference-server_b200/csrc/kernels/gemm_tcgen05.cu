// Dense matrix product for many rows (prefill) on the 5th-generation tensor cores:
//   C[M,N] = act(A[M,K] * W^T + bias),   A [M,K] and W [N,K] bfloat16 with K contiguous
// A block computes 128 x 256 tiles, one after the other.  One thread streams 128x64 tiles of A and 256x64 tiles of W
// into shared memory with TMA (cp.async.bulk.tensor, 128-byte swizzle, four stages, mbarriers with
// transaction counts); one thread issues tcgen05.mma (M=128, N=256, K=16, bf16 in, 32-bit
// accumulate) with the accumulator in tensor memory (two of 256 columns, taking turns); four warps read
// the accumulator of the tile before back with tcgen05.ld (sixteen warps: the GELU of a tile costs more instructions than its products take cycles), add the bias and apply the activation on the 32-bit sums, round ONCE and
// store.  The reference does cublasSgemm, then a bias kernel, then a GELU kernel
// (kernels/linear.cu:15-34, kernels/elementwise.cu:59-66).
//
// Every wait on an mbarrier is bounded: when a limit runs out the block sets *error, stops issuing
// work, frees its tensor memory and returns.
#include "common.cuh"

#include <cuda.h>
#include <mutex>
#include <unordered_map>

namespace cbis {

constexpr int TC_BM = 128, TC_BN = 256, TC_BK = 64, TC_STAGES = 4;
constexpr int TC_A_BYTES = TC_BM * TC_BK * 2, TC_B_BYTES = TC_BN * TC_BK * 2;
constexpr int TC_STAGE_BYTES = TC_A_BYTES + TC_B_BYTES;
constexpr int TC_EPI_WARPS = 16;  // four per quarter of tensor memory, 64 columns each
constexpr int TC_THREADS = 64 + 32 * TC_EPI_WARPS;  // warp 0: TMA, warp 1: MMA + tensor-memory allocation, then the epilogue
constexpr unsigned TC_SPIN_LIMIT = 1u << 24;

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(void* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(void* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Waits for the phase with the given parity; false if the limit ran out.
__device__ __forceinline__ bool mbar_wait(void* bar, unsigned parity, unsigned limit = TC_SPIN_LIMIT) {
  const unsigned a = smem_u32(bar);
  for (unsigned it = 0; it < limit; ++it) {
    unsigned ok;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(a), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* smem, const CUtensorMap* map, int x, int y, void* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(smem)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
// Shared-memory matrix descriptor: K-major tile of 128-byte rows, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ unsigned long long umma_desc(const void* smem) {
  unsigned long long d = 0;
  d |= (unsigned long long)((smem_u32(smem) & 0x3FFFF) >> 4);       // start address
  d |= (unsigned long long)1 << 16;                                  // leading-dimension offset (unused with swizzle)
  d |= (unsigned long long)(1024 >> 4) << 32;                        // stride between 8-row groups
  d |= (unsigned long long)1 << 46;                                  // descriptor version of sm_100
  d |= (unsigned long long)2 << 61;                                  // 128-byte swizzle
  return d;
}
// Instruction descriptor: D = F32, A = B = BF16, both K-major, N and M of the tile.
__host__ __device__ constexpr unsigned umma_idesc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(m >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(unsigned tmem_d, unsigned long long da, unsigned long long db, unsigned idesc,
                                          unsigned accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.u32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(void* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(unsigned taddr, float* v) {
  unsigned r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ void tmem_ld16(unsigned taddr, float* v) {
  unsigned r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// NC (16 or 32) consecutive columns of one row: bias, activation, ONE rounding, 16-byte stores where the row allows.
template <typename TO, int NC = 32>
__device__ __forceinline__ void store_row32(TO* dst, const float* v, const float* __restrict__ bias, int n, int N,
                                            int act, bool vec_ok) {
  float x[NC];
  if (n + NC <= N) {
#pragma unroll
    for (int i = 0; i < NC; i += 4) {
      float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
      if (bias) {
        if (((uintptr_t)(bias + n) & 15) == 0) b = *reinterpret_cast<const float4*>(bias + n + i);
        else b = make_float4(bias[n + i], bias[n + i + 1], bias[n + i + 2], bias[n + i + 3]);
      }
      x[i] = activate(v[i] + b.x, act);
      x[i + 1] = activate(v[i + 1] + b.y, act);
      x[i + 2] = activate(v[i + 2] + b.z, act);
      x[i + 3] = activate(v[i + 3] + b.w, act);
    }
    if (vec_ok) {
      if constexpr (sizeof(TO) == 2) {
#pragma unroll
        for (int i = 0; i < NC; i += 8) {
          uint4 q;
          __nv_bfloat162 p0 = __floats2bfloat162_rn(x[i], x[i + 1]), p1 = __floats2bfloat162_rn(x[i + 2], x[i + 3]);
          __nv_bfloat162 p2 = __floats2bfloat162_rn(x[i + 4], x[i + 5]), p3 = __floats2bfloat162_rn(x[i + 6], x[i + 7]);
          q.x = *reinterpret_cast<unsigned*>(&p0);
          q.y = *reinterpret_cast<unsigned*>(&p1);
          q.z = *reinterpret_cast<unsigned*>(&p2);
          q.w = *reinterpret_cast<unsigned*>(&p3);
          *reinterpret_cast<uint4*>(dst + i) = q;
        }
      } else {
#pragma unroll
        for (int i = 0; i < NC; i += 4)
          *reinterpret_cast<float4*>(dst + i) = make_float4(x[i], x[i + 1], x[i + 2], x[i + 3]);
      }
      return;
    }
#pragma unroll
    for (int i = 0; i < NC; ++i) from_f32(dst[i], x[i]);
    return;
  }
  for (int i = 0; i < NC && n + i < N; ++i) from_f32(dst[i], activate(v[i] + (bias ? bias[n + i] : 0.f), act));
}

// Persistent: a block walks over tiles (tile, tile + gridDim.x, ...).  Two accumulators of 256 columns take
// turns in tensor memory, so the epilogue of one tile runs while the products of the next are issued.
template <typename TO>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    const float* __restrict__ bias, TO* __restrict__ C, int ldc, int M, int N, int K, int act,
                    int* error, unsigned spin_limit, int starve) {
  // spin_limit: tries of every wait before it gives up (TC_SPIN_LIMIT in service).  starve != 0 (tests of the
  // give-up path only): the loading thread requests nothing, so the waits for operands wait for a signal that
  // nothing sends, run out, and the block reports, frees its tensor memory and returns with no copy in flight.
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // stages first (each tile 1024-byte aligned for the swizzle), then the barriers
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned long long* full = reinterpret_cast<unsigned long long*>(tiles + TC_STAGES * TC_STAGE_BYTES);
  unsigned long long* empty = full + TC_STAGES;
  unsigned long long* acc_full = empty + TC_STAGES;    // [2]
  unsigned long long* acc_empty = acc_full + 2;         // [2]
  unsigned long long* drained = acc_empty + 2;          // [1]: the products issued before a give-up have finished
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(drained + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (M + TC_BM - 1) / TC_BM, n_tiles = (N + TC_BN - 1) / TC_BN;
  const int num_tiles = m_tiles * n_tiles;
  const int n_kt = (K + TC_BK - 1) / TC_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < TC_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b2 = 0; b2 < 2; ++b2) {
      mbar_init(&acc_full[b2], 1);
      mbar_init(&acc_empty[b2], TC_EPI_WARPS);   // one arrival per epilogue warp
    }
    mbar_init(drained, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {  // all of tensor memory: two accumulators of 256 columns (128 lanes x 32 bit each)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(2 * TC_BN)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_base = *tmem_slot;
  // The kernel after this one may start only now that this block holds its tensor memory: a block of a later
  // kernel that allocated first and then waited for this kernel to finish would wait for ever.
  pdl_trigger();
  pdl_wait();  // A comes from the kernel before

  if (warp == 0) {
    if (lane == 0) {
      unsigned it = 0;  // k-tiles loaded so far, over all tiles of this block
      for (int tile = blockIdx.x; tile < num_tiles && !*abort_flag && !starve; tile += gridDim.x) {
        const int m0 = (tile % m_tiles) * TC_BM, n0 = (tile / m_tiles) * TC_BN;
        for (int kt = 0; kt < n_kt; ++kt, ++it) {
          const unsigned s = it % TC_STAGES, round = it / TC_STAGES;
          if (round > 0 && !mbar_wait(&empty[s], (round - 1) & 1, spin_limit)) {
            *abort_flag = 1;
            atomicExch(error, 1);
            break;
          }
          if (*abort_flag) break;
          unsigned char* sa = tiles + s * TC_STAGE_BYTES;
          mbar_expect_tx(&full[s], TC_STAGE_BYTES);
          tma_load_2d(sa, &map_a, kt * TC_BK, m0, &full[s]);
          tma_load_2d(sa + TC_A_BYTES, &map_w, kt * TC_BK, n0, &full[s]);
        }
      }
      if (*abort_flag) {
        // a give-up somewhere in the block: the copies this thread requested last may still be on their way into
        // shared memory; the block must not leave before they have landed (waits with the full limit)
        for (unsigned j = it > (unsigned)TC_STAGES ? it - TC_STAGES : 0; j < it; ++j)
          if (!mbar_wait(&full[j % TC_STAGES], (j / TC_STAGES) & 1)) atomicExch(error, 5);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr unsigned idesc = umma_idesc(TC_BM, TC_BN);
      unsigned it = 0, local = 0;
      for (int tile = blockIdx.x; tile < num_tiles && !*abort_flag; tile += gridDim.x, ++local) {
        const unsigned buf = local & 1, use = local >> 1;
        if (use > 0 && !mbar_wait(&acc_empty[buf], (use - 1) & 1, spin_limit)) {   // the epilogue has read this accumulator
          *abort_flag = 4;
          atomicExch(error, 4);
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned tmem_d = tmem_base + buf * TC_BN;
        bool ok = true;
        for (int kt = 0; kt < n_kt; ++kt, ++it) {
          const unsigned s = it % TC_STAGES, round = it / TC_STAGES;
          if (!mbar_wait(&full[s], round & 1, spin_limit)) {
            *abort_flag = 2;
            atomicExch(error, 2);
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const unsigned char* sa = tiles + s * TC_STAGE_BYTES;
          const unsigned long long da = umma_desc(sa), db = umma_desc(sa + TC_A_BYTES);
#pragma unroll
          for (int k = 0; k < TC_BK / 16; ++k)  // 16 elements = 32 bytes further along K inside the swizzled row
            umma_bf16(tmem_d, da + (unsigned long long)(k * 2), db + (unsigned long long)(k * 2), idesc,
                      (kt > 0 || k > 0) ? 1u : 0u);
          umma_commit(&empty[s]);  // the stage is free again when these products have read it
        }
        if (!ok) break;
        umma_commit(&acc_full[buf]);  // arrives when every product issued so far has finished
      }
      if (*abort_flag) {
        // products issued before the give-up may still run: tensor memory is freed only after they have finished
        umma_commit(drained);
        if (!mbar_wait(drained, 0)) atomicExch(error, 6);
      }
    }
  } else {
    // epilogue: a warp can read the 32 lanes of the quarter of tensor memory given by its index % 4; the
    // warps of a quarter split the 256 columns among them
    const int quarter = warp & 3;
    constexpr int COLS = TC_BN / (TC_EPI_WARPS / 4);
    const int col_first = ((warp - 2) >> 2) * COLS;
    const bool vec_ok = (ldc * sizeof(TO)) % 16 == 0 && ((uintptr_t)C & 15) == 0;
    unsigned local = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
      const int m0 = (tile % m_tiles) * TC_BM, n0 = (tile / m_tiles) * TC_BN;
      const unsigned buf = local & 1, use = local >> 1;
      const int row = m0 + quarter * 32 + lane;
      if (!mbar_wait(&acc_full[buf], use & 1, spin_limit)) {
        atomicExch(error, 3);
        break;
      }
      if (*abort_flag) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      for (int c0 = col_first; c0 < col_first + COLS; c0 += 32) {
        if (n0 + c0 >= N) break;
        float v[32];
        tmem_ld32(tmem_base + ((unsigned)(quarter * 32) << 16) + buf * TC_BN + (unsigned)c0, v);
        if (row < M) store_row32<TO>(C + (size_t)row * ldc + n0 + c0, v, bias, n0 + c0, N, act, vec_ok && ((n0 + c0) * sizeof(TO)) % 16 == 0);
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&acc_empty[buf])) : "memory");
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * TC_BN) : "memory");
  }
}

// ---- the same product on PAIRS of blocks (cta_group::2) -------------------------------------------
// Two blocks of a cluster, on the two SMs of one TPC, compute a 256 x 256 tile together.  Each loads ITS 128 rows
// of A and ITS 128 of the 256 rows of W per k-tile, so a block moves 32 KB per 256x256x64 step where a single
// block with a 128 x 256 tile moves 48 KB for half the work: shared-memory traffic per flop drops by a third and
// L2 traffic per flop by half.  The first block of the pair (rank 0) issues tcgen05.mma.cta_group::2 (M=256): the
// hardware reads A and W from both blocks' shared memory and writes each block's 128 rows of the result into that
// block's tensor memory.  Barriers: `full` lives in the first block and counts the bytes of both blocks' copies
// (the second block's TMA signals it across the cluster); `empty` and `acc_full` exist in both and are signalled
// by one tcgen05.commit to both; `acc_empty` lives in the first block and collects the epilogue warps of both.
constexpr int P2_STAGES = 6;
constexpr int P2_HALF_BYTES = 128 * TC_BK * 2;          // 128 rows of A, or of W, for one k-tile
constexpr int P2_STAGE_BYTES = 2 * P2_HALF_BYTES;
constexpr int P2_STAGING_BYTES = 32 * 64;               // an epilogue warp's piece of the result on its way out

__device__ __forceinline__ unsigned cluster_rank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// The address, in the cluster's shared-memory window, of the same variable in the block of the given rank.
__device__ __forceinline__ unsigned in_block_of_rank(const void* p, unsigned rank) {
  unsigned r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// A tile into THIS block's shared memory; its bytes are counted on a barrier that may lie in the pair's other block.
__device__ __forceinline__ void tma_load_2d_pair(void* smem, const CUtensorMap* map, int x, int y, unsigned bar_in_cluster) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(smem)), "l"(map), "r"(x), "r"(y), "r"(bar_in_cluster)
      : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(unsigned tmem_d, unsigned long long da, unsigned long long db, unsigned idesc,
                                               unsigned accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.u32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives, when the products issued so far have finished, on the barrier at this offset in BOTH blocks of the pair.
__device__ __forceinline__ void umma_commit_pair(void* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"((unsigned short)3)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive_in_cluster(unsigned bar_in_cluster) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_in_cluster) : "memory");
}

template <typename TO>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TC_THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                         const __grid_constant__ CUtensorMap map_c, int c_by_tma,
                         const float* __restrict__ bias, TO* __restrict__ C, int ldc, int M, int N, int K, int act,
                         int bn, int* error) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* staging = tiles + P2_STAGES * P2_STAGE_BYTES;   // 2 KB per epilogue warp: 32 rows of 64 bytes
  unsigned long long* full = reinterpret_cast<unsigned long long*>(staging + TC_EPI_WARPS * P2_STAGING_BYTES);
  unsigned long long* empty = full + P2_STAGES;
  unsigned long long* acc_full = empty + P2_STAGES;    // [2]
  unsigned long long* acc_empty = acc_full + 2;         // [2]
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned rank = cluster_rank();
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int m_tiles = (M + 255) / 256, n_tiles = (N + bn - 1) / bn;   // bn: the tile's width, a multiple of 16
  const int num_tiles = m_tiles * n_tiles;
  const int n_kt = (K + TC_BK - 1) / TC_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < P2_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b2 = 0; b2 < 2; ++b2) {
      mbar_init(&acc_full[b2], 1);
      mbar_init(&acc_empty[b2], 2 * TC_EPI_WARPS);   // one arrival per epilogue warp of either block
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {  // one warp of EACH block of the pair takes part in the allocation: all 512 columns in both
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(2 * TC_BN)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();   // the other block's barriers exist before anything here signals them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_base = *tmem_slot;
  pdl_trigger();   // only now that both blocks hold their tensor memory (see the single-block kernel)
  pdl_wait();  // A comes from the kernel before

  if (warp == 0) {
    if (lane == 0) {
      unsigned it = 0;
      for (int tile = pair; tile < num_tiles && !*abort_flag; tile += n_pairs) {
        const int m0 = (tile % m_tiles) * 256 + (int)rank * 128, n0 = (tile / m_tiles) * bn + (int)rank * (bn / 2);
        for (int kt = 0; kt < n_kt; ++kt, ++it) {
          const unsigned s = it % P2_STAGES, round = it / P2_STAGES;
          if (round > 0 && !mbar_wait(&empty[s], (round - 1) & 1)) {
            *abort_flag = 1;
            atomicExch(error, 21);
            break;
          }
          if (*abort_flag) break;
          unsigned char* sa = tiles + s * P2_STAGE_BYTES;
          const unsigned bar = in_block_of_rank(&full[s], 0);
          if (rank == 0) mbar_expect_tx(&full[s], 2 * (P2_HALF_BYTES + (bn / 2) * TC_BK * 2));   // both blocks' copies
          tma_load_2d_pair(sa, &map_a, kt * TC_BK, m0, bar);
          tma_load_2d_pair(sa + P2_HALF_BYTES, &map_w, kt * TC_BK, n0, bar);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      const unsigned idesc = umma_idesc(256, bn);
      unsigned it = 0, local = 0;
      for (int tile = pair; tile < num_tiles && !*abort_flag; tile += n_pairs, ++local) {
        const unsigned buf = local & 1, use = local >> 1;
        if (use > 0 && !mbar_wait(&acc_empty[buf], (use - 1) & 1)) {   // both epilogues have read this accumulator
          *abort_flag = 4;
          atomicExch(error, 24);
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned tmem_d = tmem_base + buf * TC_BN;
        bool ok = true;
        for (int kt = 0; kt < n_kt; ++kt, ++it) {
          const unsigned s = it % P2_STAGES, round = it / P2_STAGES;
          if (!mbar_wait(&full[s], round & 1)) {
            *abort_flag = 2;
            atomicExch(error, 22);
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const unsigned char* sa = tiles + s * P2_STAGE_BYTES;
          const unsigned long long da = umma_desc(sa), db = umma_desc(sa + P2_HALF_BYTES);
#pragma unroll
          for (int k = 0; k < TC_BK / 16; ++k)
            umma_bf16_pair(tmem_d, da + (unsigned long long)(k * 2), db + (unsigned long long)(k * 2), idesc,
                           (kt > 0 || k > 0) ? 1u : 0u);
          umma_commit_pair(&empty[s]);
        }
        if (!ok) break;
        umma_commit_pair(&acc_full[buf]);
      }
    }
  } else {
    // the four warps of a quarter of tensor memory take the tile's pieces of 16 columns in turn
    const int quarter = warp & 3, turn = (warp - 2) >> 2;
    const bool vec_ok = (ldc * sizeof(TO)) % 16 == 0 && ((uintptr_t)C & 15) == 0;
    unsigned local = 0;
    for (int tile = pair; tile < num_tiles; tile += n_pairs, ++local) {
      const int m0 = (tile % m_tiles) * 256 + (int)rank * 128, n0 = (tile / m_tiles) * bn;
      const unsigned buf = local & 1, use = local >> 1;
      const int row = m0 + quarter * 32 + lane;
      if (!mbar_wait(&acc_full[buf], use & 1)) {
        atomicExch(error, 23);
        break;
      }
      if (*abort_flag) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if constexpr (sizeof(TO) == 2) {
        if (c_by_tma) {
          // Pieces of 32 columns: a thread has 64 bytes of ITS row, which as plain stores would be 32 rows of
          // partly written lines per instruction.  The warp puts the piece into shared memory (64-byte swizzle:
          // no bank conflicts) and one TMA store writes it as whole rows; rows past M and columns past N are
          // clipped by the copy.  A width that is no multiple of 32 makes the last piece overlap the one before
          // (the same values twice).
          unsigned char* mine = staging + (warp - 2) * P2_STAGING_BYTES;
          const int n_pieces = (bn + 31) / 32;
          for (int piece = turn; piece < n_pieces; piece += TC_EPI_WARPS / 4) {
            const int c0 = min(piece * 32, bn - 32);
            if (n0 + c0 >= N) break;
            float v[32];
            tmem_ld32(tmem_base + ((unsigned)(quarter * 32) << 16) + buf * TC_BN + (unsigned)c0, v);
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the store before has read `mine`
            __syncwarp();
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              unsigned pk[4];
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int n = n0 + c0 + q * 8 + i * 2;
                const float b0 = (bias && n < N) ? bias[n] : 0.f, b1 = (bias && n + 1 < N) ? bias[n + 1] : 0.f;
                __nv_bfloat162 p = __floats2bfloat162_rn(activate(v[q * 8 + i * 2] + b0, act), activate(v[q * 8 + i * 2 + 1] + b1, act));
                pk[i] = *reinterpret_cast<unsigned*>(&p);
              }
              *reinterpret_cast<uint4*>(mine + lane * 64 + ((q ^ ((lane >> 1) & 3)) * 16)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
              asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                           ::"l"(&map_c), "r"(n0 + c0), "r"(m0 + quarter * 32), "r"(smem_u32(mine))
                           : "memory");
              asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
          }
        }
      }
      if constexpr (sizeof(TO) == 4) {
        if (c_by_tma) {
          // 32-bit results: pieces of 16 columns (the same 64 bytes of a thread's row), staged the same way; one TMA
          // copy stores the piece, or adds it into C (c_by_tma 2: C is the residual stream, C += A W^T + bias).
          // The tile's width is a multiple of 16, so the pieces do not overlap (a sum must not be added twice);
          // rows past M and columns past N are clipped by the copy.
          unsigned char* mine = staging + (warp - 2) * P2_STAGING_BYTES;
          for (int c0 = turn * 16; c0 < bn; c0 += 16 * (TC_EPI_WARPS / 4)) {
            if (n0 + c0 >= N) break;
            float v[16];
            tmem_ld16(tmem_base + ((unsigned)(quarter * 32) << 16) + buf * TC_BN + (unsigned)c0, v);
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the copy before has read `mine`
            __syncwarp();
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              float o[4];
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int n = n0 + c0 + q * 4 + i;
                o[i] = activate(v[q * 4 + i] + ((bias && n < N) ? bias[n] : 0.f), act);
              }
              *reinterpret_cast<float4*>(mine + lane * 64 + ((q ^ ((lane >> 1) & 3)) * 16)) = make_float4(o[0], o[1], o[2], o[3]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
              if (c_by_tma == 2)
                asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2}], [%3];"
                             ::"l"(&map_c), "r"(n0 + c0), "r"(m0 + quarter * 32), "r"(smem_u32(mine))
                             : "memory");
              else
                asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                             ::"l"(&map_c), "r"(n0 + c0), "r"(m0 + quarter * 32), "r"(smem_u32(mine))
                             : "memory");
              asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
          }
        }
      }
      if (!c_by_tma) {
        for (int c0 = turn * 16; c0 < bn; c0 += 16 * (TC_EPI_WARPS / 4)) {
          if (n0 + c0 >= N) break;
          float v[16];
          tmem_ld16(tmem_base + ((unsigned)(quarter * 32) << 16) + buf * TC_BN + (unsigned)c0, v);
          if (row < M)
            store_row32<TO, 16>(C + (size_t)row * ldc + n0 + c0, v, bias, n0 + c0, N, act,
                                vec_ok && ((n0 + c0) * sizeof(TO)) % 16 == 0);
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive_in_cluster(in_block_of_rank(&acc_empty[buf], 0));
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // this warp's stores have been written
  }
  // neither block leaves, nor frees tensor memory, while the other may still read its shared memory, write its
  // tensor memory or signal its barriers
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * TC_BN) : "memory");
  }
}

// ---- host side: tensor maps -------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
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

// A [rows, K] bfloat16 matrix with row pitch ld elements as a 2-D tensor (K innermost), boxes of 64 x box_rows.
static int make_map(CUtensorMap* map, const void* ptr, int rows, int K, int ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return CBIS_ERR_BAD_SIZE;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? CBIS_OK : CBIS_ERR_BAD_SIZE;
}

// CBIS_TCGEN05_PAIR=0 keeps every product on single blocks (128 x 256 tiles).
static int pair_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("CBIS_TCGEN05_PAIR");
    on = (e && e[0] == '0') ? 0 : 1;
  }
  return on;
}

// The bfloat16 result [rows, N] with row pitch ld as a 2-D tensor for stores of 32 x 32 pieces, 64-byte swizzle.
static int make_map_c(CUtensorMap* map, void* ptr, int rows, int N, int ld) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return CBIS_ERR_BAD_SIZE;
  const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {32, 32};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, ptr, dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? CBIS_OK : CBIS_ERR_BAD_SIZE;
}

// The 32-bit result [rows, N] with row pitch ld as a 2-D tensor for copies of 32 rows x 16 columns, 64-byte swizzle.
static int make_map_c_f32(CUtensorMap* map, void* ptr, int rows, int N, int ld) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return CBIS_ERR_BAD_SIZE;
  const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 4};
  const cuuint32_t box[2] = {16, 32};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, ptr, dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? CBIS_OK : CBIS_ERR_BAD_SIZE;
}

}  // namespace cbis

using namespace cbis;

// A [M, lda] and W [N, K] bfloat16 (K contiguous, lda and K multiples of 8, 16-byte aligned), bias [N] float or
// null, C [M, ldc] bfloat16 or float.  error: int on the device, set non-zero if a wait inside the kernel ran out.
// spin_limit (0: the service limit) and starve are for the single-block form (M <= 128) and exist for the test
// of the give-up path: see the kernel.  With starve the result is not computed and *error becomes non-zero.
// accumulate (32-bit C, more than 128 rows, 16-byte aligned rows of C): C += act(A W^T + bias); refused otherwise.
CBIS_EXPORT int cbis_gemm_tcgen05_bf16_ex(const void* A, int lda, const void* W, const float* bias, void* C, int ldc,
                                          int M, int N, int K, int act, int out_dtype, int* error, void* stream,
                                          unsigned spin_limit, int starve, int accumulate);

CBIS_EXPORT int cbis_gemm_tcgen05_bf16(const void* A, int lda, const void* W, const float* bias, void* C, int ldc,
                                       int M, int N, int K, int act, int out_dtype, int* error, void* stream) {
  return cbis_gemm_tcgen05_bf16_ex(A, lda, W, bias, C, ldc, M, N, K, act, out_dtype, error, stream, 0, 0, 0);
}

CBIS_EXPORT int cbis_gemm_tcgen05_bf16_ex(const void* A, int lda, const void* W, const float* bias, void* C, int ldc,
                                          int M, int N, int K, int act, int out_dtype, int* error, void* stream,
                                          unsigned spin_limit, int starve, int accumulate) {
  if (M <= 0 || N <= 0) return CBIS_OK;
  if (accumulate && (out_dtype != CBIS_F32 || M <= TC_BM || starve || !pair_enabled())) return CBIS_ERR_BAD_SIZE;
  if (spin_limit == 0) spin_limit = TC_SPIN_LIMIT;
  if (starve && M > TC_BM) return CBIS_ERR_BAD_SIZE;     // only the single-block form can be starved
  if (K <= 0 || K % 8 || lda % 8 || lda < K || ldc < N) return CBIS_ERR_BAD_SIZE;
  if (((uintptr_t)A & 15) || ((uintptr_t)W & 15) || error == nullptr) return CBIS_ERR_ALIGNMENT;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  CUtensorMap map_a, map_w;
  cudaError_t e;
  if (pair_enabled() && M > TC_BM && !starve) {
    // pairs of blocks on 256 x 256 tiles: every block loads boxes of 128 rows of A and of W
    // the tile's width: the multiple of 16 for which the pairs' rounds over the tiles take the least time (a last
    // round that only a few pairs work in costs as much as a full one)
    const int m_tiles = (M + 255) / 256, max_pairs = sms / 2;
    int bn = TC_BN;
    long long best = -1;
    for (int cand = TC_BN; cand >= 64; cand -= 16) {
      const long long tiles = (long long)m_tiles * ((N + cand - 1) / cand);
      const long long cost = ((tiles + max_pairs - 1) / max_pairs) * (cand + 16);   // + 16: a tile's fixed share
      if (best < 0 || cost < best) best = cost, bn = cand;
    }
    int st = make_map(&map_a, A, M, K, lda, 128);
    if (st != CBIS_OK) return st;
    st = make_map(&map_w, W, N, K, K, bn / 2);
    if (st != CBIS_OK) return st;
    // the result goes out through TMA when it is bfloat16, 16-byte aligned rows and at least one piece wide
    CUtensorMap map_c = map_a;
    int c_by_tma = out_dtype == CBIS_BF16 && ((uintptr_t)C & 15) == 0 && ldc % 8 == 0 && N >= 32 &&
                   make_map_c(&map_c, C, M, N, ldc) == CBIS_OK;
    // ... and when it is 32-bit with 16-byte aligned rows: pieces of 16 columns, stored or added into C
    if (out_dtype == CBIS_F32 && ((uintptr_t)C & 15) == 0 && ldc % 4 == 0 && N >= 16 &&
        make_map_c_f32(&map_c, C, M, N, ldc) == CBIS_OK)
      c_by_tma = accumulate ? 2 : 1;
    if (accumulate && c_by_tma != 2) return CBIS_ERR_ALIGNMENT;
    const size_t smem = (size_t)P2_STAGES * P2_STAGE_BYTES + TC_EPI_WARPS * P2_STAGING_BYTES + 1024 + 256;
    const int num_tiles = ((N + bn - 1) / bn) * m_tiles;
    const int pairs = num_tiles < max_pairs ? num_tiles : max_pairs;
    dim3 grid(2 * pairs);
    if (out_dtype == CBIS_BF16) {
      auto kern = gemm_tcgen05_pair_kernel<__nv_bfloat16>;
      e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
      e = launch_pdl(kern, grid, dim3(TC_THREADS), smem, (cudaStream_t)stream, map_a, map_w, map_c, c_by_tma, bias,
                     (__nv_bfloat16*)C, ldc, M, N, K, act, bn, error);
    } else if (out_dtype == CBIS_F32) {
      auto kern = gemm_tcgen05_pair_kernel<float>;
      e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
      e = launch_pdl(kern, grid, dim3(TC_THREADS), smem, (cudaStream_t)stream, map_a, map_w, map_c, c_by_tma, bias, (float*)C,
                     ldc, M, N, K, act, bn, error);
    } else {
      return CBIS_ERR_BAD_DTYPE;
    }
    return (int)e;
  }
  int st = make_map(&map_a, A, M, K, lda, TC_BM);
  if (st != CBIS_OK) return st;
  st = make_map(&map_w, W, N, K, K, TC_BN);
  if (st != CBIS_OK) return st;
  const size_t smem = (size_t)TC_STAGES * TC_STAGE_BYTES + 1024 + 256;
  const int num_tiles = ((N + TC_BN - 1) / TC_BN) * ((M + TC_BM - 1) / TC_BM);
  dim3 grid(num_tiles < sms ? num_tiles : sms);
  if (out_dtype == CBIS_BF16) {
    auto kern = gemm_tcgen05_kernel<__nv_bfloat16>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    e = launch_pdl(kern, grid, dim3(TC_THREADS), smem, (cudaStream_t)stream, map_a, map_w, bias, (__nv_bfloat16*)C, ldc,
                   M, N, K, act, error, spin_limit, starve);
  } else if (out_dtype == CBIS_F32) {
    auto kern = gemm_tcgen05_kernel<float>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    e = launch_pdl(kern, grid, dim3(TC_THREADS), smem, (cudaStream_t)stream, map_a, map_w, bias, (float*)C, ldc, M, N, K,
                   act, error, spin_limit, starve);
  } else {
    return CBIS_ERR_BAD_DTYPE;
  }
  return (int)e;
}
