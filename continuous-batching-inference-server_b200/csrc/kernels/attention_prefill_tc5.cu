// Prefill attention over the paged cache on the 5th-generation tensor cores (bfloat16, head size 128).
//
// A block takes 128 consecutive rows of one (segment, head).  Keys and values come in tiles of 128
// keys, page by page through the block table, with TMA (cp.async.bulk.tensor, 128-byte swizzle, two
// stages).  One thread issues the products: S = Q K^T (tcgen05.mma, 128x128x16, eight per tile) into
// tensor memory (double-buffered), and P V into another accumulator.  Eight warps share the query rows, two
// threads per row: they read S with tcgen05.ld (half a row per thread: no shuffles for the maximum and sum), scale
// and mask in 32-bit, keep the running maximum and sum, write P in bfloat16 into shared memory in the
// swizzled layout the product reads, and add each tile's P V to the output they keep in registers,
// rescaled in 32-bit.  V is used as it lies in the cache ([key][head dim], head dim contiguous): it is
// the MN-major B operand of P V.
//
// The mma.sync kernel in attention_prefill.cu spends 1,044 instructions per warp and 64 keys with the
// tensor pipe idle three quarters of the time; here the products run asynchronously at the tensor
// cores' own rate and a thread spends about 600 instructions per 128 keys.
//
// Every wait on an mbarrier is bounded; when a limit runs out the block sets *error, stops, frees its
// tensor memory and returns (its output rows are then invalid, and the host raises).
#include "common.cuh"

#include <cuda.h>
#include <math.h>
#include <mutex>

namespace cbis {
namespace tc5 {

constexpr int BM = 128, BN = 128, HD = 128;
constexpr int HALF_BYTES = 128 * 128;          // 128 rows of 128 bytes (64 bf16 of the head dim, or 64 keys of P)
constexpr int TILE_BYTES = 2 * HALF_BYTES;     // a 128 x 128 bf16 tile as two swizzled halves
constexpr int STAGES = 2;
constexpr int THREADS = 320;                   // warp 0: TMA, warp 1: MMA + tensor memory, warps 2..9: softmax
constexpr unsigned SPIN_LIMIT = 1u << 24;

__device__ __forceinline__ unsigned s32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void bar_init(void* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(bar)), "r"(count));
}
__device__ __forceinline__ void bar_expect(void* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bar_arrive(void* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s32(bar)) : "memory");
}
__device__ __forceinline__ bool bar_wait(void* bar, unsigned parity) {
  const unsigned a = s32(bar);
  for (unsigned it = 0; it < SPIN_LIMIT; ++it) {
    unsigned ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(a), "r"(parity) : "memory");
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
// MN-major operand (V as B of P*V: N = head dim contiguous, K = keys): atoms of 8 keys x 64 head dims (1024 bytes);
// the next atom along N (the other half of the head dim) lies `mn_stride` bytes further, the next 8 keys 1024 bytes.
__device__ __forceinline__ unsigned long long desc_mnmajor(const void* smem, unsigned mn_stride, unsigned k_stride) {
  unsigned long long d = 0;
  d |= (unsigned long long)((s32(smem) & 0x3FFFF) >> 4);
  d |= (unsigned long long)((mn_stride >> 4) & 0x3FFF) << 16;
  d |= (unsigned long long)((k_stride >> 4) & 0x3FFF) << 32;
  d |= (unsigned long long)1 << 46;
  d |= (unsigned long long)2 << 61;
  return d;
}
// D = F32, A = B = BF16, M = 128, N = 128; b_mn: B is MN-major.
__host__ __device__ constexpr unsigned idesc(bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn ? 1u : 0u) << 16) | ((unsigned)(BN >> 3) << 17) |
         ((unsigned)(BM >> 4) << 24);
}
__device__ __forceinline__ void mma(unsigned tmem_d, unsigned long long da, unsigned long long db, unsigned id,
                                    unsigned accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.u32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
               ::"r"(tmem_d), "l"(da), "l"(db), "r"(id), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void commit(void* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s32(bar)) : "memory");
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
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// grid: (row tiles of the longest segment, heads, segments from seg0 on)
__global__ void __launch_bounds__(THREADS, 1)
paged_prefill_tc5_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, const int* block_table, int max_blocks,
                         const int* cu_rows, const int* seg_start, __nv_bfloat16* out, int out_ld, int seg0, int n_head,
                         int n_kv_head, int ps, float scale_log2e, int window, int* error) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* sQ = base;                                   // 2 halves
  unsigned char* sK = sQ + TILE_BYTES;                        // STAGES tiles
  unsigned char* sV = sK + STAGES * TILE_BYTES;               // STAGES tiles
  unsigned char* sP = sV + STAGES * TILE_BYTES;               // 2 halves (keys 0..63, 64..127)
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(sP + TILE_BYTES);
  unsigned long long *q_full = bars, *kv_full = bars + 1, *kv_empty = bars + 3, *s_full = bars + 5, *p_ready = bars + 7,
                     *pv_full = bars + 8, *pair_bar = bars + 10;   // pair_bar: one per quarter of the rows
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 9);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // late row tiles have the most keys to walk: they are given out first
  const int seg = seg0 + blockIdx.z, h = blockIdx.y, tile = gridDim.x - 1 - blockIdx.x;
  pdl_trigger();
  const int r_begin = cu_rows[seg], n_rows = cu_rows[seg + 1] - r_begin;
  if (tile * BM >= n_rows) return;
  const int hk = h / (n_head / n_kv_head);
  const int pos0 = seg_start[seg] + tile * BM;
  const int rows_here = min(BM, n_rows - tile * BM);
  const int kend = pos0 + rows_here;
  const int kbegin = window > 0 ? max(0, pos0 - window + 1) : 0;
  const int live_from = (kbegin / ps) * ps;
  const int kt_first = kbegin / BN, kt_last = (kend - 1) / BN, n_tiles = kt_last - kt_first + 1;
  const int* bt = block_table + (size_t)seg * max_blocks;

  // keys and values of rows that no copy will fill must be finite: P is zero there, and 0 * NaN is NaN
  for (int i = threadIdx.x; i < 2 * STAGES * TILE_BYTES / 16; i += THREADS)
    reinterpret_cast<uint4*>(sK)[i] = make_uint4(0, 0, 0, 0);
  if (threadIdx.x == 0) {
    bar_init(q_full, 1);
    for (int s = 0; s < STAGES; ++s) {
      bar_init(&kv_full[s], 1);
      bar_init(&kv_empty[s], 1);
    }
    bar_init(&s_full[0], 1);
    bar_init(&s_full[1], 1);
    bar_init(p_ready, 8);
    bar_init(pv_full, 1);
    for (int q = 0; q < 4; ++q) bar_init(&pair_bar[q], 2);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp == 1) {  // three accumulators of 128 columns (S twice, P V) in an allocation of 512
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_s = *tmem_slot, tmem_pv = tmem_s + 256;
  pdl_wait();  // q and this step's keys/values come from the kernels before

  if (warp == 0) {
    // The whole warp produces: lane i looks up page i of the tile in the block table (one coalesced load instead of
    // a chain of dependent ones) and issues the four copies of that page; lane 0 posts the expected bytes first.
    if (lane == 0) {
      bar_expect(q_full, TILE_BYTES);
      const int qrow = r_begin + tile * BM;
      tma_2d(sQ, &map_q, h * HD, qrow, q_full);
      tma_2d(sQ + HALF_BYTES, &map_q, h * HD + 64, qrow, q_full);
    }
    const int pages_per_tile = BN / ps;
    for (int j = 0; j < n_tiles; ++j) {
      const int s = j % STAGES, kt = kt_first + j;
      int stop = 0;
      if (lane == 0) {
        if (j >= STAGES && !bar_wait(&kv_empty[s], ((j / STAGES) - 1) & 1)) {
          *abort_flag = 1;
          atomicExch(error, 11);
        }
        stop = *abort_flag;
        if (!stop) {
          int n_valid = 0;
          for (int p0 = 0; p0 < BN; p0 += ps) {
            const int j0 = kt * BN + p0;
            if (j0 < kend && j0 + ps > live_from) ++n_valid;
          }
          bar_expect(&kv_full[s], (unsigned)n_valid * ps * 128u * 2u * 2u);
        }
      }
      stop = __shfl_sync(0xffffffffu, stop, 0);
      if (stop) break;
      if (lane < pages_per_tile) {
        const int p0 = lane * ps, j0 = kt * BN + p0;
        if (j0 < kend && j0 + ps > live_from) {
          const int page = bt[j0 / ps];
          const int grow = (page * n_kv_head + hk) * ps;       // row of the page's first key in the [rows, HD] view
          unsigned char* dk = sK + s * TILE_BYTES + p0 * 128;
          unsigned char* dv = sV + s * TILE_BYTES + p0 * 128;
          tma_2d(dk, &map_k, 0, grow, &kv_full[s]);
          tma_2d(dk + HALF_BYTES, &map_k, 64, grow, &kv_full[s]);
          tma_2d(dv, &map_v, 0, grow, &kv_full[s]);
          tma_2d(dv + HALF_BYTES, &map_v, 64, grow, &kv_full[s]);
        }
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // S is double-buffered in tensor memory: Q K^T of tile j+1 is issued before the softmax of tile j is awaited,
      // so the tensor cores work while the softmax warps do.
      bool ok = bar_wait(q_full, 0);
      if (!ok) { *abort_flag = 2; atomicExch(error, 12); }
      auto issue_qk = [&](int j) -> bool {
        const int s = j % STAGES;
        if (!bar_wait(&kv_full[s], (j / STAGES) & 1)) { *abort_flag = 3; atomicExch(error, 13); return false; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {   // eight steps of 16 along the head dim, four in each 64-wide half
          const int off = (kk / 4) * HALF_BYTES + (kk % 4) * 32;
          mma(tmem_s + (j & 1) * 128, desc_kmajor(sQ + off), desc_kmajor(sK + s * TILE_BYTES + off), idesc(false),
              kk > 0 ? 1u : 0u);
        }
        commit(&s_full[j & 1]);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; j < n_tiles && ok && !*abort_flag; ++j) {
        const int s = j % STAGES;
        // the next tile's scores: its S buffer was read by the softmax of tile j-1, which p_ready(j-1) has told
        if (j + 1 < n_tiles) {
          ok = issue_qk(j + 1);
          if (!ok) break;
        }
        if (!bar_wait(p_ready, j & 1)) { *abort_flag = 4; atomicExch(error, 14); break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // P V: eight steps of 16 keys; V is MN-major: 16 keys are two 1024-byte atoms, the other half of the head dim 16 KB on
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          const int poff = (kk / 4) * HALF_BYTES + (kk % 4) * 32;
          mma(tmem_pv, desc_kmajor(sP + poff), desc_mnmajor(sV + s * TILE_BYTES + kk * 2048, HALF_BYTES, 1024),
              idesc(true), kk > 0 ? 1u : 0u);
        }
        commit(&kv_empty[s]);   // this stage's keys and values are free again when the products have read them
        commit(pv_full);
      }
    }
  } else {
    // Eight softmax warps: a warp reads the quarter of tensor memory given by its index % 4, so two warps share a
    // quarter: two threads per query row.  Thread `half` takes keys [64*half, 64*half+64) of every tile for the
    // scores and head dims [64*half, 64*half+64) of the output; the two exchange the row maximum through shared
    // memory (an mbarrier per quarter, waited on with a limit like every other) and add their parts of the row
    // sum at the end.
    __shared__ float xmax[2][BM];
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;              // this thread's query row within the tile
    const int p = pos0 + r;                         // its position
    const unsigned lane_addr = (unsigned)(quarter * 32) << 16;
    float o[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) o[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int j0 = (kt_first + j) * BN;
      if (!bar_wait(&s_full[j & 1], (j >> 1) & 1)) { atomicExch(error, 15); ok = false; break; }
      if (*abort_flag) { ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const unsigned s_addr = tmem_s + (j & 1) * 128 + lane_addr + half * 64;
      const bool edge = (j0 + BN - 1 > pos0) || (window > 0 && j0 < pos0 + BM - window + 1) || j0 + BN > kend;
      // keys this row may see in this tile: [lo, hi), as columns of the tile; this thread's columns start at c_base
      const int hi = min(min(p + 1, kend) - j0, BN);
      const int lo = window > 0 ? max(p - window + 1 - j0, 0) : 0;
      const int c_base = half * 64;
      // pass 1: the maximum of this thread's 64 raw scores (the scale is positive), then of the row
      float mx = -INFINITY;
#pragma unroll 1
      for (int c0 = 0; c0 < 64; c0 += 32) {
        float v[32];
        tmem_ld32(s_addr + c0, v);
        if (!edge) {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx = fmaxf(mx, v[i]);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c_base + c0 + i >= lo && c_base + c0 + i < hi) mx = fmaxf(mx, v[i]);
        }
      }
      xmax[half][r] = mx;
      __syncwarp();
      if (lane == 0) bar_arrive(&pair_bar[quarter]);
      if (!bar_wait(&pair_bar[quarter], j & 1)) { atomicExch(error, 17); ok = false; break; }
      mx = fmaxf(mx, xmax[half ^ 1][r]) * scale_log2e;
      const float m_new = fmaxf(m, mx);
      const float ref = m_new == -INFINITY ? 0.f : m_new;   // a row with no key in range yet
      const float corr = exp2f(m - ref);
      // pass 2: P = exp2(S * scale - max) in bfloat16 into shared memory (swizzled rows of 64 keys), and its sum
      float psum = 0.f;
#pragma unroll 1
      for (int c0 = 0; c0 < 64; c0 += 32) {
        float v[32];
        tmem_ld32(s_addr + c0, v);
        unsigned pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float e0 = exp2f(fmaf(v[i], scale_log2e, -ref)), e1 = exp2f(fmaf(v[i + 1], scale_log2e, -ref));
          if (edge) {
            if (c_base + c0 + i < lo || c_base + c0 + i >= hi) e0 = 0.f;
            if (c_base + c0 + i + 1 < lo || c_base + c0 + i + 1 >= hi) e1 = 0.f;
          }
          psum += e0 + e1;
          __nv_bfloat162 b = __floats2bfloat162_rn(e0, e1);
          pk[i >> 1] = *reinterpret_cast<unsigned*>(&b);
        }
        unsigned char* prow = sP + half * HALF_BYTES + r * 128;   // this thread's 64 keys are one swizzled row
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int chunk = (c0 / 8 + q4) ^ (r & 7);            // 16-byte piece within the 128-byte row, swizzled
          *reinterpret_cast<uint4*>(prow + chunk * 16) = make_uint4(pk[q4 * 4], pk[q4 * 4 + 1], pk[q4 * 4 + 2], pk[q4 * 4 + 3]);
        }
      }
      l = l * corr + psum;
      m = m_new;
      if (j0 + BN > kend && half == 0 && j0 + r >= kend) {
        // the last tile: values of keys past the end are whatever the page held; P is zero there, but zero
        // times a NaN left by an earlier owner of the page would still be NaN: this thread clears key row r
        unsigned char* vrow = sV + (j % STAGES) * TILE_BYTES + r * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          *reinterpret_cast<uint4*>(vrow + c * 16) = make_uint4(0, 0, 0, 0);
          *reinterpret_cast<uint4*>(vrow + HALF_BYTES + c * 16) = make_uint4(0, 0, 0, 0);
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P must be visible to the tensor cores' reads
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) bar_arrive(p_ready);
      if (!bar_wait(pv_full, j & 1)) { atomicExch(error, 16); ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
      for (int c0 = 0; c0 < 64; c0 += 32) {
        float v[32];
        tmem_ld32(tmem_pv + lane_addr + half * 64 + c0, v);
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c0 + i] = fmaf(o[c0 + i], corr, v[i]);
      }
    }
    // the two threads of a row add their parts of the row sum
    if (ok) {
      xmax[half][r] = l;
      __syncwarp();
      if (lane == 0) bar_arrive(&pair_bar[quarter]);
      if (!bar_wait(&pair_bar[quarter], n_tiles & 1)) { atomicExch(error, 17); ok = false; }
    }
    if (ok && r < rows_here) {
      const float inv = 1.f / (l + xmax[half ^ 1][r]);
      __nv_bfloat16* dst = out + (size_t)(r_begin + tile * BM + r) * out_ld + h * HD + half * 64;
#pragma unroll
      for (int i = 0; i < 64; i += 8) {
        uint4 q4;
        __nv_bfloat162 a = __floats2bfloat162_rn(o[i] * inv, o[i + 1] * inv), b = __floats2bfloat162_rn(o[i + 2] * inv, o[i + 3] * inv);
        __nv_bfloat162 c = __floats2bfloat162_rn(o[i + 4] * inv, o[i + 5] * inv), d = __floats2bfloat162_rn(o[i + 6] * inv, o[i + 7] * inv);
        q4.x = *reinterpret_cast<unsigned*>(&a);
        q4.y = *reinterpret_cast<unsigned*>(&b);
        q4.z = *reinterpret_cast<unsigned*>(&c);
        q4.w = *reinterpret_cast<unsigned*>(&d);
        *reinterpret_cast<uint4*>(dst + i) = q4;
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_s), "r"(512) : "memory");
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
// [rows, cols] bfloat16 with row pitch ld elements; boxes of 64 columns x box_rows rows, 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* ptr, long long rows, int cols, long long ld, int box_rows) {
  EncodeTiledFn fn = encoder();
  if (!fn) return CBIS_ERR_BAD_SIZE;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? CBIS_OK : CBIS_ERR_BAD_SIZE;
}

}  // namespace tc5
}  // namespace cbis

using namespace cbis;

// q: [total_rows, q_ld] bfloat16 with head h in columns h*128..; kc/vc: [num_pages, n_kv_head, ps, 128].
// Takes head size 128 and page sizes 8, 16, 32, 64, 128; refuses anything else.
CBIS_EXPORT int cbis_paged_prefill_tc5(const void* q, int q_ld, int total_rows, const void* kc, const void* vc,
                                       int num_pages, const int* block_table, int max_blocks, const int* cu_rows,
                                       const int* seg_start, void* out, int out_ld, int seg0, int n_seg,
                                       int max_seg_rows, int n_head, int n_kv_head, int hd, int ps, float scale,
                                       int window, int* error, void* stream) {
  if (n_seg <= 0 || max_seg_rows <= 0) return CBIS_OK;
  if (hd != 128 || ps < 8 || ps > 128 || (ps & (ps - 1)) || n_head <= 0 || n_kv_head <= 0 || n_head % n_kv_head)
    return CBIS_ERR_BAD_SIZE;
  if (q_ld % 8 || out_ld % 8 || ((uintptr_t)q & 15) || ((uintptr_t)kc & 15) || ((uintptr_t)vc & 15) ||
      ((uintptr_t)out & 15) || error == nullptr)
    return CBIS_ERR_ALIGNMENT;
  CUtensorMap map_q, map_k, map_v;
  int st = tc5::make_map(&map_q, q, total_rows, n_head * hd, q_ld, tc5::BM);
  if (st != CBIS_OK) return st;
  const long long cache_rows = (long long)num_pages * n_kv_head * ps;
  st = tc5::make_map(&map_k, kc, cache_rows, hd, hd, ps);
  if (st != CBIS_OK) return st;
  st = tc5::make_map(&map_v, vc, cache_rows, hd, hd, ps);
  if (st != CBIS_OK) return st;
  const size_t smem = (size_t)(2 + 2 * tc5::STAGES) * tc5::TILE_BYTES + 1024 + 256;
  auto kern = tc5::paged_prefill_tc5_kernel;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  dim3 grid((max_seg_rows + tc5::BM - 1) / tc5::BM, n_head, n_seg);
  e = launch_pdl(kern, grid, dim3(tc5::THREADS), smem, (cudaStream_t)stream, map_q, map_k, map_v, block_table, max_blocks,
                 cu_rows, seg_start, (__nv_bfloat16*)out, out_ld, seg0, n_head, n_kv_head, ps,
                 scale * 1.4426950408889634f, window, error);
  return (int)e;
}
