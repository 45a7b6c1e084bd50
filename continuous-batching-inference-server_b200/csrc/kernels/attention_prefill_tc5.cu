// Prefill attention over the paged cache on the 5th-generation tensor cores (bfloat16, head size 64 or 128; the
// numbers below are for 128).
//
// A block takes 128 consecutive rows of one (segment, head).  Keys and values come in tiles of 64 keys,
// page by page through the block table, with TMA (cp.async.bulk.tensor, 128-byte swizzle): one warp brings
// the keys and another the values, each with two stages and barriers of its own, because a stage of keys
// is free long before the stage of values of the same tile is, and because a thread issues a TMA copy
// in about 60 ns: the sixteen copies of a tile of 16-key pages would take one warp the tile's whole time.
// (Gathering them with 16-byte cp.async copies from one warp was tried and is slower: a warp cannot keep
// enough of those in flight.)
// One thread issues the products: S = Q K^T (tcgen05.mma, 128x64x16, eight per tile) into tensor memory
// (two buffers, so the scores of the next two tiles are computed while the softmax of this one runs), and
// O += P V (128x128x16, four per tile) into an accumulator that STAYS in tensor memory for the whole row
// tile.  Four warps own one query row per thread: a thread reads its row's 64 scores with tcgen05.ld,
// masks and takes the maximum in 32-bit (no shuffles, no exchange), computes P = exp2(S * scale - m) in
// 32-bit, writes it in bfloat16 into shared memory in the swizzled layout the product reads, and keeps
// the running sum.  The reference value m only has to be common to a row's numbers, not to be their
// exact maximum: it is raised, and O in tensor memory and the sum rescaled (in 32-bit), only when a
// tile's maximum exceeds it by more than 2^8, which after the first tiles is rare; the quotient
// O / sum at the end is the same.  (Two threads per row, each with half the scores, were slower: the
// exchange of the two maxima costs more than the shorter loops save.)  V is used as it lies in the cache ([key][head dim],
// head dim contiguous): it is the MN-major B operand of P V.
//
// Shared memory (113 KB) and tensor memory (256 of 512 columns) are sized for TWO blocks per SM: while
// one block's softmax warps work, the other's products run.
//
// Every wait on an mbarrier is bounded; when a limit runs out the block sets *error, stops, frees its
// tensor memory and returns (its output rows are then invalid, and the host raises).
#include "attention_merge.cuh"

#include <cuda.h>
#include <math.h>
#include <mutex>

namespace cbis {
namespace tc5 {

constexpr int BM = 128, BN = 64;
constexpr int Q_HALF_BYTES = BM * 128;         // 128 rows of 128 bytes: 64 head dims
constexpr int KV_HALF_BYTES = BN * 128;        // 64 keys of 128 bytes: 64 head dims
constexpr int P_BYTES = BM * 128;              // 128 rows of 64 keys
constexpr int STAGES = 2;
// Q, keys (one stage), values (STAGES), P (two buffers), barriers; HD: the head size, 64 or 128
constexpr int smem_bytes(int HD) { return (HD / 64) * (Q_HALF_BYTES + (1 + STAGES) * KV_HALF_BYTES) + 2 * P_BYTES + 128; }
constexpr float RAISE_BY = 8.f;                // the reference is raised when a tile's maximum exceeds it by 2^8
constexpr int THREADS = 224;                   // warp 0: Q and keys, warp 1: MMA + tensor memory, warps 2..5: softmax, warp 6: values
constexpr unsigned SPIN_LIMIT = 1u << 21;      // tries of up to 1 us each

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
    // with a time hint the thread sleeps in hardware until the phase completes (or 1 us passes) instead of polling:
    // the many waiting warps of a block leave the issue slots to the few that work
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
// D = F32, A = B = BF16, M = 128, N = n; b_mn: B is MN-major.
__host__ __device__ constexpr unsigned idesc(bool b_mn, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn ? 1u : 0u) << 16) | ((unsigned)(n >> 3) << 17) |
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
// Two loads of 32 columns in flight together, then one wait.
__device__ __forceinline__ void tmem_ld64(unsigned taddr, float* v) {
  unsigned r[64];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,"
      "%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%64];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]),
        "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]),
        "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]),
        "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]),
        "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st32(unsigned taddr, const float* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
        "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
        "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
        "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
        "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
        "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
        "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// grid: row tiles of the longest segment x heads x segments from seg0 on, in one dimension, times two: the two
// blocks of a cluster share a row tile, the first takes the first half of its key tiles and the second the rest,
// and at the end the second hands its sum, reference and output to the first through distributed shared memory.
// The row tile with the most keys decides how long the kernel runs, and its chain of tiles is halved this way.
template <int HD>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 2)
paged_prefill_tc5_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, const int* block_table, int max_blocks,
                         const int* cu_rows, const int* seg_start, __nv_bfloat16* out, int out_ld, int seg0, int n_seg,
                         int n_head, int n_kv_head, int ps, float scale_log2e, int window, int n_chunks, int chunk_keys,
                         float* partial, int row0, int* error) {
  constexpr int HALVES = HD / 64, Q_BYTES = HALVES * Q_HALF_BYTES, KV_BYTES = HALVES * KV_HALF_BYTES;
  extern __shared__ __align__(1024) unsigned char base[];   // no byte to spare for rounding the address up: checked below
  unsigned char* sQ = base;                                   // 2 halves of the head dim
  unsigned char* sK = sQ + Q_BYTES;                           // one tile: Q K^T runs two tiles ahead, so the next keys have time
  unsigned char* sV = sK + KV_BYTES;                          // STAGES tiles
  unsigned char* sP = sV + STAGES * KV_BYTES;                 // two buffers of 128 rows of 64 keys: P V of a tile runs beside the next softmax
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(sP + 2 * P_BYTES);
  // keys and values have barriers of their own: a stage of keys is free as soon as Q K^T has read it, long before
  // the values of the same tile are, so the keys of tile j+2 are on their way while tile j is still being worked on
  unsigned long long *q_full = bars, *k_full = bars + 1, *k_empty = bars + 3, *v_full = bars + 5, *v_empty = bars + 7,
                     *s_full = bars + 9, *p_ready = bars + 11, *pv_done = bars + 13;   // k_full/k_empty: [0] only; p_ready, pv_done: [2], tiles in turn
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // late row tiles have the most keys to walk: blocks are numbered so that those of ALL heads and segments come
  // first, and an SM's second block is a light one
  unsigned rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  const int chunk = ((int)blockIdx.x >> 1) % n_chunks, pair = ((int)blockIdx.x >> 1) / n_chunks;
  const int per_rank = n_head * n_seg, n_row_tiles = (int)(gridDim.x >> 1) / n_chunks / per_rank;
  const int tile = n_row_tiles - 1 - pair / per_rank, seg = seg0 + (pair % per_rank) / n_head, h = pair % n_head;
  const int r_begin = cu_rows[seg], n_rows = cu_rows[seg + 1] - r_begin;
  if (tile * BM >= n_rows) return;
  if (s32(base) & 1023) {   // the swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0) atomicExch(error, 18);
    return;
  }
  const int hk = h / (n_head / n_kv_head);
  const int pos0 = seg_start[seg] + tile * BM;
  const int rows_here = min(BM, n_rows - tile * BM);
  int kend = pos0 + rows_here;
  int kbegin = window > 0 ? max(0, pos0 - window + 1) : 0;
  if (n_chunks > 1) {   // few rows behind a long context: this cluster takes one chunk of the keys (whole key tiles,
                        // by absolute index) and leaves an unnormalised partial result for the merge kernel
    kbegin = max(kbegin, chunk * chunk_keys);
    kend = min(kend, (chunk + 1) * chunk_keys);
    if (kbegin >= kend) return;   // both blocks of the cluster alike, before any barrier or allocation
  }
  const int kt_all = kbegin / BN, n_all = (kend - 1) / BN - kt_all + 1, n_first = (n_all + 1) / 2;
  // this block's key tiles: the first takes n_first of them, the second the rest (none, if there is only one)
  const int kt_first = kt_all + (rank ? n_first : 0), n_tiles = rank ? n_all - n_first : n_first;
  const int* bt = block_table + (size_t)seg * max_blocks;

  // keys and values of rows that no copy will fill must be finite: P is zero there, and 0 * NaN is NaN
  for (int i = threadIdx.x; i < (1 + STAGES) * KV_BYTES / 16; i += THREADS)
    reinterpret_cast<uint4*>(sK)[i] = make_uint4(0, 0, 0, 0);

  if (threadIdx.x == 0) {
    bar_init(q_full, 1);
    for (int s = 0; s < STAGES; ++s) {
      bar_init(&k_full[s], 1);
      bar_init(&k_empty[s], 1);
      bar_init(&v_full[s], 1);
      bar_init(&v_empty[s], 1);
    }
    bar_init(&s_full[0], 1);
    bar_init(&s_full[1], 1);
    bar_init(&p_ready[0], 4);
    bar_init(&p_ready[1], 4);
    bar_init(&pv_done[0], 1);
    bar_init(&pv_done[1], 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp == 1) {  // half of tensor memory: S twice (64 columns each) and O (128 columns)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(tmem_slot)), "r"(256) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_s = *tmem_slot, tmem_o = tmem_s + 128;
  // The kernel after this one may start only now that this block holds its tensor memory: a block of a later
  // kernel that allocated first and then waited for this kernel to finish would wait for ever.
  pdl_trigger();
  pdl_wait();  // q and this step's keys/values come from the kernels before

  // softmax state of this thread's query row (warps 2..5; declared here because the hand-over after the loops needs it)
  const int quarter = warp & 3;
  const int r = quarter * 32 + lane;              // this thread's query row within the tile
  const unsigned lane_addr = (unsigned)(quarter * 32) << 16;
  float m = -INFINITY, l = 0.f;                   // the row's reference (log2 units) and the sum of its P
  bool ok = true;
  if (warp == 0 || warp == 6) {
    // Warp 0 brings Q and the keys, warp 6 the values, each as far ahead as its two stages allow (one thread issues
    // a TMA copy in about 60 ns, and a tile of 16-key pages is eight copies of keys and eight of values).
    // The whole warp produces: lane i looks up run i of the tile (a page, or 64 keys of a larger page) in the block
    // table and issues its two copies; lane 0 posts the expected bytes first.
    if (warp == 0 && lane == 0) {
      bar_expect(q_full, Q_BYTES);
      const int qrow = r_begin + tile * BM;
#pragma unroll
      for (int hh = 0; hh < HALVES; ++hh) tma_2d(sQ + hh * Q_HALF_BYTES, &map_q, h * HD + hh * 64, qrow, q_full);
    }
    const int piece = min(ps, BN), pieces_per_tile = BN / piece, piece_shift = 31 - __clz(piece);
    // copies tile j's keys (kv = 0) or values (kv = 1) into their stage; false when the block has given up
    auto load = [&](int j, int kv, int page) -> bool {
      const int s = kv ? j % STAGES : 0, kt = kt_first + j;   // the keys have one stage
      // runs of the tile with a key in [kbegin, kend): from the one holding the first such key to the one holding the last
      const int n_valid = ((min(kend, (kt + 1) * BN) - 1) >> piece_shift) - (max(kbegin, kt * BN) >> piece_shift) + 1;
      const int p0 = lane * piece, j0 = kt * BN + p0;
      // runs wholly before the window may lie in pages already given back: they are not read
      const bool mine = lane < pieces_per_tile && j0 < kend && j0 + piece > kbegin;
      unsigned long long* full = kv ? &v_full[s] : &k_full[s];
      int stop = 0;
      if (lane == 0) {
        if (kv ? (j >= STAGES && !bar_wait(&v_empty[s], ((j / STAGES) - 1) & 1)) : (j >= 1 && !bar_wait(&k_empty[0], (j - 1) & 1))) {
          *abort_flag = 1;
          atomicExch(error, 11);
        }
        stop = *abort_flag;
        if (!stop) bar_expect(full, (unsigned)n_valid * piece * 128u * HALVES);
      }
      stop = __shfl_sync(0xffffffffu, stop, 0);
      if (stop) return false;
      if (mine) {
        const int grow = (page * n_kv_head + hk) * ps + j0 % ps;   // row of the run's first key in the [rows, HD] view
        unsigned char* d = (kv ? sV : sK) + s * KV_BYTES + p0 * 128;
#pragma unroll
        for (int hh = 0; hh < HALVES; ++hh) tma_2d(d + hh * KV_HALF_BYTES, kv ? &map_v : &map_k, hh * 64, grow, full);
      }
      __syncwarp();
      return true;
    };
    // The page of this lane's run is looked up a tile before it is used: the block table is in global memory, and
    // a lookup inside load() would put its latency between every two tiles.
    auto page_of = [&](int j) -> int {
      const int j0 = (kt_first + j) * BN + lane * piece;
      return (j < n_tiles && lane < pieces_per_tile && j0 < kend && j0 + piece > kbegin) ? __ldg(bt + j0 / ps) : 0;
    };
    const int kv = warp == 0 ? 0 : 1;
    int page_now = page_of(0);
    for (int t = 0; t < n_tiles; ++t) {
      const int page_next = page_of(t + 1);
      if (!load(t, kv, page_now)) break;
      page_now = page_next;
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // The descriptors are built once: the one thread that issues the products has nothing to overlap their
      // arithmetic with.  An operand further on in shared memory is the same descriptor plus its offset in 16-byte
      // units (the address field holds shared-memory addresses with room to spare).
      const unsigned long long dq = desc_kmajor(sQ), dk = desc_kmajor(sK), dp = desc_kmajor(sP),
                               dv = desc_mnmajor(sV, KV_HALF_BYTES, 1024);
      bool ok = bar_wait(q_full, 0);
      if (!ok) { *abort_flag = 2; atomicExch(error, 12); }
      auto issue_qk = [&](int j) -> bool {
        if (!bar_wait(&k_full[0], j & 1)) { *abort_flag = 3; atomicExch(error, 13); return false; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {   // eight steps of 16 along the head dim, four in each 64-wide half
          mma(tmem_s + (j & 1) * BN, dq + (unsigned)(((kk / 4) * Q_HALF_BYTES + (kk % 4) * 32) >> 4),
              dk + (unsigned)(((kk / 4) * KV_HALF_BYTES + (kk % 4) * 32) >> 4), idesc(false, BN), kk > 0 ? 1u : 0u);
        }
        commit(&k_empty[0]);   // the keys' stage is free again when these products have read it
        commit(&s_full[j & 1]);
        return true;
      };
      // Q K^T runs two tiles ahead (S has two buffers), so P V of a tile is issued the moment its P is there
      if (ok && n_tiles > 0) ok = issue_qk(0);
      if (ok && n_tiles > 1) ok = issue_qk(1);
      for (int j = 0; j < n_tiles && ok && !*abort_flag; ++j) {
        const int s = j % STAGES;
        // Two barriers, tiles in turn: with one, the softmax can finish tile j+1 (its scores are there two tiles ahead)
        // before this thread has looked at tile j's phase, and a wait by parity then mistakes tile j+2's phase for it
        if (!bar_wait(&p_ready[j & 1], (j >> 1) & 1)) { *abort_flag = 4; atomicExch(error, 14); break; }
        if (!bar_wait(&v_full[s], (j / STAGES) & 1)) { *abort_flag = 3; atomicExch(error, 13); break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // O += P V: four steps of 16 keys; V is MN-major: 16 keys are two 1024-byte atoms, the other half of the
        // head dim KV_HALF_BYTES on
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          mma(tmem_o, dp + (unsigned)(((j & 1) * P_BYTES + kk * 32) >> 4), dv + (unsigned)((s * KV_BYTES + kk * 2048) >> 4), idesc(true, HD),
              (j > 0 || kk > 0) ? 1u : 0u);
        }
        commit(&v_empty[s]);   // the values' stage is free again when these products have read it
        commit(&pv_done[j & 1]);
        // the scores of tile j+2 go where those of tile j were: the softmax has read them (it said so with p_ready)
        if (j + 2 < n_tiles) ok = issue_qk(j + 2);
      }
    }
  } else {
    // Four softmax warps, one thread per query row: a warp reads the quarter of tensor memory given by its index % 4.
    // With the output in tensor memory a thread's share of a tile is one load of 64 scores, their maximum, 64
    // exponentials and eight 16-byte stores of P: no exchange between threads anywhere.
    const int p = pos0 + r;                         // this row's position
    for (int j = 0; j < n_tiles; ++j) {
      const int j0 = (kt_first + j) * BN;
      if (!bar_wait(&s_full[j & 1], (j >> 1) & 1)) { atomicExch(error, 15); ok = false; break; }
      if (*abort_flag) { ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      float v[BN];
      tmem_ld64(tmem_s + (j & 1) * BN + lane_addr, v);
      const bool edge = (j0 + BN - 1 > pos0) || (window > 0 && j0 < pos0 + BM - window + 1) || j0 + BN > kend;
      if (edge) {
        // keys this row may see in this tile: [lo, hi), as columns of the tile
        const int hi = min(min(p + 1, kend) - j0, BN);
        const int lo = window > 0 ? max(p - window + 1 - j0, 0) : 0;
#pragma unroll
        for (int i = 0; i < BN; ++i)
          if (i < lo || i >= hi) v[i] = -INFINITY;
      }
      // four independent chains: a single one would be 64 dependent instructions
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int i = 0; i < BN; i += 4) {
        mx0 = fmaxf(mx0, v[i]);
        mx1 = fmaxf(mx1, v[i + 1]);
        mx2 = fmaxf(mx2, v[i + 2]);
        mx3 = fmaxf(mx3, v[i + 3]);
      }
      const float m_tile = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * scale_log2e;
      // this tile's buffer of P was read by the products of the tile before the last
      if (j > 1 && !bar_wait(&pv_done[j & 1], ((j - 2) >> 1) & 1)) { atomicExch(error, 16); ok = false; break; }
      const bool raise = m_tile > m + RAISE_BY || (m == -INFINITY && m_tile > m);
      if (j > 0 && __any_sync(0xffffffffu, raise)) {
        // rescale the row of O in tensor memory; rows that keep their reference multiply by 1.  Only here does the
        // softmax wait for the products of the tile before, which write O.
        if (!bar_wait(&pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1)) { atomicExch(error, 16); ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const float f = raise ? exp2f(m - m_tile) : 1.f;
#pragma unroll 1
        for (int c0 = 0; c0 < HD; c0 += 32) {
          float o[32];
          tmem_ld32(tmem_o + lane_addr + c0, o);
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] *= f;
          tmem_st32(tmem_o + lane_addr + c0, o);
        }
        l *= f;
      }
      if (raise) m = m_tile;
      const float ref = m == -INFINITY ? 0.f : m;   // a row with no key in range yet: every P is exp2(-inf) = 0
      // P = exp2(S * scale - m) in bfloat16 into shared memory (rows of 64 keys, 128-byte swizzle), and its sum
      float psum = 0.f, psum1 = 0.f;
      unsigned char* prow = sP + (j & 1) * P_BYTES + r * 128;
#pragma unroll
      for (int q8 = 0; q8 < 8; ++q8) {
        unsigned pk[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float e0 = exp2f(fmaf(v[q8 * 8 + 2 * i], scale_log2e, -ref)), e1 = exp2f(fmaf(v[q8 * 8 + 2 * i + 1], scale_log2e, -ref));
          psum += e0;
          psum1 += e1;
          __nv_bfloat162 b2 = __floats2bfloat162_rn(e0, e1);
          pk[i] = *reinterpret_cast<unsigned*>(&b2);
        }
        *reinterpret_cast<uint4*>(prow + ((q8 ^ (r & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);   // swizzled
      }
      l += psum + psum1;
      if (j0 + BN > kend && r < BN && j0 + r >= kend) {
        // the last tile: values of keys past the end are whatever the page held; P is zero there, but zero
        // times a NaN left by an earlier owner of the page would still be NaN: this thread clears key row r
        if (!bar_wait(&v_full[j % STAGES], (j / STAGES) & 1)) { atomicExch(error, 13); ok = false; break; }   // they have landed
        unsigned char* vrow = sV + (j % STAGES) * KV_BYTES + r * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          *reinterpret_cast<uint4*>(vrow + c * 16) = make_uint4(0, 0, 0, 0);
          if (HALVES > 1) *reinterpret_cast<uint4*>(vrow + KV_HALF_BYTES + c * 16) = make_uint4(0, 0, 0, 0);
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P must be visible to the tensor cores' reads
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) bar_arrive(&p_ready[j & 1]);
    }
    if (ok && n_tiles > 1 && !bar_wait(&pv_done[n_tiles & 1], ((n_tiles - 2) >> 1) & 1)) { atomicExch(error, 16); ok = false; }
    if (ok && n_tiles > 0 && !bar_wait(&pv_done[(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1)) { atomicExch(error, 16); ok = false; }
  }
  // ---- the second block's part goes to the first ------------------------------------------------------------
  // In the first block's shared memory, where its keys and values were: O as [head dim / 4][row][4] floats (64 KB,
  // 16 bytes per thread and store, no bank conflicts on either side), then reference and sum per row.
  const bool softmax_warp = warp >= 2 && warp < 6;
  float* xo = reinterpret_cast<float*>(sK);
  float* xml = reinterpret_cast<float*>(sK + HD * BM * 4);   // [2][BM], after O (which ends inside P's second buffer)
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");   // the first block's products are done with that memory
  if (softmax_warp && rank == 1) {
    unsigned remote_o, remote_ml;
    asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(remote_o) : "r"(s32(xo)));
    asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(remote_ml) : "r"(s32(xml)));
    const bool have = ok && n_tiles > 0;
    if (have) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
      for (int c0 = 0; c0 < HD; c0 += 32) {
        float o[32];
        tmem_ld32(tmem_o + lane_addr + c0, o);
#pragma unroll
        for (int i = 0; i < 32; i += 4)
          asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};"
                       ::"r"(remote_o + (unsigned)((((c0 + i) >> 2) * BM + r) * 16)), "f"(o[i]), "f"(o[i + 1]), "f"(o[i + 2]), "f"(o[i + 3])
                       : "memory");
      }
    }
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote_ml + (unsigned)(r * 4)), "f"(have ? m : -INFINITY) : "memory");
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote_ml + (unsigned)((BM + r) * 4)), "f"(have ? l : 0.f) : "memory");
  }
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");   // it has arrived
  if (softmax_warp && rank == 0) {
    if (ok) {
      // O = O0 * 2^(m0 - m) + O1 * 2^(m1 - m) with m the larger reference, the sums alike; then O / sum
      const float m1 = xml[r], l1 = xml[BM + r];
      const float mm = fmaxf(m, m1);
      const float f0 = m == -INFINITY ? 0.f : exp2f(m - mm), f1 = (m1 == -INFINITY || l1 == 0.f) ? 0.f : exp2f(m1 - mm);
      // with the keys cut into chunks the sum stays unnormalised (relative to the reference mm): the merge kernel divides
      const float inv = n_chunks > 1 ? 1.f : 1.f / (l * f0 + l1 * f1);
      const float g0 = f0 * inv, g1 = f1 * inv;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      __nv_bfloat16* dst = out + (size_t)(r_begin + tile * BM + r) * out_ld + h * HD;
      float* pdst = n_chunks > 1 ? partial + (((size_t)(r_begin + tile * BM + r - row0) * n_head + h) * n_chunks + chunk) * (HD + 4)
                                 : nullptr;
      if (pdst && r < rows_here) *reinterpret_cast<float2*>(pdst + HD) = make_float2(mm, l * f0 + l1 * f1);
#pragma unroll 1
      for (int c0 = 0; c0 < HD; c0 += 32) {
        float o[32];
        tmem_ld32(tmem_o + lane_addr + c0, o);
        if (r < rows_here) {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            float4 o1 = make_float4(0.f, 0.f, 0.f, 0.f);
            if (f1 != 0.f) o1 = *reinterpret_cast<const float4*>(xo + (((c0 + i) >> 2) * BM + r) * 4);
            o[i] = (f0 != 0.f ? o[i] * g0 : 0.f) + o1.x * g1;
            o[i + 1] = (f0 != 0.f ? o[i + 1] * g0 : 0.f) + o1.y * g1;
            o[i + 2] = (f0 != 0.f ? o[i + 2] * g0 : 0.f) + o1.z * g1;
            o[i + 3] = (f0 != 0.f ? o[i + 3] * g0 : 0.f) + o1.w * g1;
          }
          if (pdst) {
#pragma unroll
            for (int i = 0; i < 32; i += 4)
              *reinterpret_cast<float4*>(pdst + c0 + i) = make_float4(o[i], o[i + 1], o[i + 2], o[i + 3]);
            continue;
          }
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 q4;
            __nv_bfloat162 a = __floats2bfloat162_rn(o[i], o[i + 1]), b = __floats2bfloat162_rn(o[i + 2], o[i + 3]);
            __nv_bfloat162 c = __floats2bfloat162_rn(o[i + 4], o[i + 5]), d = __floats2bfloat162_rn(o[i + 6], o[i + 7]);
            q4.x = *reinterpret_cast<unsigned*>(&a);
            q4.y = *reinterpret_cast<unsigned*>(&b);
            q4.z = *reinterpret_cast<unsigned*>(&c);
            q4.w = *reinterpret_cast<unsigned*>(&d);
            *reinterpret_cast<uint4*>(dst + c0 + i) = q4;
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_s), "r"(256) : "memory");
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

// q: [total_rows, q_ld] bfloat16 with head h in columns h*hd..; kc/vc: [num_pages, n_kv_head, ps, hd].
// With n_chunks > 1 the keys are cut into chunks of chunk_keys (a multiple of 64) over as many clusters: partial holds
// n_rows * n_head * n_chunks * (hd + 4) floats for the rows row0 .. row0+n_rows-1 (those of the segments), positions the
// position of every row of the step, and a second kernel merges the chunks of these rows.
// Takes head sizes 64 and 128 and page sizes 8, 16, 32, 64, 128; refuses anything else.
CBIS_EXPORT int cbis_paged_prefill_tc5(const void* q, int q_ld, int total_rows, const void* kc, const void* vc,
                                       int num_pages, const int* block_table, int max_blocks, const int* cu_rows,
                                       const int* seg_start, void* out, int out_ld, int seg0, int n_seg,
                                       int max_seg_rows, int n_head, int n_kv_head, int hd, int ps, float scale,
                                       int window, int n_chunks, int chunk_keys, float* partial, const int* positions,
                                       int row0, int n_rows, int* error, void* stream) {
  if (n_seg <= 0 || max_seg_rows <= 0) return CBIS_OK;
  if (n_chunks < 1 || (n_chunks > 1 && (chunk_keys <= 0 || chunk_keys % tc5::BN || !partial || !positions || n_rows <= 0 ||
                                        ((uintptr_t)partial & 15))))
    return CBIS_ERR_BAD_SIZE;
  if ((hd != 128 && hd != 64) || ps < 8 || ps > 128 || (ps & (ps - 1)) || n_head <= 0 || n_kv_head <= 0 || n_head % n_kv_head)
    return CBIS_ERR_BAD_SIZE;
  if (q_ld % 8 || out_ld % 8 || ((uintptr_t)q & 15) || ((uintptr_t)kc & 15) || ((uintptr_t)vc & 15) ||
      ((uintptr_t)out & 15) || error == nullptr)
    return CBIS_ERR_ALIGNMENT;
  CUtensorMap map_q, map_k, map_v;
  int st = tc5::make_map(&map_q, q, total_rows, n_head * hd, q_ld, tc5::BM);
  if (st != CBIS_OK) return st;
  const long long cache_rows = (long long)num_pages * n_kv_head * ps;
  st = tc5::make_map(&map_k, kc, cache_rows, hd, hd, ps < tc5::BN ? ps : tc5::BN);
  if (st != CBIS_OK) return st;
  st = tc5::make_map(&map_v, vc, cache_rows, hd, hd, ps < tc5::BN ? ps : tc5::BN);
  if (st != CBIS_OK) return st;
  const size_t smem = tc5::smem_bytes(hd);
  auto kern = hd == 128 ? tc5::paged_prefill_tc5_kernel<128> : tc5::paged_prefill_tc5_kernel<64>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
  if (e != cudaSuccess) return (int)e;
  dim3 grid(2u * (unsigned)((max_seg_rows + tc5::BM - 1) / tc5::BM) * n_head * n_seg * n_chunks);
  e = launch_pdl(kern, grid, dim3(tc5::THREADS), smem, (cudaStream_t)stream, map_q, map_k, map_v, block_table, max_blocks,
                 cu_rows, seg_start, (__nv_bfloat16*)out, out_ld, seg0, n_seg, n_head, n_kv_head, ps,
                 scale * 1.4426950408889634f, window, n_chunks, chunk_keys, partial, row0, error);
  if (e == cudaSuccess && n_chunks > 1)
    e = launch_pdl(prefill_merge_kernel<__nv_bfloat16, true>, dim3(n_rows), dim3(128), 0, (cudaStream_t)stream,
                   (const float*)partial, positions, (const int*)nullptr, (__nv_bfloat16*)out, out_ld, row0, n_head, hd, window,
                   n_chunks, chunk_keys);
  return (int)e;
}

// How many blocks of the kernel above an SM has room for at a time (it is sized for two), worked out from what a
// block takes (registers as compiled, dynamic + static + reserved shared memory, 256 of the 512 columns of tensor
// memory) and what the device's SMs have; negative: a CUDA error.  (The occupancy calls of the runtime answer for
// whole clusters and count an SM pair once; the profiler's counters show two blocks per SM at work.)
CBIS_EXPORT int cbis_paged_prefill_tc5_blocks_per_sm() {
  auto kern = tc5::paged_prefill_tc5_kernel<128>;
  cudaFuncAttributes fa;
  cudaError_t e = cudaFuncGetAttributes(&fa, kern);
  if (e != cudaSuccess) return -(int)e;
  int dev = 0, smem_sm = 0, smem_reserved = 0, regs_sm = 0, threads_sm = 0;
  e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return -(int)e;
  if ((e = cudaDeviceGetAttribute(&smem_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev)) != cudaSuccess) return -(int)e;
  if ((e = cudaDeviceGetAttribute(&smem_reserved, cudaDevAttrReservedSharedMemoryPerBlock, dev)) != cudaSuccess) return -(int)e;
  if ((e = cudaDeviceGetAttribute(&regs_sm, cudaDevAttrMaxRegistersPerMultiprocessor, dev)) != cudaSuccess) return -(int)e;
  if ((e = cudaDeviceGetAttribute(&threads_sm, cudaDevAttrMaxThreadsPerMultiProcessor, dev)) != cudaSuccess) return -(int)e;
  const int warps = (tc5::THREADS + 31) / 32;
  const int regs_block = warps * ((fa.numRegs * 32 + 255) / 256 * 256);          // registers come in units of 256 per warp
  const int smem_block = (tc5::smem_bytes(128) + (int)fa.sharedSizeBytes + smem_reserved + 127) / 128 * 128;
  int n = smem_sm / smem_block;
  n = regs_sm / regs_block < n ? regs_sm / regs_block : n;
  n = threads_sm / tc5::THREADS < n ? threads_sm / tc5::THREADS : n;
  n = 512 / 256 < n ? 512 / 256 : n;                                             // tensor-memory columns
  return n;
}
