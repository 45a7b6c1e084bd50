// A run of pre-norm layers (LayerNorm, attention over the paged cache, LayerNorm, dense feed-forward) for a
// decode step of up to 16 rows, as ONE persistent kernel: one block per SM stays for the whole run.
//
// The reference issues 19 launches per layer (src/transformer.cpp:67-90); the chain of this package's own decode
// kernels still has 7, and at a few rows each of them is over before the memory system has reached its stride:
// the boundaries cost a third of the step.  Here the weights of ALL products of ALL layers of the run are one
// stream per block:
//   * block b owns the output columns [b*N/G, (b+1)*N/G) of every product (G blocks), over the whole of K;
//   * a producer warp walks the whole schedule (layer by layer: QKV, O, FC, PROJ) and brings the block's rows of
//     each weight matrix into a ring of shared-memory stages with TMA (cp.async.bulk.tensor, 128-byte swizzle,
//     mbarrier transaction counts).  It never waits for activations, so the stream from HBM goes on while the
//     working warps normalise, attend, reduce or wait for the other blocks;
//   * eight working warps split the K range of a stage among them, feed the tensor cores (mma.sync m16n8k16: the
//     few rows of the step are the M side, the K order of both operands permuted alike so that a 16-byte piece is
//     two fragments), add their partial sums through shared memory and apply bias, GELU or the residual add on the
//     32-bit sums;
//   * LayerNorm is recomputed by every block from the 32-bit residual rows in L2 into shared memory (statistics in
//     32-bit, centred variance), so it costs no exchange between blocks;
//   * the attention of a (row, head, split of the keys) is the device function of the stand-alone decode kernel,
//     given to groups of four warps; it also stores the current token's key and value into their page;
//   * where a product needs ALL columns of its input (after QKV, after the attention, after O, after FC, after
//     PROJ) the blocks meet at a counter in global memory.
// Every wait (mbarrier, counter) is bounded: when a limit runs out the block sets *error and an abort flag, stops
// issuing work, waits for its copies in flight and returns.  All blocks must be resident at once: the launcher
// starts at most one block per SM and checks that the kernel fits.
#include "attention_decode_tc.cuh"

#include <cuda.h>
#include <mutex>
#include <string.h>

namespace cbis {
namespace dl {

constexpr int CONSUMER_WARPS = 8;
constexpr int CONSUMERS = CONSUMER_WARPS * 32;
constexpr int THREADS = CONSUMERS + 32;            // + the producer warp
constexpr int STAGE_BYTES = 28 * 1024;
constexpr int MAX_SUBS = 16;                       // 64-column pieces per stage at most (four 32-column blocks per warp)
constexpr int MAXKB = 2 * MAX_SUBS / CONSUMER_WARPS;
constexpr unsigned SPIN_LIMIT = 1u << 22;
constexpr int BAR_CONSUMERS = 1, BAR_GROUP0 = 2;   // hardware barriers: all working warps; the two attention groups (2, 3)

struct Product {        // one matrix product of a layer, as every block sees it
  int N, K;
  int box_rows;         // rows of W a block loads: ceil(N / blocks)
  int sub_pitch;        // bytes from one 64-column piece to the next inside a stage (box_rows * 128 rounded up to 1024)
  int subs_per_stage;   // 64-column pieces per stage
  int n_sub;            // ceil(K / 64)
};

struct LayerDesc {      // per layer, in global memory
  const float *ln1_g, *ln1_b, *b_qkv, *b_o, *ln2_g, *ln2_b, *b_fc, *b_proj;
  __nv_bfloat16 *kc, *vc;
  float eps1, eps2;
};

struct Params {
  const CUtensorMap* maps;      // [n_layers][4]: QKV, O, FC, PROJ weights as [N, K] tensors, boxes of box_rows x 64
  const LayerDesc* layers;
  int n_layers;
  Product prod[4];
  int M, d, d_q, d_kv, F, n_head, n_kv_head, ps, act, window, nsplit, max_blocks, n_stages;
  float scale;
  float* x;                     // [M, d] residual stream, 32-bit
  __nv_bfloat16 *qkv, *attn, *hidden;   // [M, d_q + 2 d_kv], [M, d_q], [M, F]
  const int *block_table, *row_seq, *positions, *slot_mapping;
  float* part;
  unsigned int* counters;
  unsigned int* grid_counter;   // zero at launch
  int* error;
  int a_pitch, red_cols;        // shared-memory row pitches: normalised rows (elements), partial sums (floats)
  unsigned long long* trace;    // measuring aid (null in service): block 0 notes the time at every phase boundary
};

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
__device__ __forceinline__ bool bar_try(void* bar, unsigned parity) {
  unsigned ok;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(ok) : "r"(s32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Waits for the phase of the given parity; false when the limit ran out or another thread of the block gave up.
__device__ __forceinline__ bool bar_wait(void* bar, unsigned parity, volatile int* abort_flag) {
  for (unsigned it = 0; it < SPIN_LIMIT; ++it) {
    if (bar_try(bar, parity)) return true;
    if (*abort_flag) return false;
  }
  return false;
}
__device__ __forceinline__ void tma_2d(void* smem, const CUtensorMap* map, int x, int y, void* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(s32(smem)), "l"(map), "r"(x), "r"(y), "r"(s32(bar)) : "memory");
}
__device__ __forceinline__ uint4 lds16(const void* p) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(s32(p)));
  return v;
}
__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void consumer_sync() { group_sync(BAR_CONSUMERS, CONSUMERS); }

struct Shared {           // what the roles of a block share besides the ring
  unsigned long long full[8], empty[8];
  volatile int abort_flag;   // set by whoever gives up; may change at any time
  volatile int go_on;        // the working warps' common decision after a meeting (written by one thread between two barriers)
};

// The blocks meet: every working thread's global writes so far are visible to every block afterwards.
// `target`: arrivals the counter must show (the number of meetings so far times the number of blocks).
__device__ __forceinline__ bool grid_meet(const Params& p, unsigned target, Shared* sh, int ctid) {
  consumer_sync();
  if (ctid == 0) {
    if (!sh->abort_flag) {
      __threadfence();
      atomicAdd(p.grid_counter, 1u);
      unsigned spins = 0;
      while (ld_acquire(p.grid_counter) < target) {
        if (++spins > SPIN_LIMIT || sh->abort_flag) {
          sh->abort_flag = 1;
          atomicExch(p.error, 31);
          break;
        }
      }
      __threadfence();
    }
    sh->go_on = !sh->abort_flag;   // one reading for all: the flag itself may change under the others' eyes
  }
  consumer_sync();
  return sh->go_on != 0;
}

enum { EPI_STORE = 0, EPI_ADD_X = 1 };

// Measuring aid: block 0 writes the nanosecond timer at the n-th phase boundary (12 per layer, 256 at most).
__device__ __forceinline__ void stamp(const Params& p, int ctid, int& n) {
  if (p.trace && blockIdx.x == 0 && ctid == 0 && n < 256) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    p.trace[n] = t;
  }
  ++n;
}

// LayerNorm of the step's rows from the residual stream (L2) into shared memory as bfloat16 [Mpad][pitch]; the
// columns from d to the next multiple of 64 are zero (the products' last piece along K reads them).
template <bool LOW8>
__device__ __forceinline__ void norm_rows(const Params& p, const float* __restrict__ gamma, const float* __restrict__ beta,
                                          float eps, __nv_bfloat16* A, int cw, int lane) {
  constexpr int MPAD = LOW8 ? 8 : 16;
  const int d = p.d, nvec = d >> 2, pitch = p.a_pitch;
  const int dpad = (d + 63) & ~63;
  for (int m = cw; m < MPAD; m += CONSUMER_WARPS) {
    __nv_bfloat16* arow = A + (size_t)m * pitch;
    if (m >= p.M) {
      for (int c = lane; c < dpad; c += 32) arow[c] = __float2bfloat16_rn(0.f);
      continue;
    }
    const float4* xrow = reinterpret_cast<const float4*>(p.x + (size_t)m * d);
    float mean, inv;
    if (nvec <= 32 * 16) {   // the row stays in registers
      float4 v[16];
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int c = lane + 32 * i;
        v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < nvec) {
          v[i] = __ldcg(xrow + c);
          sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
        }
      }
      mean = warp_sum(sum) / (float)d;
      float sq = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        if (lane + 32 * i < nvec) {
          const float a = v[i].x - mean, b = v[i].y - mean, c2 = v[i].z - mean, e = v[i].w - mean;
          sq += (a * a + b * b) + (c2 * c2 + e * e);
        }
      }
      inv = rsqrtf(warp_sum(sq) / (float)d + eps);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int c = lane + 32 * i;
        if (c < nvec) {
          const float4 gm = __ldg(reinterpret_cast<const float4*>(gamma) + c);
          const float4 bt = __ldg(reinterpret_cast<const float4*>(beta) + c);
          __nv_bfloat162 lo = __floats2bfloat162_rn((v[i].x - mean) * inv * gm.x + bt.x, (v[i].y - mean) * inv * gm.y + bt.y);
          __nv_bfloat162 hi = __floats2bfloat162_rn((v[i].z - mean) * inv * gm.z + bt.z, (v[i].w - mean) * inv * gm.w + bt.w);
          uint2 r;
          r.x = *reinterpret_cast<unsigned*>(&lo);
          r.y = *reinterpret_cast<unsigned*>(&hi);
          *reinterpret_cast<uint2*>(arow + 4 * c) = r;
        }
      }
    } else {                 // wider rows are read from L2 three times
      float sum = 0.f;
      for (int c = lane; c < nvec; c += 32) {
        const float4 v = __ldcg(xrow + c);
        sum += (v.x + v.y) + (v.z + v.w);
      }
      mean = warp_sum(sum) / (float)d;
      float sq = 0.f;
      for (int c = lane; c < nvec; c += 32) {
        const float4 v = __ldcg(xrow + c);
        const float a = v.x - mean, b = v.y - mean, c2 = v.z - mean, e = v.w - mean;
        sq += (a * a + b * b) + (c2 * c2 + e * e);
      }
      inv = rsqrtf(warp_sum(sq) / (float)d + eps);
      for (int c = lane; c < nvec; c += 32) {
        const float4 v = __ldcg(xrow + c);
        const float4 gm = __ldg(reinterpret_cast<const float4*>(gamma) + c);
        const float4 bt = __ldg(reinterpret_cast<const float4*>(beta) + c);
        __nv_bfloat162 lo = __floats2bfloat162_rn((v.x - mean) * inv * gm.x + bt.x, (v.y - mean) * inv * gm.y + bt.y);
        __nv_bfloat162 hi = __floats2bfloat162_rn((v.z - mean) * inv * gm.z + bt.z, (v.w - mean) * inv * gm.w + bt.w);
        uint2 r;
        r.x = *reinterpret_cast<unsigned*>(&lo);
        r.y = *reinterpret_cast<unsigned*>(&hi);
        *reinterpret_cast<uint2*>(arow + 4 * c) = r;
      }
    }
    for (int c = d + lane; c < dpad; c += 32) arow[c] = __float2bfloat16_rn(0.f);
  }
}

// One product by the working warps: acc += A[M, K] * W[rows of this block, K]^T stage by stage from the ring, then
// the partial sums of the warps are added and the epilogue applied.  A_SMEM: A is the normalised rows in shared
// memory; else A [M, lda] bfloat16 in global memory, fetched a stage ahead into registers.
// `it`: stages consumed so far by this block (the producer counts the same way).
template <int NT, bool A_SMEM, bool LOW8>
__device__ __forceinline__ void product(const Params& p, const Product& pr, unsigned& it, unsigned char* ring,
                                        Shared* sh, const __nv_bfloat16* a_smem, const __nv_bfloat16* a_glob, int lda,
                                        float* red, const float* __restrict__ bias, int epi, int act,
                                        __nv_bfloat16* out, int ldo, int cw, int lane) {
  constexpr int MPAD = LOW8 ? 8 : 16;
  const int g = lane >> 2, t = lane & 3;
  const int n_lo = (int)(((long long)blockIdx.x * pr.N) / gridDim.x);
  const int n_hi = (int)(((long long)(blockIdx.x + 1) * pr.N) / gridDim.x);
  const int rows_mine = n_hi - n_lo;
  const int nt_used = (pr.box_rows + 7) >> 3;
  const int ctid = cw * 32 + lane;
  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

  uint4 nxt_lo[MAXKB], nxt_hi[MAXKB];
  const int row_lo = min(g, p.M - 1), row_hi = min(g + 8, p.M - 1);
  auto fetch_a = [&](int sub0) {   // this warp's pieces of A for the stage that starts at piece sub0
    const int nkb = 2 * min(pr.subs_per_stage, pr.n_sub - sub0);
#pragma unroll
    for (int i = 0; i < MAXKB; ++i) {
      const int kbi = cw + CONSUMER_WARPS * i;
      nxt_lo[i] = nxt_hi[i] = make_uint4(0, 0, 0, 0);
      if (kbi < nkb) {
        const int k0 = (sub0 + (kbi >> 1)) * 64 + (kbi & 1) * 32 + t * 8;
        if (k0 < pr.K) {
          nxt_lo[i] = ldcg16(a_glob + (size_t)row_lo * lda + k0);
          if (!LOW8) nxt_hi[i] = ldcg16(a_glob + (size_t)row_hi * lda + k0);
        }
      }
    }
  };
  if (!A_SMEM) fetch_a(0);

  bool ok = __all_sync(0xffffffffu, !sh->abort_flag);
  for (int sub0 = 0; sub0 < pr.n_sub && ok; sub0 += pr.subs_per_stage, ++it) {
    const unsigned slot = it % (unsigned)p.n_stages, use = it / (unsigned)p.n_stages;
    const int nsub = min(pr.subs_per_stage, pr.n_sub - sub0);
    uint4 cur_lo[MAXKB], cur_hi[MAXKB];
    if (!A_SMEM) {
#pragma unroll
      for (int i = 0; i < MAXKB; ++i) {
        cur_lo[i] = nxt_lo[i];
        cur_hi[i] = nxt_hi[i];
      }
      if (sub0 + pr.subs_per_stage < pr.n_sub) fetch_a(sub0 + pr.subs_per_stage);   // in flight during this stage
    }
    // every lane sees the phase complete itself; the warp goes on only if all did
    if (!__all_sync(0xffffffffu, bar_wait(&sh->full[slot], use & 1, &sh->abort_flag))) {
      if (!sh->abort_flag) {
        sh->abort_flag = 1;
        atomicExch(p.error, 32);
      }
      ok = false;
      break;
    }
    const unsigned char* stage = ring + (size_t)slot * STAGE_BYTES;
#pragma unroll
    for (int i = 0; i < MAXKB; ++i) {
      const int kbi = cw + CONSUMER_WARPS * i;
      if (kbi < 2 * nsub) {
        const int sub = kbi >> 1, kbs = kbi & 1;
        uint4 lo, hi = make_uint4(0, 0, 0, 0);
        if (A_SMEM) {
          const int k0 = (sub0 + sub) * 64 + kbs * 32 + t * 8;
          lo = lds16(a_smem + (size_t)g * p.a_pitch + k0);
          if (!LOW8) hi = lds16(a_smem + (size_t)(g + 8) * p.a_pitch + k0);
        } else {
          lo = cur_lo[i];
          hi = cur_hi[i];
        }
        const unsigned char* tile = stage + (size_t)sub * pr.sub_pitch;
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          if (j < nt_used) {
            const int r = j * 8 + g;
            const uint4 b = lds16(tile + r * 128 + (((kbs * 4 + t) ^ (r & 7)) << 4));
            mma_16816(acc[j], lo.x, hi.x, lo.y, hi.y, b.x, b.y);
            mma_16816(acc[j], lo.z, hi.z, lo.w, hi.w, b.z, b.w);
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) bar_arrive(&sh->empty[slot]);
  }
  // the warps' partial sums meet in shared memory: red[warp][row][column]
  const int rc = p.red_cols;
  float* mine = red + (size_t)cw * MPAD * rc;
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    if (j < nt_used) {
      mine[g * rc + j * 8 + 2 * t] = acc[j][0];
      mine[g * rc + j * 8 + 2 * t + 1] = acc[j][1];
      if (!LOW8) {
        mine[(g + 8) * rc + j * 8 + 2 * t] = acc[j][2];
        mine[(g + 8) * rc + j * 8 + 2 * t + 1] = acc[j][3];
      }
    }
  }
  consumer_sync();
  if (!sh->abort_flag) {
    for (int idx = ctid; idx < p.M * rows_mine; idx += CONSUMERS) {
      const int m = idx / rows_mine, c = idx - m * rows_mine;
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < CONSUMER_WARPS; ++w) v += red[((size_t)w * MPAD + m) * rc + c];
      const int n = n_lo + c;
      if (bias) v += __ldg(bias + n);
      if (epi == EPI_STORE) {
        out[(size_t)m * ldo + n] = __float2bfloat16_rn(activate(v, act));
      } else {
        float* xp = p.x + (size_t)m * p.d + n;
        *xp = __ldcg(xp) + v;
      }
    }
  }
  consumer_sync();
}

template <bool A_SMEM, bool LOW8>
__device__ __forceinline__ void product_any(const Params& p, const Product& pr, unsigned& it, unsigned char* ring,
                                            Shared* sh, const __nv_bfloat16* a_smem, const __nv_bfloat16* a_glob, int lda,
                                            float* red, const float* bias, int epi, int act, __nv_bfloat16* out, int ldo,
                                            int cw, int lane) {
  const int nt = (pr.box_rows + 7) >> 3;
  if (nt <= 2) product<2, A_SMEM, LOW8>(p, pr, it, ring, sh, a_smem, a_glob, lda, red, bias, epi, act, out, ldo, cw, lane);
  else if (nt <= 4) product<4, A_SMEM, LOW8>(p, pr, it, ring, sh, a_smem, a_glob, lda, red, bias, epi, act, out, ldo, cw, lane);
  else if (nt <= 8) product<8, A_SMEM, LOW8>(p, pr, it, ring, sh, a_smem, a_glob, lda, red, bias, epi, act, out, ldo, cw, lane);
  else product<16, A_SMEM, LOW8>(p, pr, it, ring, sh, a_smem, a_glob, lda, red, bias, epi, act, out, ldo, cw, lane);
}

template <int HD, bool LOW8>
__global__ void __launch_bounds__(THREADS, 1) decode_layers_kernel(const __grid_constant__ Params p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  constexpr int MPAD = LOW8 ? 8 : 16;
  unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __nv_bfloat16* a_smem = reinterpret_cast<__nv_bfloat16*>(ring + (size_t)p.n_stages * STAGE_BYTES);
  float* red = reinterpret_cast<float*>(a_smem + (size_t)MPAD * p.a_pitch);
  DecodeTcShared<HD>* att = reinterpret_cast<DecodeTcShared<HD>*>(red + (size_t)CONSUMER_WARPS * MPAD * p.red_cols);
  Shared* sh = reinterpret_cast<Shared*>((reinterpret_cast<uintptr_t>(att + 2) + 15) & ~(uintptr_t)15);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < p.n_stages; ++s) {
      bar_init(&sh->full[s], 1);
      bar_init(&sh->empty[s], CONSUMER_WARPS);
    }
    sh->abort_flag = 0;
    sh->go_on = 1;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();
  pdl_trigger();

  if (warp == CONSUMER_WARPS) {
    // ---- the producer: the block's rows of every weight matrix, in the order the working warps use them ----
    if (lane == 0) {
      unsigned it = 0;
      bool ok = true;
      for (int l = 0; l < p.n_layers && ok; ++l) {
        for (int q = 0; q < 4 && ok; ++q) {
          const Product& pr = p.prod[q];
          const CUtensorMap* map = p.maps + (size_t)l * 4 + q;
          const int n_lo = (int)(((long long)blockIdx.x * pr.N) / gridDim.x);
          for (int sub0 = 0; sub0 < pr.n_sub; sub0 += pr.subs_per_stage, ++it) {
            const unsigned slot = it % (unsigned)p.n_stages, use = it / (unsigned)p.n_stages;
            if (use > 0 && !bar_wait(&sh->empty[slot], (use - 1) & 1, &sh->abort_flag)) {
              if (!sh->abort_flag) {
                sh->abort_flag = 1;
                atomicExch(p.error, 33);
              }
              ok = false;
              break;
            }
            if (sh->abort_flag) {
              ok = false;
              break;
            }
            const int nsub = min(pr.subs_per_stage, pr.n_sub - sub0);
            unsigned char* stage = ring + (size_t)slot * STAGE_BYTES;
            bar_expect(&sh->full[slot], (unsigned)(nsub * pr.box_rows * 128));
            for (int i = 0; i < nsub; ++i)
              tma_2d(stage + (size_t)i * pr.sub_pitch, map, (sub0 + i) * 64, n_lo, &sh->full[slot]);
          }
        }
      }
      if (!ok || sh->abort_flag) {
        // a give-up somewhere in the block: the copies requested last may still be on their way into shared memory,
        // and the block must not leave before they have landed
        for (unsigned j = it > (unsigned)p.n_stages ? it - p.n_stages : 0; j < it; ++j) {
          bool landed = false;
          for (unsigned tries = 0; tries < SPIN_LIMIT && !landed; ++tries)
            landed = bar_try(&sh->full[j % p.n_stages], (j / p.n_stages) & 1);
          if (!landed) atomicExch(p.error, 34);
        }
      }
    }
    return;
  }

  // ---- the working warps ----
  const int cw = warp, ctid = threadIdx.x;
  const int group = cw / DEC_WARPS, gtid = ctid % (DEC_WARPS * 32);
  const int n_qkv = p.d_q + 2 * p.d_kv;
  unsigned it = 0, meetings = 0;
  int ns = 0;
  pdl_wait();   // the residual stream comes from the kernel before
  bool ok = true;
  for (int l = 0; l < p.n_layers && ok; ++l) {
    const LayerDesc L = p.layers[l];
    stamp(p, ctid, ns);
    // q | k | v = LN1(x) W^T + b
    norm_rows<LOW8>(p, L.ln1_g, L.ln1_b, L.eps1, a_smem, cw, lane);
    consumer_sync();
    stamp(p, ctid, ns);
    product_any<true, LOW8>(p, p.prod[0], it, ring, sh, a_smem, nullptr, 0, red, L.b_qkv, EPI_STORE, CBIS_ACT_NONE, p.qkv,
                            n_qkv, cw, lane);
    stamp(p, ctid, ns);
    if (!(ok = grid_meet(p, ++meetings * gridDim.x, sh, ctid))) break;
    stamp(p, ctid, ns);
    // attention: (row, head, split) items over the groups of four warps of all blocks
    {
      const int n_items = p.M * p.n_head * p.nsplit, n_groups = gridDim.x * (CONSUMER_WARPS / DEC_WARPS);
      for (int item = blockIdx.x * (CONSUMER_WARPS / DEC_WARPS) + group; item < n_items; item += n_groups) {
        const int split = item % p.nsplit, rh = item / p.nsplit;
        decode_tc_item<HD, false>(p.qkv, n_qkv, p.d_q, p.d_q + p.d_kv, L.kc, L.vc, p.block_table, p.max_blocks, p.row_seq,
                                  p.positions, p.slot_mapping, p.attn, p.d_q, p.part, p.counters, p.n_head, p.n_kv_head,
                                  p.ps, p.scale, p.window, p.nsplit, rh / p.n_head, rh % p.n_head, split, gtid, att[group],
                                  BAR_GROUP0 + group);
        group_sync(BAR_GROUP0 + group, DEC_WARPS * 32);
      }
    }
    stamp(p, ctid, ns);
    if (!(ok = grid_meet(p, ++meetings * gridDim.x, sh, ctid))) break;
    stamp(p, ctid, ns);
    // x += attn W_o^T + b_o
    product_any<false, LOW8>(p, p.prod[1], it, ring, sh, nullptr, p.attn, p.d_q, red, L.b_o, EPI_ADD_X, 0, nullptr, 0, cw, lane);
    stamp(p, ctid, ns);
    if (!(ok = grid_meet(p, ++meetings * gridDim.x, sh, ctid))) break;
    stamp(p, ctid, ns);
    // hidden = act(LN2(x) W_fc^T + b_fc)
    norm_rows<LOW8>(p, L.ln2_g, L.ln2_b, L.eps2, a_smem, cw, lane);
    consumer_sync();
    stamp(p, ctid, ns);
    product_any<true, LOW8>(p, p.prod[2], it, ring, sh, a_smem, nullptr, 0, red, L.b_fc, EPI_STORE, p.act, p.hidden, p.F, cw, lane);
    stamp(p, ctid, ns);
    if (!(ok = grid_meet(p, ++meetings * gridDim.x, sh, ctid))) break;
    stamp(p, ctid, ns);
    // x += hidden W_proj^T + b_proj
    product_any<false, LOW8>(p, p.prod[3], it, ring, sh, nullptr, p.hidden, p.F, red, L.b_proj, EPI_ADD_X, 0, nullptr, 0, cw, lane);
    stamp(p, ctid, ns);
    if (l + 1 < p.n_layers && !(ok = grid_meet(p, ++meetings * gridDim.x, sh, ctid))) break;
  }
  stamp(p, ctid, ns);
}

// ---- host side --------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* q = nullptr;
    cudaDriverEntryPointQueryResult r;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &q, cudaEnableDefault, &r) == cudaSuccess &&
        r == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(q);
  });
  return fn;
}

static void plan_product(Product* pr, int N, int K, int blocks) {
  pr->N = N;
  pr->K = K;
  pr->box_rows = (N + blocks - 1) / blocks;
  pr->sub_pitch = (pr->box_rows * 128 + 1023) / 1024 * 1024;
  int s = STAGE_BYTES / pr->sub_pitch;
  pr->subs_per_stage = s < 1 ? 1 : (s > MAX_SUBS ? MAX_SUBS : s);
  pr->n_sub = (K + 63) / 64;
}

static size_t shared_bytes(int n_stages, int mpad, int a_pitch, int red_cols, int hd) {
  const size_t att = hd == 128 ? sizeof(DecodeTcShared<128>) : sizeof(DecodeTcShared<64>);
  return 1024 + (size_t)n_stages * STAGE_BYTES + (size_t)mpad * a_pitch * 2 + (size_t)CONSUMER_WARPS * mpad * red_cols * 4 +
         2 * att + sizeof(Shared) + 64;
}

}  // namespace dl
}  // namespace cbis

using namespace cbis;

// How many blocks the persistent decode kernel runs with on the current device: one per SM, fewer when the
// narrowest product has fewer than 8 columns per block.
CBIS_EXPORT int cbis_decode_layers_blocks(int n_min) {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return -1;
  int b = n_min / 8;
  b = b < 1 ? 1 : b;
  return b < sms ? b : sms;
}

// Writes the 128-byte tensor map of a weight matrix W [N, K] bfloat16 (K contiguous, 16-byte aligned, K a multiple of 8)
// for `blocks` blocks into `out` (host memory): boxes of ceil(N / blocks) rows by 64 columns, 128-byte swizzle.
CBIS_EXPORT int cbis_decode_layers_map(void* out, const void* w, int N, int K, int blocks) {
  dl::EncodeTiledFn fn = dl::encode_fn();
  if (!fn || !out || !w || N <= 0 || K <= 0 || K % 8 || blocks <= 0) return CBIS_ERR_BAD_SIZE;
  if ((uintptr_t)w & 15) return CBIS_ERR_ALIGNMENT;
  const int box_rows = (N + blocks - 1) / blocks;
  if (box_rows > 128) return CBIS_ERR_TOO_LARGE;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)N};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  CUtensorMap map;
  const CUresult r = fn(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(w), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return CBIS_ERR_BAD_SIZE;
  memcpy(out, &map, sizeof(map));
  return CBIS_OK;
}

// Bytes of one per-layer record in the device array `layers` (8 float pointers, 2 cache pointers, 2 floats).
CBIS_EXPORT int cbis_decode_layers_desc_bytes() { return (int)sizeof(dl::LayerDesc); }

// Runs `n_layers` layers on the M rows of a decode step (see the top of this file).
// maps: device array of n_layers * 4 tensor maps made by cbis_decode_layers_map with the same `blocks`;
// layers: device array of n_layers records; x [M, d] float; qkv [M, d_q + 2 d_kv], attn [M, d_q], hidden [M, F]
// bfloat16 scratch; part / counters: the decode attention's scratch for M rows, n_head heads and nsplit splits
// (counters zero); grid_counter: one unsigned int, zero at launch; error: int, set non-zero if a wait ran out;
// trace: null, or 256 x 8 bytes that take block 0's timer at every phase boundary (12 per layer) for measuring.
// Refuses (CBIS_ERR_BAD_SIZE / CBIS_ERR_TOO_LARGE) what it does not take: the caller then runs the layers kernel by kernel.
CBIS_EXPORT int cbis_decode_layers(const void* maps, const void* layers, int n_layers, int blocks, int M, int d, int n_head,
                                   int n_kv_head, int hd, int F, int ps, int act, int window, float scale, int nsplit,
                                   float* x, void* qkv, void* attn, void* hidden, const int* block_table, int max_blocks,
                                   const int* row_seq, const int* positions, const int* slot_mapping, float* part,
                                   unsigned int* counters, unsigned int* grid_counter, int* error, void* stream,
                                   unsigned long long* trace) {
  if (n_layers <= 0 || M <= 0) return CBIS_OK;
  if (M > 16 || (hd != 64 && hd != 128) || ps <= 0 || ps % 16 || d <= 0 || d % 8 || F <= 0 || F % 8 || n_head <= 0 ||
      n_kv_head <= 0 || n_head % n_kv_head || nsplit < 1 || nsplit > 32 || blocks <= 0)
    return CBIS_ERR_BAD_SIZE;
  if (((uintptr_t)maps & 63) || ((uintptr_t)x & 15) || ((uintptr_t)qkv & 15) || ((uintptr_t)attn & 15) || ((uintptr_t)hidden & 15) ||
      !grid_counter || !error)
    return CBIS_ERR_ALIGNMENT;
  int dev = 0, sms = 0, smem_max = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaDeviceGetAttribute(&smem_max, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  if (blocks > sms) return CBIS_ERR_BAD_SIZE;
  dl::Params p = {};
  p.maps = static_cast<const CUtensorMap*>(maps);
  p.layers = static_cast<const dl::LayerDesc*>(layers);
  p.n_layers = n_layers;
  p.M = M; p.d = d; p.d_q = n_head * hd; p.d_kv = n_kv_head * hd; p.F = F; p.n_head = n_head; p.n_kv_head = n_kv_head;
  p.ps = ps; p.act = act; p.window = window; p.nsplit = nsplit; p.max_blocks = max_blocks; p.scale = scale;
  p.x = x; p.qkv = (__nv_bfloat16*)qkv; p.attn = (__nv_bfloat16*)attn; p.hidden = (__nv_bfloat16*)hidden;
  p.block_table = block_table; p.row_seq = row_seq; p.positions = positions; p.slot_mapping = slot_mapping;
  p.part = part; p.counters = counters; p.grid_counter = grid_counter; p.error = error; p.trace = trace;
  dl::plan_product(&p.prod[0], p.d_q + 2 * p.d_kv, d, blocks);
  dl::plan_product(&p.prod[1], d, p.d_q, blocks);
  dl::plan_product(&p.prod[2], F, d, blocks);
  dl::plan_product(&p.prod[3], d, F, blocks);
  int box_max = 0;
  for (int q = 0; q < 4; ++q) {
    if (p.prod[q].box_rows > 128) return CBIS_ERR_TOO_LARGE;
    box_max = p.prod[q].box_rows > box_max ? p.prod[q].box_rows : box_max;
  }
  const bool low8 = M <= 8;
  const int mpad = low8 ? 8 : 16;
  p.a_pitch = ((d + 63) & ~63) + 8;
  p.red_cols = ((box_max + 7) & ~7) + 1;
  int n_stages = 8;
  while (n_stages >= 3 && dl::shared_bytes(n_stages, mpad, p.a_pitch, p.red_cols, hd) > (size_t)smem_max) --n_stages;
  if (n_stages < 3) return CBIS_ERR_TOO_LARGE;
  p.n_stages = n_stages;
  const size_t smem = dl::shared_bytes(n_stages, mpad, p.a_pitch, p.red_cols, hd);
  void (*kern)(const dl::Params);
  if (hd == 128) kern = low8 ? dl::decode_layers_kernel<128, true> : dl::decode_layers_kernel<128, false>;
  else kern = low8 ? dl::decode_layers_kernel<64, true> : dl::decode_layers_kernel<64, false>;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  int per_sm = 0;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, dl::THREADS, smem);
  if (e != cudaSuccess) return (int)e;
  if (per_sm < 1) return CBIS_ERR_TOO_LARGE;     // the blocks wait for one another: all of them must be resident
  return (int)launch_pdl(kern, dim3(blocks), dim3(dl::THREADS), smem, (cudaStream_t)stream, p);
}
