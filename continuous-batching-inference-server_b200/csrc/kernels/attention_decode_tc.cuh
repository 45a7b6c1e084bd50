// The split-KV decode attention for head sizes 64 and 128 on pages of a multiple of 16 keys, as a device function
// for a group of four warps: the stand-alone kernel (attention_decode.cu) gives it a block, the persistent decode
// kernel (decode_layers.cu) gives it half of its working warps at a time.
#pragma once
#include "common.cuh"
#include <math.h>

namespace cbis {

constexpr int DEC_WARPS = 4;

// Eight bfloat16 -> float with shifts and masks (a bfloat16 is the upper half of the float): the conversion
// instruction runs on the special-function pipe, which the value tiles of a decode step kept 58 % busy.
__device__ __forceinline__ void unpack8(const uint4& r, float* f) {
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

// All `n` threads (a multiple of 32) of a group meet at the hardware barrier `id` (id 0 with a whole block's
// threads is __syncthreads).
__device__ __forceinline__ void group_sync(int id, int n) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }

// ---------------------------------------------------------------------------------------------
// The fast form for head sizes 64 and 128 and pages of a multiple of 16 keys.  A warp takes 16
// keys of a page at a time: K and V of the tile are each one contiguous run in the page, fetched
// with 16-byte loads that bypass L1.  The 16 scores come from the tensor cores (mma.sync
// m16n8k16, the query in row 0 of the A operand, the K order of both operands permuted alike so
// that a 16-byte load of a key is two B fragments); they are scaled and masked in 32-bit, the
// running (max, sum) is kept in 32-bit, and P*V is accumulated in 32-bit on the FP32 units from
// the coalesced V loads.  That is about a sixth of the instructions per key of the form above,
// which issues too many to keep up with HBM.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 ldcg16(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
// Keys and values are read once per step: they are marked to leave L2 first, so that they do not push
// out the weights that the products have prefetched.
__device__ __forceinline__ unsigned long long l2_evict_first_policy() {
  unsigned long long pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\n" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ uint4 ldcg16_stream(const void* p, unsigned long long pol) {
  uint4 v;
  asm volatile("ld.global.cg.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p), "l"(pol));
  return v;
}

__device__ __forceinline__ void mma_16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Shared memory of one group of four warps.
template <int HD>
struct DecodeTcShared {
  float m[DEC_WARPS], l[DEC_WARPS];
  float acc[DEC_WARPS][HD];
  float p[DEC_WARPS][32];      // a warp's weights of the keys of its one or two tiles
  float w[32];
  float inv;
  int is_last;
};

// One (row, head, split) by a group of DEC_WARPS warps: `tid` is the thread's index in the group (0..127), `bar` the
// hardware barrier the group meets at.  STANDALONE: the group is a block launched for this alone, which waits for
// the kernels ahead (programmatic dependent launch) after it has fetched what they do not write.  The group's
// threads must have met (group_sync) between two calls, since the calls share `sm`.
template <int HD, bool STANDALONE, int TPW = 1>
__device__ __forceinline__ void decode_tc_item(const __nv_bfloat16* qkv, int ld, int k_off, int v_off, __nv_bfloat16* kc,
                                               __nv_bfloat16* vc, const int* block_table, int max_blocks,
                                               const int* row_seq, const int* positions, const int* slot_mapping,
                                               __nv_bfloat16* out, int out_ld, float* part, unsigned int* counters,
                                               int n_head, int n_kv_head, int ps, float scale, int window, int nsplit,
                                               int row, int h, int split, int tid, DecodeTcShared<HD>& sm, int bar) {
  constexpr int NC = HD / 32;        // 16-byte loads per key for the score fragments (4 lanes x 16 B = 32 dims each)
  constexpr int LPK = HD / 8;        // lanes per key in the coalesced V loads
  constexpr int KPL = 32 / LPK;      // keys per warp-wide V load
  constexpr int NV = 16 / KPL;       // V loads per 16-key tile
  constexpr int NT = DEC_WARPS * 32;
  // TPW: 16-key tiles a warp fetches together and takes through one update of its running maximum and sum.  The
  // stand-alone kernel takes two at head size 64: as many bytes on their way per warp (8 KB) as at head size 128,
  // and half the bookkeeping per key.
  static_assert(TPW == 1 || TPW == 2, "the warp's weights have room for two tiles");
  // The step's tables (rows, positions, block tables) were written before the step's first kernel and the
  // cached keys and values of earlier positions by earlier steps: they are read, and this warp's first
  // tile is fetched, while the kernels ahead (the projection of this step's q, k, v) still run.
  const int lane = tid & 31, warp = tid >> 5;
  const int seq = row_seq[row];
  if (seq < 0) {  // a padding row of a fixed-size batch
    if (STANDALONE) pdl_wait();
    if (split == 0)
      for (int t = tid; t < HD; t += NT) out[(size_t)row * out_ld + h * HD + t] = __float2bfloat16_rn(0.f);
    return;
  }
  const int hk = h / (n_head / n_kv_head);
  const int pos = positions[row];
  const int kend = pos + 1;
  const int kstart = window > 0 ? max(0, kend - window) : 0;
  const int first_tile = kstart >> 4;
  const int per = (((kend - (first_tile << 4)) + nsplit - 1) / nsplit + 31) & ~31;   // keys per split, whole tiles
  const int ks = (first_tile << 4) + split * per;
  const int ke = min(kend, ks + per);
  const int* bt = block_table + (size_t)seq * max_blocks;
  const int g = lane >> 2, t = lane & 3;

  const int vsub = lane % LPK, vgrp = lane / LPK;
  const int ps_shift = (ps & (ps - 1)) == 0 ? 31 - __clz(ps) : -1;
  const unsigned long long pol = l2_evict_first_policy();
  uint4 kb[TPW][2][NC], vb[TPW][NV];
  // The warp's TPW tiles from `tile` on, as far as they hold keys of this split: the keys first (with the tiles'
  // places in the pages, kept for the values), the values later.
  size_t base[TPW];
  auto load_keys = [&](int tile) {
#pragma unroll
    for (int u = 0; u < TPW; ++u) {
      const int j0 = (tile + u) << 4;
      if (j0 < ke) {
        const int pi = ps_shift >= 0 ? (j0 >> ps_shift) : j0 / ps;      // a shift where the page size is a power of two
        base[u] = (((size_t)bt[pi] * n_kv_head + hk) * ps + (j0 - pi * ps)) * HD;   // 16 keys from here are one run
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int c = 0; c < NC; ++c)
            kb[u][nt][c] = ldcg16_stream(kc + base[u] + (size_t)(nt * 8 + g) * HD + c * 32 + t * 8, pol);
      }
    }
  };
  auto load_values = [&](int tile) {      // after load_keys(tile), before the next load_keys
#pragma unroll
    for (int u = 0; u < TPW; ++u)
      if (((tile + u) << 4) < ke) {
#pragma unroll
        for (int i = 0; i < NV; ++i) vb[u][i] = ldcg16_stream(vc + base[u] + (size_t)i * 256 + lane * 8, pol);
      }
  };
  int tile = (ks >> 4) + warp * TPW;
  // not the tiles that hold the current token: its key and value are stored below, after the wait
  const bool preloaded = (tile << 4) < ke && ((pos >> 4) < tile || (pos >> 4) >= tile + TPW);
  if (preloaded) {
    load_keys(tile);
    load_values(tile);
  }
  if (STANDALONE) pdl_wait();

  // The current token's key and value go into their page first; the loop below then reads them
  // like any other key.  (Blocks of query heads that share this key/value head store the same values.)
  if (k_off >= 0 && pos >= ks && pos < ke) {
    const int slot = slot_mapping[row];
    if (slot >= 0 && tid < 2 * LPK) {
      const int which = tid / LPK, sub = tid % LPK;
      const uint4 v = ldcg16(qkv + (size_t)row * ld + (which ? v_off : k_off) + hk * HD + sub * 8);
      const size_t dst = (((size_t)(slot / ps) * n_kv_head + hk) * ps + (slot % ps)) * HD + sub * 8;
      *reinterpret_cast<uint4*>((which ? vc : kc) + dst) = v;
    }
    group_sync(bar, NT);
  }

  // the query as A fragments: row 0 only, so lanes 0..3 hold it and the rest hold zeros
  uint4 qa[NC];
#pragma unroll
  for (int c = 0; c < NC; ++c)
    qa[c] = g == 0 ? ldcg16(qkv + (size_t)row * ld + h * HD + c * 32 + t * 8) : make_uint4(0, 0, 0, 0);

  float m = -INFINITY, l = 0.f, acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;

  // A round: the values of this round's tiles are asked for, the scores are taken from the keys (asked for a round
  // earlier), the keys of the next round are asked for, and the softmax update and P V of this round run while they
  // come: a warp has loads on their way nearly all the time, not only while it waits for them.
  bool have_keys = preloaded, have_values = preloaded;
  for (; (tile << 4) < ke; tile += DEC_WARPS * TPW) {
    if (!have_keys) load_keys(tile);
    if (!have_values) load_values(tile);
    have_values = false;
    // scores of the 16 keys of each tile: row 0 of the product sits in lanes 0..3 (keys 8nt + 2t, 8nt + 2t + 1).
    // The warp's tiles share one update of the running maximum and sum.
    float s4[TPW][4], mx = -INFINITY;
#pragma unroll
    for (int u = 0; u < TPW; ++u) {
      const int j0 = (tile + u) << 4;
      float sc[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
      if (j0 < ke) {                                  // uniform over the warp
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int c = 0; c < NC; ++c) {
            mma_16816(sc[nt], qa[c].x, 0u, qa[c].y, 0u, kb[u][nt][c].x, kb[u][nt][c].y);
            mma_16816(sc[nt], qa[c].z, 0u, qa[c].w, 0u, kb[u][nt][c].z, kb[u][nt][c].w);
          }
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = j0 + (e >> 1) * 8 + 2 * t + (e & 1);
        s4[u][e] = (g == 0 && j >= kstart && j < ke) ? sc[e >> 1][e & 1] * scale : -INFINITY;
        mx = fmaxf(mx, s4[u][e]);
      }
    }
    have_keys = ((tile + DEC_WARPS * TPW) << 4) < ke;
    if (have_keys) load_keys(tile + DEC_WARPS * TPW);   // the scores above were the last use of this round's keys
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    mx = __shfl_sync(0xffffffffu, mx, 0);
    const float m_new = fmaxf(m, mx);
    if (m_new == -INFINITY) continue;                 // no key of these tiles is in range (uniform over the warp)
    const float corr = expf(m - m_new);
    if (g == 0) {
      float psum = 0.f;
#pragma unroll
      for (int u = 0; u < TPW; ++u)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float p = expf(s4[u][e] - m_new);
          psum += p;
          sm.p[warp][u * 16 + (e >> 1) * 8 + 2 * t + (e & 1)] = p;
        }
      l = l * corr + psum;                            // lanes 0..3 each carry a part of the sum
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] *= corr;
#pragma unroll
    for (int u = 0; u < TPW; ++u) {
      if (((tile + u) << 4) < ke) {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          const float p = sm.p[warp][u * 16 + i * KPL + vgrp];
          if (p != 0.f) {                             // keys out of range have p = 0 and whatever the page holds
            float vf[8];
            unpack8(vb[u][i], vf);
#pragma unroll
            for (int d = 0; d < 8; ++d) acc[d] = fmaf(p, vf[d], acc[d]);
          }
        }
      }
    }
    __syncwarp();
    m = m_new;
  }
  // merge within the warp: the sum's parts (lanes 0..3) and the accumulators of the key groups
  l += __shfl_xor_sync(0xffffffffu, l, 1);
  l += __shfl_xor_sync(0xffffffffu, l, 2);
#pragma unroll
  for (int o = LPK; o < 32; o <<= 1)
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
  if (lane == 0) {
    sm.m[warp] = m;
    sm.l[warp] = l;
  }
  if (vgrp == 0) {
#pragma unroll
    for (int i = 0; i < 8; ++i) sm.acc[warp][vsub * 8 + i] = acc[i];
  }
  group_sync(bar, NT);
  float M = -INFINITY;
#pragma unroll
  for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, sm.m[w]);
  float wgt[DEC_WARPS], L = 0.f;
#pragma unroll
  for (int w = 0; w < DEC_WARPS; ++w) {
    wgt[w] = sm.m[w] > -INFINITY ? expf(sm.m[w] - M) : 0.f;
    L += sm.l[w] * wgt[w];
  }
  for (int tt = tid; tt < HD; tt += NT) {
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) v += sm.acc[w][tt] * wgt[w];
    if (nsplit == 1) {
      out[(size_t)row * out_ld + h * HD + tt] = __float2bfloat16_rn(v / L);
    } else {
      float* p = part + (((size_t)row * n_head + h) * nsplit + split) * (HD + 2);
      p[tt] = v;
      if (tt == 0) {
        p[HD] = M;
        p[HD + 1] = L;
      }
    }
  }
  if (nsplit == 1) return;
  __threadfence();
  group_sync(bar, NT);
  if (tid == 0) sm.is_last = atomicAdd(&counters[row * n_head + h], 1u) == (unsigned)nsplit - 1;
  group_sync(bar, NT);
  if (!sm.is_last) return;
  __threadfence();
  // weights of the splits first (one thread per split), then every thread sums its dims over the splits
  const float* p = part + ((size_t)row * n_head + h) * nsplit * (HD + 2);
  if (warp == 0) {
    const float ms = lane < nsplit ? __ldcg(p + (size_t)lane * (HD + 2) + HD) : -INFINITY;
    const float ls = lane < nsplit ? __ldcg(p + (size_t)lane * (HD + 2) + HD + 1) : 0.f;
    const float Mx = warp_max(ms);
    const float w = ms > -INFINITY ? expf(ms - Mx) : 0.f;
    sm.w[lane] = w;
    const float Ls = warp_sum(ls * w);
    if (lane == 0) sm.inv = 1.f / Ls;
  }
  group_sync(bar, NT);
  for (int tt = tid; tt < HD; tt += NT) {
    float v = 0.f;
#pragma unroll 8
    for (int s = 0; s < nsplit; ++s) v = fmaf(__ldcg(p + (size_t)s * (HD + 2) + tt), sm.w[s], v);
    out[(size_t)row * out_ld + h * HD + tt] = __float2bfloat16_rn(v * sm.inv);
  }
  if (tid == 0) counters[row * n_head + h] = 0;
}

}  // namespace cbis
