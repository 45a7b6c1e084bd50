// Decode attention over the paged cache for bfloat16: one query token per request, keys split
// over several blocks (split-KV); the block of a (row, head) that finishes last merges the
// partial softmax states.
//
// The reference runs one warp per (row, head) that walks the keys one after the other
// (kernels/attention.cu:57-98): at decode that is n_head warps per request and a chain of
// dependent loads.  Here a block of 4 warps takes (row, head, split); inside it the lanes are
// grouped LPK to a key, each lane holding 8 head dims (one 16-byte load per key for K and one for
// V, rows read in full 16-byte pieces side by side), every group keeps its own running
// (max, sum, acc) over the keys it meets, four keys in flight per group, and the groups, warps and
// splits are merged at the end with the usual rescaling.  All softmax arithmetic is 32-bit.
//
// The current token's key and value can come straight from the step's projections (`k_off >= 0`):
// the block that meets position p takes them from `qkv` and stores them into the page, so the
// separate cache-write launch is not needed at decode.
#include "attention_decode_tc.cuh"
#include <math.h>

namespace cbis {

constexpr int DEC_U = 4;  // keys in flight per lane group

// part: [rows][n_head][nsplit][hd + 2] floats: acc[hd] (not normalised), max, sum.
template <int LPK>
__global__ void __launch_bounds__(DEC_WARPS * 32)
paged_decode_bf16_kernel(const __nv_bfloat16* qkv, int ld, int k_off, int v_off,
                         __nv_bfloat16* kc, __nv_bfloat16* vc,
                         const int* block_table, int max_blocks, const int* row_seq,
                         const int* positions, const int* slot_mapping,
                         __nv_bfloat16* __restrict__ out, int out_ld, float* part,
                         unsigned int* counters, int n_head, int n_kv_head, int hd, int ps, float scale,
                         int window, int nsplit) {
  constexpr int G = 32 / LPK;             // key groups per warp
  constexpr int NW = DEC_WARPS * G;       // key workers per block
  __shared__ float sm_m[DEC_WARPS], sm_l[DEC_WARPS];
  __shared__ float sm_acc[DEC_WARPS][256];
  __shared__ bool is_last;
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x, h = blockIdx.y, split = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int seq = row_seq[row];
  if (seq < 0) {  // a padding row of a fixed-size batch
    if (split == 0)
      for (int t = threadIdx.x; t < hd; t += blockDim.x) out[(size_t)row * out_ld + h * hd + t] = __float2bfloat16_rn(0.f);
    return;
  }
  const int hk = h / (n_head / n_kv_head);
  const int pos = positions[row];
  const int kend = pos + 1;
  const int kstart = window > 0 ? max(0, kend - window) : 0;
  const int per = (((kend - kstart) + nsplit - 1) / nsplit + 31) & ~31;
  const int ks = kstart + split * per;
  const int ke = min(kend, ks + per);
  const int sub = lane % LPK, group = lane / LPK;
  const bool active = sub * 8 < hd;
  const int* bt = block_table + (size_t)seq * max_blocks;
  const bool fused = k_off >= 0;

  float q[8];
  {
    uint4 raw = make_uint4(0, 0, 0, 0);
    if (active) raw = *reinterpret_cast<const uint4*>(qkv + (size_t)row * ld + h * hd + sub * 8);
    unpack8(raw, q);
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] *= scale;
  }
  float m = -INFINITY, l = 0.f, acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;

  const int wkr = warp * G + group;
  uint4 knext[DEC_U], vnext[DEC_U];
  // Loads of the keys/values base + u*NW + wkr (u < DEC_U); the current token's pair comes from qkv and is stored.
  auto fetch = [&](int base, uint4* kk, uint4* vv) {
#pragma unroll
    for (int u = 0; u < DEC_U; ++u) {
      const int j = base + u * NW + wkr;
      kk[u] = make_uint4(0, 0, 0, 0);
      vv[u] = make_uint4(0, 0, 0, 0);
      if (j < ke && active) {
        if (fused && j == pos) {
          kk[u] = *reinterpret_cast<const uint4*>(qkv + (size_t)row * ld + k_off + hk * hd + sub * 8);
          vv[u] = *reinterpret_cast<const uint4*>(qkv + (size_t)row * ld + v_off + hk * hd + sub * 8);
          const int slot = slot_mapping[row];
          if (slot >= 0) {
            const size_t dst = (((size_t)(slot / ps) * n_kv_head + hk) * ps + (slot % ps)) * hd + sub * 8;
            *reinterpret_cast<uint4*>(kc + dst) = kk[u];
            *reinterpret_cast<uint4*>(vc + dst) = vv[u];
          }
        } else {
          const int page = bt[j / ps];
          const size_t src = (((size_t)page * n_kv_head + hk) * ps + (j % ps)) * hd + sub * 8;
          kk[u] = *reinterpret_cast<const uint4*>(kc + src);
          vv[u] = *reinterpret_cast<const uint4*>(vc + src);
        }
      }
    }
  };
  if (ks < ke) fetch(ks, knext, vnext);
  for (int base = ks; base < ke; base += NW * DEC_U) {
    uint4 kraw[DEC_U], vraw[DEC_U];
    bool valid[DEC_U];
#pragma unroll
    for (int u = 0; u < DEC_U; ++u) {
      kraw[u] = knext[u];
      vraw[u] = vnext[u];
      valid[u] = base + u * NW + wkr < ke;
    }
    if (base + NW * DEC_U < ke) fetch(base + NW * DEC_U, knext, vnext);  // the next batch is in flight during the math
    float s[DEC_U];
#pragma unroll
    for (int u = 0; u < DEC_U; ++u) {
      float kf[8];
      unpack8(kraw[u], kf);
      float d = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) d = fmaf(q[i], kf[i], d);
#pragma unroll
      for (int o = LPK / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
      s[u] = valid[u] ? d : -INFINITY;
    }
    float m_new = m;
#pragma unroll
    for (int u = 0; u < DEC_U; ++u) m_new = fmaxf(m_new, s[u]);
    if (m_new > -INFINITY) {  // uniform within a lane group; no shuffles below
      const float corr = expf(m - m_new);
      float p[DEC_U], psum = 0.f;
#pragma unroll
      for (int u = 0; u < DEC_U; ++u) {
        p[u] = expf(s[u] - m_new);
        psum += p[u];
      }
      l = l * corr + psum;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] *= corr;
#pragma unroll
      for (int u = 0; u < DEC_U; ++u) {
        float vf[8];
        unpack8(vraw[u], vf);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = fmaf(p[u], vf[i], acc[i]);
      }
      m = m_new;
    }
  }
  // merge the lane groups of the warp
#pragma unroll
  for (int o = LPK; o < 32; o <<= 1) {
    const float mo = __shfl_xor_sync(0xffffffffu, m, o);
    const float lo = __shfl_xor_sync(0xffffffffu, l, o);
    const float M = fmaxf(m, mo);
    const float a = m > -INFINITY ? expf(m - M) : 0.f;
    const float b = mo > -INFINITY ? expf(mo - M) : 0.f;
    l = l * a + lo * b;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float ao = __shfl_xor_sync(0xffffffffu, acc[i], o);
      acc[i] = acc[i] * a + ao * b;
    }
    m = M;
  }
  if (lane == 0) {
    sm_m[warp] = m;
    sm_l[warp] = l;
  }
  if (group == 0 && active) {
#pragma unroll
    for (int i = 0; i < 8; ++i) sm_acc[warp][sub * 8 + i] = acc[i];
  }
  __syncthreads();
  float M = -INFINITY;
#pragma unroll
  for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, sm_m[w]);
  float wgt[DEC_WARPS], L = 0.f;
#pragma unroll
  for (int w = 0; w < DEC_WARPS; ++w) {
    wgt[w] = sm_m[w] > -INFINITY ? expf(sm_m[w] - M) : 0.f;
    L += sm_l[w] * wgt[w];
  }
  for (int t = threadIdx.x; t < hd; t += blockDim.x) {
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) v += sm_acc[w][t] * wgt[w];
    if (nsplit == 1) {
      out[(size_t)row * out_ld + h * hd + t] = __float2bfloat16_rn(v / L);
    } else {
      float* p = part + (((size_t)row * n_head + h) * nsplit + split) * (hd + 2);
      p[t] = v;
      if (t == 0) {
        p[hd] = M;
        p[hd + 1] = L;
      }
    }
  }
  if (nsplit == 1) return;
  // The block of this (row, head) that finishes last merges the splits (and sets the counter back to zero).
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) is_last = atomicAdd(&counters[row * n_head + h], 1u) == (unsigned)nsplit - 1;
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  const float* p = part + ((size_t)row * n_head + h) * nsplit * (hd + 2);
  float Mx = -INFINITY;
  for (int s = 0; s < nsplit; ++s) Mx = fmaxf(Mx, __ldcg(p + (size_t)s * (hd + 2) + hd));
  for (int t = threadIdx.x; t < hd; t += blockDim.x) {
    float Ls = 0.f, v = 0.f;
    for (int s = 0; s < nsplit; ++s) {
      const float* ps_ = p + (size_t)s * (hd + 2);
      const float ms = __ldcg(ps_ + hd);
      const float w = ms > -INFINITY ? expf(ms - Mx) : 0.f;
      Ls += __ldcg(ps_ + hd + 1) * w;
      v += __ldcg(ps_ + t) * w;
    }
    out[(size_t)row * out_ld + h * hd + t] = __float2bfloat16_rn(v / Ls);
  }
  if (threadIdx.x == 0) counters[row * n_head + h] = 0;
}

// ---------------------------------------------------------------------------------------------
// The fast form for head sizes 64 and 128 and pages of a multiple of 16 keys: decode_tc_item of
// attention_decode_tc.cuh, one block of four warps per (row, head, split).
// ---------------------------------------------------------------------------------------------
template <int HD>
__global__ void __launch_bounds__(DEC_WARPS * 32, 4)   // 128 registers: four blocks per SM
paged_decode_tc_kernel(const __nv_bfloat16* qkv, int ld, int k_off, int v_off, __nv_bfloat16* kc, __nv_bfloat16* vc,
                       const int* block_table, int max_blocks, const int* row_seq, const int* positions,
                       const int* slot_mapping, __nv_bfloat16* __restrict__ out, int out_ld, float* part,
                       unsigned int* counters, int n_head, int n_kv_head, int ps, float scale, int window,
                       int nsplit) {
  __shared__ DecodeTcShared<HD> sm;
  pdl_trigger();
  decode_tc_item<HD, true, (HD <= 64 ? 2 : 1)>(qkv, ld, k_off, v_off, kc, vc, block_table, max_blocks, row_seq, positions, slot_mapping, out,
                           out_ld, part, counters, n_head, n_kv_head, ps, scale, window, nsplit, blockIdx.x, blockIdx.y,
                           blockIdx.z, threadIdx.x, sm, 0);
}

// After a decode step whose next tokens were chosen on the device: the chosen token becomes the
// row's input, its position moves on by one, and so do the segment's first position and length.
__global__ void decode_advance_kernel(int* tokens, int* positions, int* seg_start, int* seg_ctx,
                                      const int* sampled, int n) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= n) return;
  tokens[r] = sampled[r];
  positions[r] += 1;
  seg_start[r] += 1;
  seg_ctx[r] += 1;
}

// slot_mapping[r] = page(position) * page_size + offset, from the request's block table; -1 for padding rows
// and for positions whose page is not there.
__global__ void slots_from_table_kernel(const int* positions, const int* row_seq,
                                        const int* block_table, int max_blocks, int ps,
                                        int* slot_mapping, int n) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= n) return;
  const int seq = row_seq[r], pos = positions[r];
  int slot = -1;
  if (seq >= 0 && pos >= 0 && pos / ps < max_blocks) {
    const int page = block_table[(size_t)seq * max_blocks + pos / ps];
    if (page >= 0) slot = page * ps + pos % ps;
  }
  slot_mapping[r] = slot;
}

}  // namespace cbis

using namespace cbis;

// Scratch of the decode kernel for `rows` rows split `nsplit` ways: `part` holds
// cbis_paged_decode_scratch_floats() floats of partial results; `counters` holds rows*n_head
// unsigned ints that are zero before the first launch (every launch leaves them zero).  The two
// are separate so that a region once used for partial results is never read as a counter.
CBIS_EXPORT long long cbis_paged_decode_scratch_floats(int rows, int n_head, int hd, int nsplit) {
  return nsplit <= 1 ? 0 : (long long)rows * n_head * nsplit * (hd + 2);
}

// qkv: this step's projections [rows, ld], queries at column 0.  k_off/v_off >= 0: take the current
// token's key/value from qkv and store them at slot_mapping[row]; < 0: the cache holds them already.
CBIS_EXPORT int cbis_paged_decode_bf16(const void* qkv, int ld, int k_off, int v_off, void* kc, void* vc,
                                       const int* block_table, int max_blocks, const int* row_seq,
                                       const int* positions, const int* slot_mapping, void* out, int out_ld,
                                       float* part, unsigned int* counters, int rows, int n_head, int n_kv_head,
                                       int hd, int ps, float scale, int window, int nsplit, void* stream) {
  if (rows <= 0) return CBIS_OK;
  if (hd <= 0 || hd > 256 || hd % 8 || ps <= 0 || n_head <= 0 || n_kv_head <= 0 || n_head % n_kv_head || nsplit < 1 || nsplit > 32)
    return CBIS_ERR_BAD_SIZE;
  if (ld % 8 || out_ld % 8 || (k_off >= 0 && (k_off % 8 || v_off % 8)) || ((uintptr_t)qkv & 15) || ((uintptr_t)kc & 15) ||
      ((uintptr_t)vc & 15))
    return CBIS_ERR_ALIGNMENT;
  if (nsplit > 1 && (part == nullptr || counters == nullptr)) return CBIS_ERR_BAD_SIZE;
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid(rows, n_head, nsplit);
  const int chunks = hd / 8;
  cudaError_t e;
  if ((hd == 64 || hd == 128) && ps % 16 == 0) {
    if (hd == 128)
      e = launch_pdl(paged_decode_tc_kernel<128>, grid, dim3(DEC_WARPS * 32), 0, st, (const __nv_bfloat16*)qkv, ld, k_off,
                     v_off, (__nv_bfloat16*)kc, (__nv_bfloat16*)vc, block_table, max_blocks, row_seq, positions,
                     slot_mapping, (__nv_bfloat16*)out, out_ld, part, counters, n_head, n_kv_head, ps, scale, window,
                     nsplit);
    else
      e = launch_pdl(paged_decode_tc_kernel<64>, grid, dim3(DEC_WARPS * 32), 0, st, (const __nv_bfloat16*)qkv, ld, k_off,
                     v_off, (__nv_bfloat16*)kc, (__nv_bfloat16*)vc, block_table, max_blocks, row_seq, positions,
                     slot_mapping, (__nv_bfloat16*)out, out_ld, part, counters, n_head, n_kv_head, ps, scale, window,
                     nsplit);
    return (int)e;
  }
#define CBIS_DEC(LPK)                                                                                             \
  e = launch_pdl(paged_decode_bf16_kernel<LPK>, grid, dim3(DEC_WARPS * 32), 0, st, (const __nv_bfloat16*)qkv, ld, \
                 k_off, v_off, (__nv_bfloat16*)kc, (__nv_bfloat16*)vc, block_table, max_blocks, row_seq, positions, \
                 slot_mapping, (__nv_bfloat16*)out, out_ld, part, counters, n_head, n_kv_head, hd, ps, scale, window, \
                 nsplit)
  if (chunks <= 2) CBIS_DEC(2);
  else if (chunks <= 4) CBIS_DEC(4);
  else if (chunks <= 8) CBIS_DEC(8);
  else if (chunks <= 16) CBIS_DEC(16);
  else CBIS_DEC(32);
#undef CBIS_DEC
  return (int)e;
}

CBIS_EXPORT int cbis_decode_advance(int* tokens, int* positions, int* seg_start, int* seg_ctx, const int* sampled,
                                    int n, void* stream) {
  if (n <= 0) return CBIS_OK;
  return (int)launch_pdl(decode_advance_kernel, dim3((n + 127) / 128), dim3(128), 0, (cudaStream_t)stream, tokens,
                         positions, seg_start, seg_ctx, sampled, n);
}

CBIS_EXPORT int cbis_slots_from_table(const int* positions, const int* row_seq, const int* block_table, int max_blocks,
                                      int ps, int* slot_mapping, int n, void* stream) {
  if (n <= 0) return CBIS_OK;
  if (ps <= 0) return CBIS_ERR_BAD_SIZE;
  return (int)launch_pdl(slots_from_table_kernel, dim3((n + 127) / 128), dim3(128), 0, (cudaStream_t)stream, positions,
                         row_seq, block_table, max_blocks, ps, slot_mapping, n);
}
