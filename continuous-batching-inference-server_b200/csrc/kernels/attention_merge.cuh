// Merge of partial attention results over chunks of keys, shared by the attention kernels that cut a long
// context over several blocks.  A block that took chunk c of the keys of (row, head) left, in scratch memory,
// hd unnormalised sums, its maximum m_c and its denominator l_c ((hd + 4) floats); the row's result is
// sum_c w_c o_c / sum_c w_c l_c with w_c = exp(m_c - max_c m_c), the online-softmax merge of the reference's
// running (m, l, acc) (kernels/attention.cu:74-95) applied across chunks.  Chunks are runs of chunk_keys keys by
// absolute index, so the chunks of a row are those that hold a key of max(0, p - window + 1) .. p.
#pragma once
#include "common.cuh"
#include <cuda_bf16.h>
#include <math.h>

namespace cbis {

// grid: the rows row0 .. row0+gridDim.x-1 of the step; a thread takes 4 head dims of one head at a time.
// row_seq (may be null): the request of every row, negative for padding rows.
// BASE2: the maxima are in the base-2 domain (scores times log2 e), else natural.
template <typename TO, bool BASE2>
__global__ void __launch_bounds__(128)
prefill_merge_kernel(const float* partial, const int* positions, const int* row_seq, TO* out, int out_ld, int row0,
                     int n_head, int hd, int window, int n_chunks, int chunk_keys) {
  pdl_trigger();
  pdl_wait();
  const int row = row0 + blockIdx.x;
  if (row_seq && row_seq[row] < 0) return;   // a padding row of a fixed-size batch: nothing was computed for it
  const int p = positions[row];
  const int c_lo = (window > 0 ? max(0, p - window + 1) : 0) / chunk_keys, c_hi = p / chunk_keys;
  const int units = n_head * (hd / 4);
  for (int u = threadIdx.x; u < units; u += blockDim.x) {
    const int h = u / (hd / 4), d = (u % (hd / 4)) * 4;
    const float* src = partial + ((size_t)blockIdx.x * n_head + h) * n_chunks * (hd + 4);
    float mx = -INFINITY;
    for (int c = c_lo; c <= c_hi; ++c) mx = fmaxf(mx, src[(size_t)c * (hd + 4) + hd]);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float l = 0.f;
    for (int c = c_lo; c <= c_hi; ++c) {
      const float* s = src + (size_t)c * (hd + 4);
      const float w = BASE2 ? exp2f(s[hd] - mx) : expf(s[hd] - mx);   // a chunk without a visible key: maximum -inf, weight 0
      const float4 o = *reinterpret_cast<const float4*>(s + d);
      acc.x = fmaf(w, o.x, acc.x);
      acc.y = fmaf(w, o.y, acc.y);
      acc.z = fmaf(w, o.z, acc.z);
      acc.w = fmaf(w, o.w, acc.w);
      l = fmaf(w, s[hd + 1], l);
    }
    const float inv = 1.f / l;
    TO* dst = out + (size_t)row * out_ld + h * hd + d;
    if constexpr (sizeof(TO) == 4) {
      *reinterpret_cast<float4*>(dst) = make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
    } else {
      __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x * inv, acc.y * inv), hi = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
      uint2 v;
      v.x = *reinterpret_cast<uint32_t*>(&lo);
      v.y = *reinterpret_cast<uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(dst) = v;
    }
  }
}

}  // namespace cbis
