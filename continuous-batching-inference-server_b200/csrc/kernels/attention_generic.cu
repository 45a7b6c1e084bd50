// Paged key/value cache: writing a step's keys and values into pages, and a general
// attention kernel over the pages (any head size up to 256, any page size, query heads
// grouped over fewer key/value heads, optional window), in 32-bit arithmetic for both
// storage types.  It is the whole attention of the 32-bit path and the fallback of the
// bfloat16 path for head sizes the tensor-core kernels do not take.
//
// Cache of one layer: K and V each [num_pages][n_kv_head][page_size][head_dim]; the
// reference keeps [page][page_size][head][head_dim] (kernels/attention.cu:14,80).
#include "attention_merge.cuh"

namespace cbis {

// Row r of the step's projections goes to token slot slot_mapping[r] = page*page_size + offset
// (reference: scatter_kv_kernel, kernels/attention.cu:7-19).  A negative slot writes nothing.
template <typename TT>
__global__ void kv_write_kernel(const TT* qkv, int ld, int k_off, int v_off, TT* kc,
                                TT* vc, const int* slot_mapping, int n_kv_head,
                                int hd, int ps) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const int slot = slot_mapping[r];
  if (slot < 0) return;
  const int page = slot / ps, off = slot % ps;
  const TT* krow = qkv + (size_t)r * ld + k_off;
  const TT* vrow = qkv + (size_t)r * ld + v_off;
  const int width = n_kv_head * hd;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const int h = c / hd, i = c % hd;
    const size_t dst = (((size_t)page * n_kv_head + h) * ps + off) * hd + i;
    kc[dst] = krow[c];
    vc[dst] = vrow[c];
  }
}

// The same with 16-byte moves, for head sizes that are a multiple of 8 (bfloat16) or 4 (float).
template <typename TT>
__global__ void kv_write_vec_kernel(const TT* qkv, int ld, int k_off, int v_off, TT* kc, TT* vc,
                                    const int* slot_mapping, int n_kv_head, int hd, int ps) {
  constexpr int E = 16 / sizeof(TT);  // elements per 16 bytes
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const int slot = slot_mapping[r];
  if (slot < 0) return;
  const int page = slot / ps, off = slot % ps;
  const TT* krow = qkv + (size_t)r * ld + k_off;
  const TT* vrow = qkv + (size_t)r * ld + v_off;
  const int chunks = n_kv_head * hd / E, per_head = hd / E;
  for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
    const int h = c / per_head, i = (c % per_head) * E;
    const size_t dst = (((size_t)page * n_kv_head + h) * ps + off) * hd + i;
    *reinterpret_cast<uint4*>(kc + dst) = *reinterpret_cast<const uint4*>(krow + c * E);
    *reinterpret_cast<uint4*>(vc + dst) = *reinterpret_cast<const uint4*>(vrow + c * E);
  }
}

// One warp per (row, query head).  The query at position p sees keys max(0, p-window+1)..p
// (window 0: all keys 0..p; the loop bound is the causal mask, kernels/attention.cu:67-68,78).
// Online softmax with running max m, normaliser l and accumulator acc as in
// kernels/attention.cu:74-95, G keys at a time (the loads of a group are all in flight together: with four
// a short context was one round trip to memory per four keys, 36 us for 36 keys).  Lane i owns head dims
// i, i+32, ...  A group starts at kstart + a multiple of G, whatever the step brought: the logits do not depend
// on how a request was cut.
template <typename TT, int NPER, int G>
__global__ void paged_attention_generic_kernel(
    const TT* q, int q_ld, const TT* kc, const TT* vc,
    const int* block_table, int max_blocks, const int* row_seq,
    const int* positions, TT* __restrict__ out, int out_ld, int n_rows, int n_head, int n_kv_head,
    int hd, int ps, float scale, int window, int n_chunks, int chunk_keys, float* partial) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int wc = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (wc >= n_rows * n_head * n_chunks) return;
  const int w = wc / n_chunks, chunk = wc % n_chunks;
  const int row = w / n_head, h = w % n_head;
  const int hk = h / (n_head / n_kv_head);
  const int pos = positions[row];
  const int seq = row_seq[row];
  if (seq < 0) {  // a padding row of a fixed-size batch
    if (chunk == 0)
      for (int dim = lane; dim < hd; dim += 32) from_f32(out[(size_t)row * out_ld + h * hd + dim], 0.f);
    return;
  }
  const int* bt = block_table + (size_t)seq * max_blocks;
  int kend = pos + 1;
  int kstart = window > 0 ? max(0, kend - window) : 0;
  if (n_chunks > 1) {   // this warp's share of the keys: chunks by absolute index, merged by a second kernel
    kstart = max(kstart, chunk * chunk_keys);
    kend = min(kend, (chunk + 1) * chunk_keys);
    if (kstart >= kend) return;
  }

  float qv[NPER], acc[NPER];
#pragma unroll
  for (int i = 0; i < NPER; ++i) {
    const int dim = lane + 32 * i;
    qv[i] = dim < hd ? to_f32(q[(size_t)row * q_ld + h * hd + dim]) : 0.f;
    acc[i] = 0.f;
  }
  float m = -INFINITY, l = 0.f;

  for (int j0 = kstart; j0 < kend; j0 += G) {
    float s[G];
    const TT* vptr[G];
#pragma unroll
    for (int u = 0; u < G; ++u) {
      const int j = j0 + u;
      float part = 0.f;
      vptr[u] = nullptr;
      if (j < kend) {
        const int page = bt[j / ps];
        const size_t base = (((size_t)page * n_kv_head + hk) * ps + (j % ps)) * hd;
        const TT* kp = kc + base;
        vptr[u] = vc + base;
#pragma unroll
        for (int i = 0; i < NPER; ++i) {
          const int dim = lane + 32 * i;
          if (dim < hd) part = fmaf(qv[i], to_f32(kp[dim]), part);
        }
      }
      s[u] = part;
    }
#pragma unroll
    for (int u = 0; u < G; ++u) s[u] = (j0 + u < kend) ? warp_sum(s[u]) * scale : -INFINITY;
    float m_new = m;
#pragma unroll
    for (int u = 0; u < G; ++u) m_new = fmaxf(m_new, s[u]);
    const float corr = expf(m - m_new);  // first group: exp(-inf) = 0
    float p[G];
    float psum = 0.f;
#pragma unroll
    for (int u = 0; u < G; ++u) {
      p[u] = (j0 + u < kend) ? expf(s[u] - m_new) : 0.f;
      psum += p[u];
    }
    l = l * corr + psum;
#pragma unroll
    for (int i = 0; i < NPER; ++i) {
      const int dim = lane + 32 * i;
      float a = acc[i] * corr;
      if (dim < hd) {
#pragma unroll
        for (int u = 0; u < G; ++u)
          if (vptr[u]) a = fmaf(p[u], to_f32(vptr[u][dim]), a);
      }
      acc[i] = a;
    }
    m = m_new;
  }
  if (n_chunks > 1) {
    float* dst = partial + ((size_t)w * n_chunks + chunk) * (hd + 4);
#pragma unroll
    for (int i = 0; i < NPER; ++i) {
      const int dim = lane + 32 * i;
      if (dim < hd) dst[dim] = acc[i];
    }
    if (lane == 0) {
      dst[hd] = m;
      dst[hd + 1] = l;
    }
    return;
  }
  const float inv = 1.f / l;
#pragma unroll
  for (int i = 0; i < NPER; ++i) {
    const int dim = lane + 32 * i;
    if (dim < hd) from_f32(out[(size_t)row * out_ld + h * hd + dim], acc[i] * inv);
  }
}

}  // namespace cbis

using namespace cbis;

CBIS_EXPORT int cbis_kv_write(const void* qkv, int ld, int k_off, int v_off, void* kc, void* vc,
                              const int* slot_mapping, int T, int n_kv_head, int hd, int ps, int dtype,
                              void* stream) {
  if (T <= 0) return CBIS_OK;
  if (n_kv_head <= 0 || hd <= 0 || ps <= 0) return CBIS_ERR_BAD_SIZE;
  const int width = n_kv_head * hd;
  const int threads = width >= 1024 ? 256 : (width >= 256 ? 128 : 64);
  cudaStream_t st = (cudaStream_t)stream;
  const int esz = dtype == CBIS_F32 ? 4 : 2, per16 = 16 / esz;
  const bool vec = hd % per16 == 0 && ld % per16 == 0 && k_off % per16 == 0 && v_off % per16 == 0 &&
                   !(((uintptr_t)qkv | (uintptr_t)kc | (uintptr_t)vc) & 15);
  if (vec && dtype == CBIS_F32)
    return (int)launch_pdl(kv_write_vec_kernel<float>, dim3(T), dim3(128), 0, st, (const float*)qkv, ld, k_off, v_off,
                           (float*)kc, (float*)vc, slot_mapping, n_kv_head, hd, ps);
  if (vec && dtype == CBIS_BF16)
    return (int)launch_pdl(kv_write_vec_kernel<__nv_bfloat16>, dim3(T), dim3(128), 0, st, (const __nv_bfloat16*)qkv, ld,
                           k_off, v_off, (__nv_bfloat16*)kc, (__nv_bfloat16*)vc, slot_mapping, n_kv_head, hd, ps);
  if (dtype == CBIS_F32)
    return (int)launch_pdl(kv_write_kernel<float>, dim3(T), dim3(threads), 0, st, (const float*)qkv, ld, k_off, v_off,
                           (float*)kc, (float*)vc, slot_mapping, n_kv_head, hd, ps);
  if (dtype == CBIS_BF16)
    return (int)launch_pdl(kv_write_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, st, (const __nv_bfloat16*)qkv, ld,
                           k_off, v_off, (__nv_bfloat16*)kc, (__nv_bfloat16*)vc, slot_mapping, n_kv_head, hd, ps);
  return CBIS_ERR_BAD_DTYPE;
}

template <typename TT>
static int launch_generic(const void* q, int q_ld, const void* kc, const void* vc, const int* block_table,
                          int max_blocks, const int* row_seq, const int* positions, void* out, int out_ld,
                          int n_rows, int n_head, int n_kv_head, int hd, int ps, float scale, int window,
                          int n_chunks, int chunk_keys, float* partial, cudaStream_t st) {
  const int warps = 4;
  const long long total = (long long)n_rows * n_head * n_chunks;
  const int blocks = (int)((total + warps - 1) / warps);
  cudaError_t e;
#define CBIS_LAUNCH(NPER)                                                                                            \
  e = launch_pdl(paged_attention_generic_kernel<TT, NPER, (NPER <= 2 ? 16 : (NPER <= 4 ? 8 : 4))>, dim3(blocks), dim3(warps * 32), 0, st, (const TT*)q, q_ld, \
                 (const TT*)kc, (const TT*)vc, block_table, max_blocks, row_seq, positions, (TT*)out, out_ld, n_rows, \
                 n_head, n_kv_head, hd, ps, scale, window, n_chunks, chunk_keys, partial)
  if (hd <= 32) CBIS_LAUNCH(1);
  else if (hd <= 64) CBIS_LAUNCH(2);
  else if (hd <= 128) CBIS_LAUNCH(4);
  else CBIS_LAUNCH(8);
#undef CBIS_LAUNCH
  if (e == cudaSuccess && n_chunks > 1)
    e = launch_pdl(prefill_merge_kernel<TT, false>, dim3(n_rows), dim3(128), 0, st, (const float*)partial, positions, row_seq,
                   (TT*)out, out_ld, 0, n_head, hd, window, n_chunks, chunk_keys);
  return (int)e;
}

// With n_chunks > 1 (head sizes that are a multiple of 4, 16-byte aligned rows of out) every (row, head) is cut into
// chunks of chunk_keys keys over as many warps: partial holds n_rows * n_head * n_chunks * (hd + 4) floats and a
// second kernel merges the chunks.
CBIS_EXPORT int cbis_paged_attention_generic(const void* q, int q_ld, const void* kc, const void* vc,
                                             const int* block_table, int max_blocks, const int* row_seq,
                                             const int* positions, void* out, int out_ld, int n_rows, int n_head,
                                             int n_kv_head, int hd, int ps, float scale, int window, int dtype,
                                             int n_chunks, int chunk_keys, float* partial, void* stream) {
  if (n_rows <= 0) return CBIS_OK;
  if (hd <= 0 || hd > 256 || ps <= 0 || n_head <= 0 || n_kv_head <= 0 || n_head % n_kv_head) return CBIS_ERR_BAD_SIZE;
  if (n_chunks < 1 || (n_chunks > 1 && (chunk_keys <= 0 || !partial || hd % 4 || out_ld % 4 || ((uintptr_t)partial & 15) ||
                                        ((uintptr_t)out & 15))))
    return CBIS_ERR_BAD_SIZE;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == CBIS_F32)
    return launch_generic<float>(q, q_ld, kc, vc, block_table, max_blocks, row_seq, positions, out, out_ld, n_rows,
                                 n_head, n_kv_head, hd, ps, scale, window, n_chunks, chunk_keys, partial, st);
  if (dtype == CBIS_BF16)
    return launch_generic<__nv_bfloat16>(q, q_ld, kc, vc, block_table, max_blocks, row_seq, positions, out, out_ld,
                                         n_rows, n_head, n_kv_head, hd, ps, scale, window, n_chunks, chunk_keys, partial, st);
  return CBIS_ERR_BAD_DTYPE;
}
