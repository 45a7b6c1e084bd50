// Prefill attention over the paged cache in true 32-bit (no tensor cores): the 32-bit path's counterpart of the
// tiled kernels.  The reference gives every (row, head) a warp that walks all keys of the prefix one by one, so a
// prefill re-reads the prefix once per row (kernels/attention.cu:57-98); the general kernel of this package does
// the same, and a 32,767-token prompt in portions of 512 took it 5.5 s at the reference's sizes.  Here a block
// takes 64 consecutive rows of one (segment, head): keys and values go through shared memory once per 64 rows, in
// tiles of 32 keys gathered page by page through the block table.  Four threads share a query row: each computes
// 8 of the tile's 32 scores (fused multiply-adds over the head dim, 16 bytes of Q and K per load), the four
// combine maximum and sum with two shuffles, P goes through shared memory, and each thread accumulates its
// quarter of the head dims of P V.  A thread does this for two rows at once, 32 apart: with one row a thread the
// kernel ran at 85 % of the shared-memory load rate and a quarter of the FFMA rate, and every key and value it
// loads now serves two rows.  Everything is 32-bit arithmetic; the softmax is the online form with running
// maximum and sum per row (kernels/attention.cu:74-95).
//
// A long context with few rows (a 512-token portion behind 30,000 cached tokens, 8 heads) gives too few blocks
// for 148 SMs, each with a thousand key tiles to walk: the keys are then cut into chunks of chunk_keys (absolute
// key indices, so a key's chunk does not depend on how the prompt was cut), a block takes (row tile, head, chunk)
// and leaves its unnormalised sum, maximum and denominator in scratch memory, and a second kernel merges the
// chunks of every row.
#include "attention_merge.cuh"

namespace cbis {

constexpr int F_BM = 64, F_BN = 32, F_THREADS = 128;
constexpr int P_PITCH = F_BN + 4;   // floats per row of P: the four threads of eight rows store to 32 different banks

// grid: (row tiles of the longest segment, heads, segments from seg0 on).  HD4: head dims per thread in P V (hd / 4).
template <int HD>
__global__ void __launch_bounds__(F_THREADS)
paged_prefill_f32_kernel(const float* q, int q_ld, const float* kc, const float* vc, const int* block_table, int max_blocks,
                         const int* cu_rows, const int* seg_start, float* out, int out_ld, int seg0, int n_head, int n_kv_head,
                         int ps, float scale, int window, int n_chunks, int chunk_keys, float* partial, int row0) {
  constexpr int PITCH = HD + 4;     // floats per shared-memory row: 16 bytes of padding spread the rows over the banks
  constexpr int D4 = HD / 4;        // head dims of the output per thread
  extern __shared__ __align__(16) float smem_f[];
  float* sQ = smem_f;                       // [F_BM][PITCH]
  float* sK = sQ + F_BM * PITCH;            // [F_BN][PITCH]
  float* sV = sK + F_BN * PITCH;            // [F_BN][PITCH]
  float* sP = sV + F_BN * PITCH;            // [F_BM][P_PITCH]
  pdl_trigger();
  pdl_wait();
  // late row tiles have the most keys to walk: they are given out first
  const int seg = seg0 + blockIdx.z, h = blockIdx.y;
  const int chunk = blockIdx.x % n_chunks, tile = gridDim.x / n_chunks - 1 - blockIdx.x / n_chunks;
  const int r_begin = cu_rows[seg], n_rows = cu_rows[seg + 1] - r_begin;
  if (tile * F_BM >= n_rows) return;
  const int hk = h / (n_head / n_kv_head);
  const int pos0 = seg_start[seg] + tile * F_BM;
  const int rows_here = min(F_BM, n_rows - tile * F_BM);
  int kend = pos0 + rows_here;
  int kbegin = window > 0 ? max(0, pos0 - window + 1) : 0;
  if (n_chunks > 1) {   // this block's share of the keys; a chunk wholly outside the rows' range leaves nothing
    kbegin = max(kbegin, chunk * chunk_keys);
    kend = min(kend, (chunk + 1) * chunk_keys);
    if (kbegin >= kend) return;
  }
  const int* bt = block_table + (size_t)seg * max_blocks;
  const int tid = threadIdx.x;
  // a thread has TWO rows of the tile, r0 and r0 + 32 (the keys and values it loads from shared memory serve both:
  // the kernel is bound by those loads), and is one of the four threads of each
  const int r0 = tid >> 2, part = tid & 3;
  const int rr2[2] = {r0, r0 + F_BM / 2};
  const int p2[2] = {pos0 + r0, pos0 + r0 + F_BM / 2};   // the rows' positions

  for (int i = tid; i < F_BM * (HD / 4); i += F_THREADS) {
    const int rr = i / (HD / 4), c = (i % (HD / 4)) * 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (rr < rows_here) v = *reinterpret_cast<const float4*>(q + (size_t)(r_begin + tile * F_BM + rr) * q_ld + h * HD + c);
    *reinterpret_cast<float4*>(sQ + rr * PITCH + c) = v;
  }
  float o[2][D4];
#pragma unroll
  for (int w = 0; w < 2; ++w)
#pragma unroll
    for (int d = 0; d < D4; ++d) o[w][d] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  const int kt_first = kbegin / F_BN, kt_last = (kend - 1) / F_BN;
  for (int kt = kt_first; kt <= kt_last; ++kt) {
    const int j0 = kt * F_BN;
    __syncthreads();   // the tile before has been used up (and, the first time, Q is in place)
    for (int i = tid; i < F_BN * (HD / 4); i += F_THREADS) {
      const int rr = i / (HD / 4), c = (i % (HD / 4)) * 4;
      const int j = j0 + rr;
      float4 kv = make_float4(0.f, 0.f, 0.f, 0.f), vv = kv;
      if (j < kend && j >= kbegin) {   // keys before the window may lie in pages already given back
        const size_t src = (((size_t)bt[j / ps] * n_kv_head + hk) * ps + (j % ps)) * HD + c;
        kv = *reinterpret_cast<const float4*>(kc + src);
        vv = *reinterpret_cast<const float4*>(vc + src);
      }
      *reinterpret_cast<float4*>(sK + rr * PITCH + c) = kv;
      *reinterpret_cast<float4*>(sV + rr * PITCH + c) = vv;
    }
    __syncthreads();
    // scores of keys part, part + 4, ... (8 of the 32), for both rows
    float s[2][F_BN / 4];
#pragma unroll
    for (int w = 0; w < 2; ++w)
#pragma unroll
      for (int u = 0; u < F_BN / 4; ++u) s[w][u] = 0.f;
#pragma unroll 2
    for (int c = 0; c < HD; c += 4) {
      const float4 qa = *reinterpret_cast<const float4*>(sQ + rr2[0] * PITCH + c);
      const float4 qb = *reinterpret_cast<const float4*>(sQ + rr2[1] * PITCH + c);
#pragma unroll
      for (int u = 0; u < F_BN / 4; ++u) {
        const float4 kv = *reinterpret_cast<const float4*>(sK + (part + 4 * u) * PITCH + c);
        s[0][u] = fmaf(qa.x, kv.x, s[0][u]);
        s[0][u] = fmaf(qa.y, kv.y, s[0][u]);
        s[0][u] = fmaf(qa.z, kv.z, s[0][u]);
        s[0][u] = fmaf(qa.w, kv.w, s[0][u]);
        s[1][u] = fmaf(qb.x, kv.x, s[1][u]);
        s[1][u] = fmaf(qb.y, kv.y, s[1][u]);
        s[1][u] = fmaf(qb.z, kv.z, s[1][u]);
        s[1][u] = fmaf(qb.w, kv.w, s[1][u]);
      }
    }
    float corr[2];
#pragma unroll
    for (int w = 0; w < 2; ++w) {
      float mx = -INFINITY;
#pragma unroll
      for (int u = 0; u < F_BN / 4; ++u) {
        const int j = j0 + part + 4 * u;
        const bool seen = j <= p2[w] && j < kend && (window == 0 || j >= p2[w] - window + 1);
        s[w][u] = seen ? s[w][u] * scale : -INFINITY;
        mx = fmaxf(mx, s[w][u]);
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m[w], mx);
      const float base = m_new == -INFINITY ? 0.f : m_new;   // a row with no key in range yet
      corr[w] = expf(m[w] - base);
      float psum = 0.f;
#pragma unroll
      for (int u = 0; u < F_BN / 4; ++u) {
        const float e = expf(s[w][u] - base);
        psum += e;
        sP[rr2[w] * P_PITCH + part + 4 * u] = e;
      }
      psum += __shfl_xor_sync(0xffffffffu, psum, 1);
      psum += __shfl_xor_sync(0xffffffffu, psum, 2);
      l[w] = l[w] * corr[w] + psum;
      m[w] = m_new;
#pragma unroll
      for (int d = 0; d < D4; ++d) o[w][d] *= corr[w];
    }
    __syncwarp();   // the four threads of a row are neighbours in one warp: P of both rows is complete
    const float* pa = sP + rr2[0] * P_PITCH;
    const float* pb = sP + rr2[1] * P_PITCH;
#pragma unroll 4
    for (int j = 0; j < F_BN; ++j) {
      const float p0 = pa[j], p1 = pb[j];
      const float* vrow = sV + j * PITCH + part * D4;
#pragma unroll
      for (int d = 0; d < D4; d += 4) {
        const float4 vv = *reinterpret_cast<const float4*>(vrow + d);
        o[0][d] = fmaf(p0, vv.x, o[0][d]);
        o[0][d + 1] = fmaf(p0, vv.y, o[0][d + 1]);
        o[0][d + 2] = fmaf(p0, vv.z, o[0][d + 2]);
        o[0][d + 3] = fmaf(p0, vv.w, o[0][d + 3]);
        o[1][d] = fmaf(p1, vv.x, o[1][d]);
        o[1][d + 1] = fmaf(p1, vv.y, o[1][d + 1]);
        o[1][d + 2] = fmaf(p1, vv.z, o[1][d + 2]);
        o[1][d + 3] = fmaf(p1, vv.w, o[1][d + 3]);
      }
    }
  }
#pragma unroll
  for (int w = 0; w < 2; ++w) {
    const int r = rr2[w];
    if (r >= rows_here) continue;
    if (n_chunks > 1) {
      float* dst = partial + (((size_t)(r_begin + tile * F_BM + r - row0) * n_head + h) * n_chunks + chunk) * (HD + 4);
#pragma unroll
      for (int d = 0; d < D4; d += 4)
        *reinterpret_cast<float4*>(dst + part * D4 + d) = make_float4(o[w][d], o[w][d + 1], o[w][d + 2], o[w][d + 3]);
      if (part == 0) *reinterpret_cast<float2*>(dst + HD) = make_float2(m[w], l[w]);
      continue;
    }
    const float inv = 1.f / l[w];
    float* dst = out + (size_t)(r_begin + tile * F_BM + r) * out_ld + h * HD + part * D4;
#pragma unroll
    for (int d = 0; d < D4; d += 4)
      *reinterpret_cast<float4*>(dst + d) = make_float4(o[w][d] * inv, o[w][d + 1] * inv, o[w][d + 2] * inv, o[w][d + 3] * inv);
  }
}

}  // namespace cbis

using namespace cbis;

// Attention of the segments seg0 .. seg0+n_seg-1 of a step (each a run of rows, cu_rows) over their pages, in
// 32-bit.  Takes head sizes 16, 32, ... 128 (any page size); refuses anything else.  With chunk_keys > 0 (a
// multiple of 32) the keys are cut into n_chunks chunks of that many: partial then holds
// n_rows * n_head * n_chunks * (hd + 4) floats for the rows row0 .. row0+n_rows-1 (those of the segments), positions
// the position of every row of the step, and a second kernel merges the chunks of these rows.
CBIS_EXPORT int cbis_paged_prefill_f32(const float* q, int q_ld, const float* kc, const float* vc, const int* block_table,
                                       int max_blocks, const int* cu_rows, const int* seg_start, float* out, int out_ld,
                                       int seg0, int n_seg, int max_seg_rows, int n_head, int n_kv_head, int hd, int ps,
                                       float scale, int window, int n_chunks, int chunk_keys, float* partial,
                                       const int* positions, int row0, int n_rows, void* stream) {
  if (n_seg <= 0 || max_seg_rows <= 0) return CBIS_OK;
  if (n_chunks < 1 || (n_chunks > 1 && (chunk_keys <= 0 || chunk_keys % F_BN || !partial || !positions || n_rows <= 0 ||
                                        ((uintptr_t)partial & 15))))
    return CBIS_ERR_BAD_SIZE;
  if (hd < 16 || hd > 128 || hd % 16 || ps <= 0 || n_head <= 0 || n_kv_head <= 0 || n_head % n_kv_head) return CBIS_ERR_BAD_SIZE;
  if (q_ld % 4 || out_ld % 4 || ((uintptr_t)q & 15) || ((uintptr_t)kc & 15) || ((uintptr_t)vc & 15) || ((uintptr_t)out & 15))
    return CBIS_ERR_ALIGNMENT;
  dim3 grid(((max_seg_rows + F_BM - 1) / F_BM) * n_chunks, n_head, n_seg);
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaErrorInvalidValue;
#define CBIS_PF32(HD_)                                                                                               \
  if (hd == HD_) {                                                                                                   \
    auto kern = paged_prefill_f32_kernel<HD_>;                                                                       \
    const size_t smem = ((size_t)(F_BM + 2 * F_BN) * (HD_ + 4) + (size_t)F_BM * P_PITCH) * sizeof(float);            \
    if (smem > 48 * 1024) {                                                                                          \
      e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                        \
      if (e != cudaSuccess) return (int)e;                                                                           \
    }                                                                                                                \
    e = launch_pdl(kern, grid, dim3(F_THREADS), smem, st, q, q_ld, kc, vc, block_table, max_blocks, cu_rows, seg_start, out, \
                   out_ld, seg0, n_head, n_kv_head, ps, scale, window, n_chunks, chunk_keys, partial, row0);         \
  }
  CBIS_PF32(16) CBIS_PF32(32) CBIS_PF32(48) CBIS_PF32(64) CBIS_PF32(80) CBIS_PF32(96) CBIS_PF32(112) CBIS_PF32(128)
#undef CBIS_PF32
  if (e == cudaSuccess && n_chunks > 1)
    e = launch_pdl(prefill_merge_kernel<float, false>, dim3(n_rows), dim3(128), 0, st, (const float*)partial, positions, (const int*)nullptr, out, out_ld, row0,
                   n_head, hd, window, n_chunks, chunk_keys);
  return (int)e;
}
