// Prefill attention over the paged cache for bfloat16: the rows of a portion of a prompt attend to
// all keys of their request up to their own position (the earlier portions in the cache and this
// portion, which the cache-write kernel has stored before).
//
// The reference gives every (row, head) a warp that walks all keys of the prefix one by one, so a
// prefill re-reads the prefix once per row (kernels/attention.cu:57-98).  Here a block takes 64
// consecutive rows of one (segment, head): the keys and values go through shared memory once per
// 64 rows, in tiles of 64 keys gathered page by page through the block table (cp.async, two
// tiles in flight); Q*K^T and P*V run on the tensor cores (mma.sync m16n8k16, bf16 in, 32-bit
// accumulate; ldmatrix from rows padded by 16 bytes), and the softmax is the online form with
// running max and sum per row in 32-bit, P rounded to bf16 only as the operand of P*V.
#include "attention_merge.cuh"
#include <math.h>

namespace cbis {

constexpr int PF_BM = 64;   // query rows per block (4 warps x 16)
constexpr int PF_BN = 64;   // keys per tile
constexpr int PF_WARPS = 4;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int n = valid ? 16 : 0;  // 0 source bytes: the 16 destination bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t* r, const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t* r, const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t* r, const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_pf(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// grid: (row tiles of the longest segment, heads, segments from seg0 on).  cu_rows/seg_start are the
// step's segment tables: rows cu_rows[s]..cu_rows[s+1] of q/out belong to segment s and start at
// position seg_start[s].
template <int HD>
__global__ void __launch_bounds__(PF_WARPS * 32, 3)
paged_prefill_bf16_kernel(const __nv_bfloat16* q, int q_ld, const __nv_bfloat16* kc, const __nv_bfloat16* vc,
                          const int* block_table, int max_blocks, const int* cu_rows, const int* seg_start,
                          __nv_bfloat16* out, int out_ld, int seg0, int n_head, int n_kv_head, int ps_shift,
                          float scale_log2e, int window, int n_chunks, int chunk_keys, float* partial, int row0) {
  constexpr int PITCH = HD + 8;  // elements per shared-memory row: 16 bytes of padding keep ldmatrix conflict-free
  constexpr int KS = HD / 16;    // k-steps of Q*K^T
  constexpr int DT = HD / 8;     // 8-wide column tiles of the output
  constexpr int CHUNKS = HD / 8; // 16-byte pieces per key row
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* sK = reinterpret_cast<__nv_bfloat16*>(smem_raw);            // [2][PF_BN][PITCH]
  __nv_bfloat16* sV = sK + 2 * PF_BN * PITCH;                                // [2][PF_BN][PITCH]
  pdl_trigger();
  pdl_wait();
  // late row tiles have the most keys to walk: they are given out first, the short ones fill the end
  const int seg = seg0 + blockIdx.z, h = blockIdx.y;
  const int chunk = blockIdx.x % n_chunks, tile = gridDim.x / n_chunks - 1 - blockIdx.x / n_chunks;
  const int r_begin = cu_rows[seg], n_rows = cu_rows[seg + 1] - r_begin;
  if (tile * PF_BM >= n_rows) return;
  const int hk = h / (n_head / n_kv_head);
  const int ps = 1 << ps_shift;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int pos0 = seg_start[seg] + tile * PF_BM;           // position of the tile's first row
  const int rows_here = min(PF_BM, n_rows - tile * PF_BM);
  int kend = pos0 + rows_here;                              // keys 0 .. kend-1 can matter to this tile
  int kbegin = window > 0 ? max(0, pos0 - window + 1) : 0;
  if (n_chunks > 1) {   // this block's share of the keys (chunks by absolute index, whole key tiles)
    kbegin = max(kbegin, chunk * chunk_keys);
    kend = min(kend, (chunk + 1) * chunk_keys);
    if (kbegin >= kend) return;
  }
  const int* bt = block_table + (size_t)seg * max_blocks;

  // this thread's two rows: g and g + 8 of the warp's 16
  const int lr0 = warp * 16 + g, lr1 = lr0 + 8;
  const int p0 = pos0 + lr0, p1 = pos0 + lr1;
  uint32_t qf[KS][4];
  {
    const __nv_bfloat16* q0 = q + (size_t)(r_begin + tile * PF_BM + lr0) * q_ld + h * HD;
    const __nv_bfloat16* q1 = q + (size_t)(r_begin + tile * PF_BM + lr1) * q_ld + h * HD;
    const bool v0 = lr0 < rows_here, v1 = lr1 < rows_here;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      qf[ks][0] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 2 * t) : 0u;
      qf[ks][1] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 2 * t) : 0u;
      qf[ks][2] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 8 + 2 * t) : 0u;
      qf[ks][3] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 8 + 2 * t) : 0u;
    }
  }
  float o[DT][4];
#pragma unroll
  for (int d = 0; d < DT; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  const int kt_first = kbegin / PF_BN, kt_last = (kend - 1) / PF_BN;
  const int live_from = (kbegin >> ps_shift) << ps_shift;
  auto load_tile = [&](int kt, int stage) {
    __nv_bfloat16* dk = sK + (size_t)stage * PF_BN * PITCH;
    __nv_bfloat16* dv = sV + (size_t)stage * PF_BN * PITCH;
    for (int idx = threadIdx.x; idx < PF_BN * CHUNKS; idx += PF_WARPS * 32) {
      const int r = idx / CHUNKS, c = idx % CHUNKS;
      const int j = kt * PF_BN + r;
      const bool valid = j < kend && j >= live_from;   // pages behind the window may have been given back
      size_t src = 0;
      if (valid) {
        const int page = bt[j >> ps_shift];
        src = (((size_t)page * n_kv_head + hk) * ps + (j & (ps - 1))) * HD + c * 8;
      }
      cp_async16(dk + r * PITCH + c * 8, kc + src, valid);
      cp_async16(dv + r * PITCH + c * 8, vc + src, valid);
    }
    cp_async_commit();
  };

  load_tile(kt_first, 0);
  for (int kt = kt_first; kt <= kt_last; ++kt) {
    const int stage = (kt - kt_first) & 1;
    if (kt < kt_last) {
      load_tile(kt + 1, stage ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const __nv_bfloat16* tk = sK + (size_t)stage * PF_BN * PITCH;
    const __nv_bfloat16* tv = sV + (size_t)stage * PF_BN * PITCH;
    // S = Q K^T for this warp's 16 rows x 64 keys
    float s[PF_BN / 8][4];
#pragma unroll
    for (int nt = 0; nt < PF_BN / 8; ++nt) {
      s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks + 1 < KS; ks += 2) {
        uint32_t b[4];
        ldmatrix_x4(b, tk + (size_t)(nt * 8 + (lane & 7)) * PITCH + ks * 16 + (lane >> 3) * 8);
        mma_pf(s[nt], qf[ks], b[0], b[1]);
        mma_pf(s[nt], qf[ks + 1], b[2], b[3]);
      }
      if constexpr (KS & 1) {   // a head size that is an odd multiple of 16: the last 16 dims on their own
        uint32_t b[2];
        ldmatrix_x2(b, tk + (size_t)(nt * 8 + (lane & 7)) * PITCH + (KS - 1) * 16 + ((lane >> 3) & 1) * 8);
        mma_pf(s[nt], qf[KS - 1], b[0], b[1]);
      }
    }
    // scale (into the base-2 domain), mask, running max
    const int j0 = kt * PF_BN;
    const bool edge = (j0 + PF_BN - 1 > pos0) || (window > 0 && j0 < pos0 + PF_BM - window + 1);
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < PF_BN / 8; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int j = j0 + nt * 8 + 2 * t + e;
        float a = s[nt][e] * scale_log2e, b2 = s[nt][2 + e] * scale_log2e;
        if (edge) {
          if (j > p0 || (window > 0 && j < p0 - window + 1)) a = -INFINITY;
          if (j > p1 || (window > 0 && j < p1 - window + 1)) b2 = -INFINITY;
        }
        s[nt][e] = a;
        s[nt][2 + e] = b2;
        mx0 = fmaxf(mx0, a);
        mx1 = fmaxf(mx1, b2);
      }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float base0 = mn0 == -INFINITY ? 0.f : mn0, base1 = mn1 == -INFINITY ? 0.f : mn1;  // rows with no key yet
    const float c0 = exp2f(m0 - base0), c1 = exp2f(m1 - base1);
    m0 = mn0;
    m1 = mn1;
    float ps0 = 0.f, ps1 = 0.f;
    uint32_t pf[PF_BN / 16][4];
#pragma unroll
    for (int nt = 0; nt < PF_BN / 8; ++nt) {
      const float a0 = exp2f(s[nt][0] - base0), a1 = exp2f(s[nt][1] - base0);
      const float b0 = exp2f(s[nt][2] - base1), b1 = exp2f(s[nt][3] - base1);
      ps0 += a0 + a1;
      ps1 += b0 + b1;
      pf[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16(a0, a1);
      pf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(b0, b1);
    }
    l0 = l0 * c0 + ps0;
    l1 = l1 * c1 + ps1;
#pragma unroll
    for (int d = 0; d < DT; ++d) {
      o[d][0] *= c0;
      o[d][1] *= c0;
      o[d][2] *= c1;
      o[d][3] *= c1;
    }
    // O += P V
#pragma unroll
    for (int kk = 0; kk < PF_BN / 16; ++kk)
#pragma unroll
      for (int d = 0; d < DT; d += 2) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, tv + (size_t)(kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * PITCH + (d + (lane >> 4)) * 8);
        mma_pf(o[d], pf[kk], b[0], b[1]);
        mma_pf(o[d + 1], pf[kk], b[2], b[3]);
      }
    __syncthreads();  // everyone is done with this stage before the next load overwrites it
  }
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  if (n_chunks > 1) {   // unnormalised sums, maximum (base-2 domain) and denominator for the merge kernel
    float* d0 = partial + (((size_t)(r_begin + tile * PF_BM + lr0 - row0) * n_head + h) * n_chunks + chunk) * (HD + 4);
    float* d1 = partial + (((size_t)(r_begin + tile * PF_BM + lr1 - row0) * n_head + h) * n_chunks + chunk) * (HD + 4);
#pragma unroll
    for (int d = 0; d < DT; ++d) {
      if (lr0 < rows_here) *reinterpret_cast<float2*>(d0 + d * 8 + 2 * t) = make_float2(o[d][0], o[d][1]);
      if (lr1 < rows_here) *reinterpret_cast<float2*>(d1 + d * 8 + 2 * t) = make_float2(o[d][2], o[d][3]);
    }
    if (t == 0 && lr0 < rows_here) *reinterpret_cast<float2*>(d0 + HD) = make_float2(m0, l0);
    if (t == 0 && lr1 < rows_here) *reinterpret_cast<float2*>(d1 + HD) = make_float2(m1, l1);
    return;
  }
  const float i0 = 1.f / l0, i1 = 1.f / l1;
  __nv_bfloat16* o0 = out + (size_t)(r_begin + tile * PF_BM + lr0) * out_ld + h * HD;
  __nv_bfloat16* o1 = out + (size_t)(r_begin + tile * PF_BM + lr1) * out_ld + h * HD;
#pragma unroll
  for (int d = 0; d < DT; ++d) {
    if (lr0 < rows_here) *reinterpret_cast<uint32_t*>(o0 + d * 8 + 2 * t) = pack_bf16(o[d][0] * i0, o[d][1] * i0);
    if (lr1 < rows_here) *reinterpret_cast<uint32_t*>(o1 + d * 8 + 2 * t) = pack_bf16(o[d][2] * i1, o[d][3] * i1);
  }
}

}  // namespace cbis

using namespace cbis;

// Attention of the segments seg0 .. seg0+n_seg-1 of a step (each a run of rows, cu_rows) over their pages.
// Takes head sizes 16, 32, ... 128 and page sizes that are powers of two; refuses anything else.  With
// n_chunks > 1 the keys are cut into chunks of chunk_keys (a multiple of 64) over more blocks: partial then holds
// n_rows * n_head * n_chunks * (hd + 4) floats for the rows row0 .. row0+n_rows-1 (those of the segments),
// positions the position of every row of the step, and a second kernel merges the chunks of these rows.
CBIS_EXPORT int cbis_paged_prefill_bf16(const void* q, int q_ld, const void* kc, const void* vc,
                                        const int* block_table, int max_blocks, const int* cu_rows,
                                        const int* seg_start, void* out, int out_ld, int seg0, int n_seg,
                                        int max_seg_rows, int n_head, int n_kv_head, int hd, int ps, float scale,
                                        int window, int n_chunks, int chunk_keys, float* partial, const int* positions,
                                        int row0, int n_rows, void* stream) {
  if (n_seg <= 0 || max_seg_rows <= 0) return CBIS_OK;
  if (n_chunks < 1 || (n_chunks > 1 && (chunk_keys <= 0 || chunk_keys % PF_BN || !partial || !positions || n_rows <= 0 ||
                                        ((uintptr_t)partial & 15) || out_ld % 4 || ((uintptr_t)out & 7))))
    return CBIS_ERR_BAD_SIZE;
  if (hd < 16 || hd > 128 || hd % 16 || ps <= 0 || (ps & (ps - 1)) || n_head <= 0 || n_kv_head <= 0 || n_head % n_kv_head)
    return CBIS_ERR_BAD_SIZE;
  if (q_ld % 8 || out_ld % 2 || ((uintptr_t)q & 15) || ((uintptr_t)kc & 15) || ((uintptr_t)vc & 15) || ((uintptr_t)out & 3))
    return CBIS_ERR_ALIGNMENT;
  int ps_shift = 0;
  while ((1 << ps_shift) < ps) ++ps_shift;
  dim3 grid(((max_seg_rows + PF_BM - 1) / PF_BM) * n_chunks, n_head, n_seg);
  const float scale_log2e = scale * 1.4426950408889634f;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e;
  e = cudaErrorInvalidValue;
#define CBIS_PF(HD_)                                                                                                  \
  if (hd == HD_) {                                                                                                    \
    auto kern = paged_prefill_bf16_kernel<HD_>;                                                                       \
    const size_t smem = (size_t)4 * PF_BN * (HD_ + 8) * sizeof(__nv_bfloat16);                                        \
    if (smem > 48 * 1024) {                                                                                           \
      e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                         \
      if (e != cudaSuccess) return (int)e;                                                                            \
    }                                                                                                                 \
    e = launch_pdl(kern, grid, dim3(PF_WARPS * 32), smem, st, (const __nv_bfloat16*)q, q_ld, (const __nv_bfloat16*)kc, \
                   (const __nv_bfloat16*)vc, block_table, max_blocks, cu_rows, seg_start, (__nv_bfloat16*)out, out_ld, seg0, \
                   n_head, n_kv_head, ps_shift, scale_log2e, window, n_chunks, chunk_keys, partial, row0);            \
  }
  CBIS_PF(16) CBIS_PF(32) CBIS_PF(48) CBIS_PF(64) CBIS_PF(80) CBIS_PF(96) CBIS_PF(112) CBIS_PF(128)
#undef CBIS_PF
  if (e == cudaSuccess && n_chunks > 1)
    e = launch_pdl(prefill_merge_kernel<__nv_bfloat16, true>, dim3(n_rows), dim3(128), 0, st, (const float*)partial, positions,
                   (const int*)nullptr, (__nv_bfloat16*)out, out_ld, row0, n_head, hd, window, n_chunks, chunk_keys);
  return (int)e;
}
