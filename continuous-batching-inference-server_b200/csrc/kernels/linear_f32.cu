// 32-bit matrix product on the FP32 units (FFMA only: no TF32, no tensor cores), with the
// bias and the activation applied to the 32-bit sum before it is stored.
//   C[M,N] = act(A[M,K] * W + bias)     W is [K,N] (GPT-2 Conv1D layout) or [N,K] (a token table as head)
// The reference calls cublasSgemm and adds the bias in a second kernel (kernels/linear.cu:15-34).
#include "common.cuh"

namespace cbis {

template <int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
linear_f32_kernel(const float* A, const float* __restrict__ W, const float* __restrict__ bias,
                  float* __restrict__ C, int M, int N, int K, int w_is_nk, int act, int lda, int ldc) {
  constexpr int THREADS = (BM / TM) * (BN / TN);
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  pdl_trigger();
  pdl_wait();
  const int tid = threadIdx.x;
  const int tx = tid % (BN / TN), ty = tid / (BN / TN);
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    // A tile: BM x BK, consecutive threads along k (rows of A are contiguous in k)
    for (int i = tid; i < BM * BK; i += THREADS) {
      const int mm = i / BK, kk = i % BK;
      const int m = m0 + mm, k = k0 + kk;
      As[kk][mm] = (m < M && k < K) ? A[(size_t)m * lda + k] : 0.f;
    }
    if (w_is_nk) {
      for (int i = tid; i < BN * BK; i += THREADS) {
        const int nn = i / BK, kk = i % BK;
        const int n = n0 + nn, k = k0 + kk;
        Bs[kk][nn] = (n < N && k < K) ? W[(size_t)n * K + k] : 0.f;
      }
    } else {
      for (int i = tid; i < BN * BK; i += THREADS) {
        const int kk = i / BN, nn = i % BN;
        const int n = n0 + nn, k = k0 + kk;
        Bs[kk][nn] = (n < N && k < K) ? W[(size_t)k * N + n] : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Bs[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[n];
      C[(size_t)m * ldc + n] = activate(v, act);
    }
  }
}

// More than 16 rows with W stored [N, K] (both operands contiguous along k, 16-byte aligned): tiles of BM x BN
// outputs, k in pieces of 32 that arrive by 16-byte cp.async in two buffers (the next piece is on its way while
// this one is multiplied), operands kept [row][k] in shared memory so that the copy is straight and a thread reads
// four k of a row at once.  A thread owns the outputs (ty + 16 i, tx + 16 j) and walks k from left to right with
// one fused multiply-add per element: the order of the kernels above and below, hence the same bits.  The tile
// shrinks (64x64, 32x64, 32x32) until the grid fills the SMs: a 512 x 256 x 1024 product had 8 blocks of the
// 128 x 128 kernel above and took 190 us.
__device__ __forceinline__ void cp_async16_f32(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;   // 0 bytes read: the 16 bytes in shared memory are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}

template <int BM, int BN>
__global__ void __launch_bounds__(256)
linear_f32_nk_kernel(const float* A, const float* __restrict__ W, const float* __restrict__ bias, float* __restrict__ C,
                     int M, int N, int K, int act, int lda, int ldc) {
  constexpr int BK = 32, PITCH = BK + 4, TM = BM / 16, TN = BN / 16;
  extern __shared__ __align__(16) float nk_smem[];
  float (*As)[BM][PITCH] = reinterpret_cast<float (*)[BM][PITCH]>(nk_smem);                      // [2][BM][PITCH]
  float (*Ws)[BN][PITCH] = reinterpret_cast<float (*)[BN][PITCH]>(nk_smem + 2 * BM * PITCH);     // [2][BN][PITCH]
  pdl_trigger();
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  auto load_w = [&](int k0, int stage) {
    for (int i = tid; i < BN * (BK / 4); i += 256) {
      const int r = i / (BK / 4), c = (i % (BK / 4)) * 4;
      const bool valid = n0 + r < N && k0 + c < K;
      cp_async16_f32(&Ws[stage][r][c], valid ? W + (size_t)(n0 + r) * K + k0 + c : W, valid);
    }
  };
  auto load_a = [&](int k0, int stage) {
    for (int i = tid; i < BM * (BK / 4); i += 256) {
      const int r = i / (BK / 4), c = (i % (BK / 4)) * 4;
      const bool valid = m0 + r < M && k0 + c < K;
      cp_async16_f32(&As[stage][r][c], valid ? A + (size_t)(m0 + r) * lda + k0 + c : A, valid);
    }
  };
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  load_w(0, 0);   // the weights do not come from the kernel before
  pdl_wait();
  load_a(0, 0);
  asm volatile("cp.async.commit_group;\n" ::);
  const int n_kt = (K + BK - 1) / BK;
  for (int kt = 0; kt < n_kt; ++kt) {
    const int stage = kt & 1;
    if (kt + 1 < n_kt) {
      load_w((kt + 1) * BK, stage ^ 1);
      load_a((kt + 1) * BK, stage ^ 1);
      asm volatile("cp.async.commit_group;\n" ::);
      asm volatile("cp.async.wait_group 1;\n" ::);
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::);
    }
    __syncthreads();
    const int kc = min(BK, K - kt * BK);   // a multiple of 4; the sum stops at K (0 * 0 could still flip the sign of a zero)
#pragma unroll 2
    for (int kk = 0; kk < kc; kk += 4) {
      float4 a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = *reinterpret_cast<const float4*>(&As[stage][ty + 16 * i][kk]);
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = *reinterpret_cast<const float4*>(&Ws[stage][tx + 16 * j][kk]);
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
          float v = acc[i][j];
          v = fmaf(a[i].x, b[j].x, v);
          v = fmaf(a[i].y, b[j].y, v);
          v = fmaf(a[i].z, b[j].z, v);
          v = fmaf(a[i].w, b[j].w, v);
          acc[i][j] = v;
        }
    }
    __syncthreads();   // this buffer is free for the piece after the next
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty + 16 * i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx + 16 * j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[n];
      C[(size_t)m * ldc + n] = activate(v, act);
    }
  }
}

// Up to 16 rows (decoding) with W stored [N, K]: the tiled kernel above would run N / 64 blocks that walk K in
// steps of 16 with two barriers each: 62 us for a 16 x 768 x 256 product.  Here a block takes 16 output columns
// and a thread owns ONE output (lane m of a half-warp: row m; the half-warp: one column).  K comes in pieces of
// 256: the block copies the piece of A (16 rows) and of W (16 rows) into shared memory with coalesced 16-byte
// loads, all in flight at once, and every thread then walks its piece from left to right with one fused
// multiply-add per element: the same order as the tiled kernel, hence the same bits, so that a token decoded
// alone and the same token inside a prompt portion still agree exactly.
constexpr int FR_KC = 256;
__global__ void __launch_bounds__(256)
linear_f32_few_rows_kernel(const float* A, const float* __restrict__ W, const float* __restrict__ bias, float* __restrict__ C,
                           int M, int N, int K, int act, int lda, int ldc) {
  __shared__ __align__(16) float As[16][FR_KC + 4];
  __shared__ __align__(16) float Ws[16][FR_KC + 4];
  pdl_trigger();
  const int tid = threadIdx.x;
  const int m = tid & 15, c = tid >> 4, n0 = blockIdx.x * 16, n = n0 + c;
  const bool vec = (K & 3) == 0 && (lda & 3) == 0 && (((uintptr_t)A | (uintptr_t)W) & 15) == 0;
  pdl_wait();  // A comes from the kernel before
  float acc = 0.f;
  for (int k0 = 0; k0 < K; k0 += FR_KC) {
    const int kc = min(FR_KC, K - k0);
    if (vec) {
      for (int i = tid; i < 16 * (FR_KC / 4); i += 256) {
        const int r = i / (FR_KC / 4), k = (i % (FR_KC / 4)) * 4;
        float4 av = make_float4(0.f, 0.f, 0.f, 0.f), wv = av;
        if (k < kc) {
          if (r < M) av = *reinterpret_cast<const float4*>(A + (size_t)r * lda + k0 + k);
          if (n0 + r < N) wv = __ldg(reinterpret_cast<const float4*>(W + (size_t)(n0 + r) * K + k0 + k));
        }
        *reinterpret_cast<float4*>(&As[r][k]) = av;
        *reinterpret_cast<float4*>(&Ws[r][k]) = wv;
      }
    } else {
      for (int i = tid; i < 16 * FR_KC; i += 256) {
        const int r = i / FR_KC, k = i % FR_KC;
        As[r][k] = (k < kc && r < M) ? A[(size_t)r * lda + k0 + k] : 0.f;
        Ws[r][k] = (k < kc && n0 + r < N) ? __ldg(W + (size_t)(n0 + r) * K + k0 + k) : 0.f;
      }
    }
    __syncthreads();
    // (a piece shorter than 256 ends in zeros of A and W: adding 0 * 0 changes no bit of the sum... except the sign of
    // a zero sum, so the loop stops at the piece's end)
    int k = 0;
    for (; k + 4 <= kc; k += 4) {
      const float4 av = *reinterpret_cast<const float4*>(&As[m][k]), wv = *reinterpret_cast<const float4*>(&Ws[c][k]);
      acc = fmaf(av.x, wv.x, acc);
      acc = fmaf(av.y, wv.y, acc);
      acc = fmaf(av.z, wv.z, acc);
      acc = fmaf(av.w, wv.w, acc);
    }
    for (; k < kc; ++k) acc = fmaf(As[m][k], Ws[c][k], acc);
    __syncthreads();
  }
  if (m < M && n < N) {
    if (bias) acc += bias[n];
    C[(size_t)m * ldc + n] = activate(acc, act);
  }
}

}  // namespace cbis

using namespace cbis;

// lda / ldc: row strides of A and C in elements (>= K, >= N).
// variant: 0 the launcher's choice; 1 never the cp.async kernel (the older tiled kernels: all give the same bits).
CBIS_EXPORT int cbis_linear_f32(const float* A, const float* W, const float* bias, float* C, int M, int N, int K,
                                int w_is_nk, int act, int lda, int ldc, int variant, void* stream) {
  if (M <= 0 || N <= 0) return CBIS_OK;
  if (K <= 0 || lda < K || ldc < N) return CBIS_ERR_BAD_SIZE;
  cudaStream_t st = (cudaStream_t)stream;
  if (variant != 1 && w_is_nk && M > 16 && K % 4 == 0 && lda % 4 == 0 && !(((uintptr_t)A | (uintptr_t)W) & 15)) {
    // (a 128 x 128 tile, 8 x 8 outputs a thread, was measured too: 198 registers, one block per SM, no faster than 64 x 64)
    const long long b64 = (long long)((M + 63) / 64) * ((N + 63) / 64),
                    b32 = (long long)((M + 31) / 32) * ((N + 63) / 64);
#define CBIS_NK(BM_, BN_)                                                                                              \
  {                                                                                                                    \
    auto kern = linear_f32_nk_kernel<BM_, BN_>;                                                                        \
    const size_t smem = (size_t)2 * (BM_ + BN_) * 36 * sizeof(float);                                                  \
    if (smem > 48 * 1024) {                                                                                            \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);              \
      if (e != cudaSuccess) return (int)e;                                                                             \
    }                                                                                                                  \
    return (int)launch_pdl(kern, dim3((N + BN_ - 1) / BN_, (M + BM_ - 1) / BM_), dim3(256), smem, st, A, W, bias, C, M, N, K, \
                           act, lda, ldc);                                                                             \
  }
    if (b64 >= 2 * 148) CBIS_NK(64, 64)
    if (b32 >= 148) CBIS_NK(32, 64)
    CBIS_NK(32, 32)
#undef CBIS_NK
  }
  if (M > 256) {
    dim3 grid((N + 127) / 128, (M + 127) / 128);
    return (int)launch_pdl(linear_f32_kernel<128, 128, 8, 8, 8>, grid, dim3(256), 0, st, A, W, bias, C, M, N, K, w_is_nk,
                           act, lda, ldc);
  }
  if (M > 16) {
    dim3 grid((N + 63) / 64, (M + 63) / 64);
    return (int)launch_pdl(linear_f32_kernel<64, 64, 16, 4, 4>, grid, dim3(256), 0, st, A, W, bias, C, M, N, K, w_is_nk,
                           act, lda, ldc);
  }
  if (w_is_nk) {   // decoding: one thread per output, 16 outputs (rows) x 2 columns per warp, 8 warps per block
    return (int)launch_pdl(linear_f32_few_rows_kernel, dim3((N + 15) / 16), dim3(256), 0, st, A, W, bias, C, M, N, K, act, lda,
                           ldc);
  }
  dim3 grid((N + 63) / 64, (M + 15) / 16);
  return (int)launch_pdl(linear_f32_kernel<16, 64, 16, 1, 4>, grid, dim3(256), 0, st, A, W, bias, C, M, N, K, w_is_nk,
                         act, lda, ldc);
}
