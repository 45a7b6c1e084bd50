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
CBIS_EXPORT int cbis_linear_f32(const float* A, const float* W, const float* bias, float* C, int M, int N, int K,
                                int w_is_nk, int act, int lda, int ldc, void* stream) {
  if (M <= 0 || N <= 0) return CBIS_OK;
  if (K <= 0 || lda < K || ldc < N) return CBIS_ERR_BAD_SIZE;
  cudaStream_t st = (cudaStream_t)stream;
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
