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
  dim3 grid((N + 63) / 64, (M + 15) / 16);
  return (int)launch_pdl(linear_f32_kernel<16, 64, 16, 1, 4>, grid, dim3(256), 0, st, A, W, bias, C, M, N, K, w_is_nk,
                         act, lda, ldc);
}
