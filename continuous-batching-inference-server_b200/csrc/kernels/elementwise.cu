// Embedding + learned positions, residual-add + LayerNorm (with row selection), bias + activation.
// All arithmetic in 32-bit; the residual stream is 32-bit in both precisions.
#include "common.cuh"

namespace cbis {

// x[r,:] = wte[tok[r],:] + wpe[pos[r],:]   (reference: kernels/elementwise.cu:7-17)
// A token or position outside its table sets *err (1 = token, 2 = position) and gives a zero row.
template <typename TT>
__global__ void embed_pos_add_kernel(const int* tokens, const int* positions,
                                     const TT* __restrict__ wte, const TT* __restrict__ wpe,
                                     float* __restrict__ out, int d, int vocab, int n_pos, int* err) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const int tok = tokens[r];
  const int pos = positions[r];
  const bool tok_ok = tok >= 0 && tok < vocab;
  const bool pos_ok = wpe == nullptr || (pos >= 0 && pos < n_pos);
  if (threadIdx.x == 0) {
    if (!tok_ok) atomicExch(err, 1);
    else if (!pos_ok) atomicExch(err, 2);
  }
  const TT* trow = wte + (size_t)(tok_ok ? tok : 0) * d;
  const TT* prow = wpe ? wpe + (size_t)(pos_ok ? pos : 0) * d : nullptr;
  float* orow = out + (size_t)r * d;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float v = 0.f;
    if (tok_ok && pos_ok) {
      v = to_f32(trow[c]);
      if (prow) v += to_f32(prow[c]);
    }
    orow[c] = v;
  }
}

// One block per output row r; src row s = rows ? rows[r] : r.
//   v = x[s,:] (+ delta[s,:]) (+ delta_bias[:])           32-bit
//   if rows == nullptr and (delta or bias): x[s,:] = v      the residual stream moves on
//   out[r,:] = (v - mean) * rsqrt(var + eps) * gamma + beta
// var is the centred, biased variance (the reference uses E[x^2]-mean^2, kernels/elementwise.cu:50).
// The row is staged in shared memory (d floats), so x is read once.
template <typename TD, typename TO>
__global__ void add_layernorm_kernel(float* __restrict__ x, const TD* delta,
                                     const float* __restrict__ delta_bias, const float* __restrict__ gamma,
                                     const float* __restrict__ beta, float eps, TO* __restrict__ out,
                                     const int* rows, int d) {
  extern __shared__ float smem[];
  float* row = smem;          // d floats
  float* red = smem + d;      // 33 floats
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const int s = rows ? rows[r] : r;
  float* xrow = x + (size_t)s * d;
  const TD* drow = delta ? delta + (size_t)s * d : nullptr;
  float sum = 0.f;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float v = xrow[c];
    if (drow) v += to_f32(drow[c]);
    if (delta_bias) v += delta_bias[c];
    row[c] = v;
    sum += v;
  }
  const float mean = block_sum(sum, red) / (float)d;
  float sq = 0.f;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    const float t = row[c] - mean;
    sq += t * t;
  }
  const float var = block_sum(sq, red) / (float)d;
  const float inv = rsqrtf(var + eps);
  const bool write_x = rows == nullptr && (drow != nullptr || delta_bias != nullptr);
  TO* orow = out + (size_t)r * d;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    const float v = row[c];
    if (write_x) xrow[c] = v;
    from_f32(orow[c], (v - mean) * inv * gamma[c] + beta[c]);
  }
}

// x[m,n] = act(x[m,n] + bias[n]) in place (reference: add_bias_rowmajor kernels/linear.cu:6-12 + gelu_kernel).
template <typename TT>
__global__ void bias_act_kernel(TT* __restrict__ x, const float* __restrict__ bias, int act, size_t total, int n) {
  pdl_trigger();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    float v = to_f32(x[i]);
    if (bias) v += bias[i % n];
    from_f32(x[i], activate(v, act));
  }
}

// dst[m,n] = act(src[m,n] + bias[n]): the 32-bit sums of a matrix product become the stored
// activations with one rounding.
template <typename TO>
__global__ void bias_act_out_kernel(const float* src, const float* __restrict__ bias, int act, TO* __restrict__ dst,
                                    size_t total, int n) {
  pdl_trigger();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    float v = src[i];
    if (bias) v += bias[i % n];
    from_f32(dst[i], activate(v, act));
  }
}

}  // namespace cbis

using namespace cbis;

CBIS_EXPORT int cbis_embed_pos_add(const int* tokens, const int* positions, const void* wte, const void* wpe,
                                   float* out, int T, int d, int vocab, int n_pos, int table_dtype, int* err,
                                   void* stream) {
  if (T <= 0) return CBIS_OK;
  if (d <= 0) return CBIS_ERR_BAD_SIZE;
  const int threads = d >= 1024 ? 256 : (d >= 256 ? 128 : 64);
  cudaStream_t st = (cudaStream_t)stream;
  if (table_dtype == CBIS_F32)
    return (int)launch_after(false, embed_pos_add_kernel<float>, dim3(T), dim3(threads), 0, st, tokens, positions,
                           (const float*)wte, (const float*)wpe, out, d, vocab, n_pos, err);
  if (table_dtype == CBIS_BF16)
    return (int)launch_after(false, embed_pos_add_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, st, tokens, positions,
                           (const __nv_bfloat16*)wte, (const __nv_bfloat16*)wpe, out, d, vocab, n_pos, err);
  return CBIS_ERR_BAD_DTYPE;
}

template <typename TD, typename TO>
static int launch_add_layernorm(float* x, const void* delta, const float* delta_bias, const float* gamma,
                                const float* beta, float eps, void* out, const int* rows, int R, int d,
                                cudaStream_t st) {
  const size_t smem = (size_t)(d + 33) * sizeof(float);
  if (smem > 200 * 1024) return CBIS_ERR_TOO_LARGE;
  auto kern = add_layernorm_kernel<TD, TO>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int threads = d >= 2048 ? 512 : (d >= 512 ? 256 : 128);
  return (int)launch_pdl(kern, dim3(R), dim3(threads), smem, st, x, (const TD*)delta, delta_bias, gamma, beta, eps,
                         (TO*)out, rows, d);
}

// delta_dtype / out_dtype: CBIS_F32 or CBIS_BF16.  delta, delta_bias and rows may be null.
CBIS_EXPORT int cbis_add_layernorm(float* x, const void* delta, int delta_dtype, const float* delta_bias,
                                   const float* gamma, const float* beta, float eps, void* out, int out_dtype,
                                   const int* rows, int R, int d, void* stream) {
  if (R <= 0) return CBIS_OK;
  if (d <= 0) return CBIS_ERR_BAD_SIZE;
  cudaStream_t st = (cudaStream_t)stream;
  if (delta_dtype == CBIS_F32 && out_dtype == CBIS_F32)
    return launch_add_layernorm<float, float>(x, delta, delta_bias, gamma, beta, eps, out, rows, R, d, st);
  if (delta_dtype == CBIS_F32 && out_dtype == CBIS_BF16)
    return launch_add_layernorm<float, __nv_bfloat16>(x, delta, delta_bias, gamma, beta, eps, out, rows, R, d, st);
  if (delta_dtype == CBIS_BF16 && out_dtype == CBIS_BF16)
    return launch_add_layernorm<__nv_bfloat16, __nv_bfloat16>(x, delta, delta_bias, gamma, beta, eps, out, rows, R, d, st);
  if (delta_dtype == CBIS_BF16 && out_dtype == CBIS_F32)
    return launch_add_layernorm<__nv_bfloat16, float>(x, delta, delta_bias, gamma, beta, eps, out, rows, R, d, st);
  return CBIS_ERR_BAD_DTYPE;
}

CBIS_EXPORT int cbis_bias_act(void* x, const float* bias, int act, int M, int N, int dtype, void* stream) {
  if (M <= 0 || N <= 0) return CBIS_OK;
  const size_t total = (size_t)M * N;
  const int threads = 256;
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == CBIS_F32)
    return (int)launch_pdl(bias_act_kernel<float>, dim3((int)blocks), dim3(threads), 0, st, (float*)x, bias, act, total, N);
  if (dtype == CBIS_BF16)
    return (int)launch_pdl(bias_act_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(threads), 0, st, (__nv_bfloat16*)x,
                           bias, act, total, N);
  return CBIS_ERR_BAD_DTYPE;
}

CBIS_EXPORT int cbis_bias_act_out(const float* src, const float* bias, int act, void* dst, int M, int N, int dst_dtype,
                                  void* stream) {
  if (M <= 0 || N <= 0) return CBIS_OK;
  const size_t total = (size_t)M * N;
  const int threads = 256;
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  cudaStream_t st = (cudaStream_t)stream;
  if (dst_dtype == CBIS_F32)
    return (int)launch_pdl(bias_act_out_kernel<float>, dim3((int)blocks), dim3(threads), 0, st, src, bias, act,
                           (float*)dst, total, N);
  if (dst_dtype == CBIS_BF16)
    return (int)launch_pdl(bias_act_out_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(threads), 0, st, src, bias, act,
                           (__nv_bfloat16*)dst, total, N);
  return CBIS_ERR_BAD_DTYPE;
}
