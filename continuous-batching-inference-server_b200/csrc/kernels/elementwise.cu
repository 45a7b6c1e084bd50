// Embedding + learned positions, residual-add + LayerNorm (with row selection), bias + activation.
// All arithmetic in 32-bit; the residual stream is 32-bit in both precisions.
#include "common.cuh"

namespace cbis {

// x[r,:] = wte[tok[r],:] * tok_scale + wpe[pos[r],:]   (reference: kernels/elementwise.cu:7-17, no scale there)
// A token or position outside its table sets *err (1 = token, 2 = position) and gives a zero row.
template <typename TT>
__global__ void embed_pos_add_kernel(const int* tokens, const int* positions,
                                     const TT* __restrict__ wte, const TT* __restrict__ wpe,
                                     float* __restrict__ out, int d, int vocab, int n_pos, float tok_scale, int* err) {
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
      v = to_f32(trow[c]) * tok_scale;
      if (prow) v += to_f32(prow[c]);
    }
    orow[c] = v;
  }
}

// One block per output row r; src row s = rows ? rows[r] : r.
//   v = x[s,:] (+ delta[s,:]) (+ delta_bias[:])           32-bit
//   if rows == nullptr and (delta or bias): x[s,:] = v      the residual stream moves on
//   out[r,:] = (v - mean) * rsqrt(var + eps) * gamma + beta      (gamma == nullptr: out[r,:] = v, no norm)
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
    from_f32(orow[c], gamma ? (v - mean) * inv * gamma[c] + (beta ? beta[c] : 0.f) : v);
  }
}

// The same for widths that are a multiple of 4 and at most 128*4*NV: the row stays in registers
// (NV float4 per thread, 128 threads per row), every access is 16 bytes wide, no staging in shared
// memory.  TD/TO: float or bfloat16.
template <typename TT>
__device__ __forceinline__ float4 load4(const TT* p);
template <>
__device__ __forceinline__ float4 load4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <>
__device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 r = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 r;
  r.x = *reinterpret_cast<uint32_t*>(&a);
  r.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = r;
}

template <typename TD, typename TO, int NV>
__global__ void __launch_bounds__(128)
add_layernorm_reg_kernel(float* x, const TD* delta, const float* __restrict__ delta_bias,
                         const float* __restrict__ gamma, const float* __restrict__ beta, float eps, TO* __restrict__ out,
                         const int* rows, int d) {
  __shared__ float red[33];
  pdl_trigger();
  const int nvec = d >> 2;
  // parameters first: no earlier kernel writes them, so they are fetched while the kernels ahead still run
  float4 gm[NV], bt[NV], db[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = threadIdx.x + i * 128;
    gm[i] = bt[i] = db[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < nvec) {
      if (gamma) gm[i] = *reinterpret_cast<const float4*>(gamma + 4 * c);
      if (beta) bt[i] = *reinterpret_cast<const float4*>(beta + 4 * c);
      if (delta_bias) db[i] = *reinterpret_cast<const float4*>(delta_bias + 4 * c);
    }
  }
  pdl_wait();
  const int r = blockIdx.x;
  const int s = rows ? rows[r] : r;
  float* xrow = x + (size_t)s * d;
  const TD* drow = delta ? delta + (size_t)s * d : nullptr;
  float4 v[NV];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = threadIdx.x + i * 128;
    v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < nvec) {
      v[i] = *reinterpret_cast<const float4*>(xrow + 4 * c);
      if (drow) {
        const float4 t = load4<TD>(drow + 4 * c);
        v[i].x += t.x; v[i].y += t.y; v[i].z += t.z; v[i].w += t.w;
      }
      v[i].x += db[i].x; v[i].y += db[i].y; v[i].z += db[i].z; v[i].w += db[i].w;
      sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
  }
  const float mean = block_sum(sum, red) / (float)d;
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    if (threadIdx.x + i * 128 < nvec) {
      const float a = v[i].x - mean, b = v[i].y - mean, c2 = v[i].z - mean, e = v[i].w - mean;
      sq += (a * a + b * b) + (c2 * c2 + e * e);
    }
  }
  const float var = block_sum(sq, red) / (float)d;
  const float inv = rsqrtf(var + eps);
  const bool write_x = rows == nullptr && (drow != nullptr || delta_bias != nullptr);
  TO* orow = out + (size_t)r * d;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = threadIdx.x + i * 128;
    if (c < nvec) {
      if (write_x) *reinterpret_cast<float4*>(xrow + 4 * c) = v[i];
      float4 y = v[i];
      if (gamma) {
        y.x = (v[i].x - mean) * inv * gm[i].x + bt[i].x;
        y.y = (v[i].y - mean) * inv * gm[i].y + bt[i].y;
        y.z = (v[i].z - mean) * inv * gm[i].z + bt[i].z;
        y.w = (v[i].w - mean) * inv * gm[i].w + bt[i].w;
      }
      store4(orow + 4 * c, y);
    }
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

// x = cap > 0 ? cap * tanh(x * scale / cap) : x * scale, in place (logits of a head with a scale or a soft cap).
__global__ void scale_soft_cap_kernel(float* x, float scale, float cap, size_t total) {
  pdl_trigger();
  pdl_wait();
  const float inv_cap = cap > 0.f ? 1.0f / cap : 0.f;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const float v = x[i] * scale;
    x[i] = cap > 0.f ? cap * tanhf(v * inv_cap) : v;
  }
}

}  // namespace cbis

using namespace cbis;

// The widest row the norm kernel takes (it is staged in shared memory beyond 8,192 columns).
CBIS_EXPORT int cbis_norm_max_width() { return (200 * 1024) / (int)sizeof(float) - 33; }

CBIS_EXPORT int cbis_scale_soft_cap(float* x, float scale, float cap, int M, int N, void* stream) {
  if (M <= 0 || N <= 0) return CBIS_OK;
  const size_t total = (size_t)M * N;
  size_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  return (int)launch_pdl(scale_soft_cap_kernel, dim3((int)blocks), dim3(256), 0, (cudaStream_t)stream, x, scale, cap, total);
}

CBIS_EXPORT int cbis_embed_pos_add(const int* tokens, const int* positions, const void* wte, const void* wpe,
                                   float* out, int T, int d, int vocab, int n_pos, int table_dtype, float tok_scale,
                                   int* err, void* stream) {
  if (T <= 0) return CBIS_OK;
  if (d <= 0) return CBIS_ERR_BAD_SIZE;
  const int threads = d >= 1024 ? 256 : (d >= 256 ? 128 : 64);
  cudaStream_t st = (cudaStream_t)stream;
  if (table_dtype == CBIS_F32)
    return (int)launch_after(false, embed_pos_add_kernel<float>, dim3(T), dim3(threads), 0, st, tokens, positions,
                           (const float*)wte, (const float*)wpe, out, d, vocab, n_pos, tok_scale, err);
  if (table_dtype == CBIS_BF16)
    return (int)launch_after(false, embed_pos_add_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, st, tokens, positions,
                           (const __nv_bfloat16*)wte, (const __nv_bfloat16*)wpe, out, d, vocab, n_pos, tok_scale, err);
  return CBIS_ERR_BAD_DTYPE;
}

template <typename TD, typename TO>
static int launch_add_layernorm(float* x, const void* delta, const float* delta_bias, const float* gamma,
                                const float* beta, float eps, void* out, const int* rows, int R, int d,
                                cudaStream_t st) {
  const bool aligned = !(((uintptr_t)x | (uintptr_t)delta | (uintptr_t)delta_bias | (uintptr_t)gamma | (uintptr_t)beta |
                          (uintptr_t)out) & 15);
  if (d % 4 == 0 && d <= 128 * 4 * 16 && aligned) {  // the row fits into the registers of 128 threads
#define CBIS_LN(NV)                                                                                              \
  return (int)launch_pdl(add_layernorm_reg_kernel<TD, TO, NV>, dim3(R), dim3(128), 0, st, x, (const TD*)delta, \
                         delta_bias, gamma, beta, eps, (TO*)out, rows, d)
    if (d <= 128 * 4 * 1) CBIS_LN(1);
    if (d <= 128 * 4 * 2) CBIS_LN(2);
    if (d <= 128 * 4 * 4) CBIS_LN(4);
    if (d <= 128 * 4 * 8) CBIS_LN(8);
    CBIS_LN(16);
#undef CBIS_LN
  }
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
