// Layer normalisation with a weight and no bias, alone and fused with what follows a sublayer whose
// result is normed before it joins the residual stream.
//
//   LN(y)_i = (y_i - mean(y)) / sqrt(var(y) + eps) * w_i,   var = mean((y - mean)^2)
//   alone:     out[r] = LN(x[rows[r]] or x[r])                       (activation dtype)
//   residual:  x[r] += LN(y[r]) * s        (s: a per-channel scale, or none)
//              h[r]  = x[r] in the activation dtype, if asked for: what the next sublayer reads
//
// All arithmetic is float; the mean is taken first and the variance from the deviations (two passes
// over a row that the first pass left in L1).  One block per row.
#include "api.h"
#include "common.cuh"

template <typename T>
__global__ void layernorm_kernel(const float* __restrict__ x, const float* __restrict__ w, T* __restrict__ out,
                                 const int* __restrict__ rows, int dim, float eps) {
  __shared__ float red[32];
  pdl_wait();
  pdl_launch();
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows ? rows[r] : r) * dim;
  float s = 0.0f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) s += xr[i];
  const float mean = block_sum(s, red) / (float)dim;
  float q = 0.0f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    const float d = xr[i] - mean;
    q += d * d;
  }
  const float inv = 1.0f / sqrtf(block_sum(q, red) / (float)dim + eps);
  T* o = out + (size_t)r * dim;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) o[i] = from_f32<T>(((xr[i] - mean) * inv) * w[i]);
}

template <typename T>
__global__ void layernorm_residual_kernel(const float* __restrict__ y, int ldy, const float* __restrict__ w,
                                          const float* __restrict__ scale, float* __restrict__ x,
                                          T* __restrict__ h, int dim, float eps) {
  __shared__ float red[32];
  pdl_wait();
  pdl_launch();
  const int r = blockIdx.x;
  const float* yr = y + (size_t)r * ldy;
  float s = 0.0f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) s += yr[i];
  const float mean = block_sum(s, red) / (float)dim;
  float q = 0.0f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    const float d = yr[i] - mean;
    q += d * d;
  }
  const float inv = 1.0f / sqrtf(block_sum(q, red) / (float)dim + eps);
  float* xr = x + (size_t)r * dim;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    float v = ((yr[i] - mean) * inv) * w[i];
    if (scale) v *= scale[i];
    const float n = xr[i] + v;
    xr[i] = n;
    if (h) h[(size_t)r * dim + i] = from_f32<T>(n);
  }
}

static int ln_threads(int dim) { return dim >= 2048 ? 512 : (dim >= 512 ? 256 : 128); }

extern "C" int hb_layernorm(int dtype, const float* x, const float* w, void* out, const int* rows, int n_rows,
                            int dim, float eps, void* stream) {
  HB_REQUIRE(n_rows > 0 && dim > 0, "layernorm: sizes must be positive");
  if (dtype == HB_F32)
    hb_launch(layernorm_kernel<float>, dim3(n_rows), dim3(ln_threads(dim)), 0, (cudaStream_t)stream, x, w, (float*)out, rows, dim, eps);
  else
    hb_launch(layernorm_kernel<bf16>, dim3(n_rows), dim3(ln_threads(dim)), 0, (cudaStream_t)stream, x, w, (bf16*)out, rows, dim, eps);
  HB_CHECK_LAUNCH("layernorm");
  return 0;
}

extern "C" int hb_layernorm_residual(int dtype, const float* y, int ldy, const float* w, const float* scale,
                                     float* x, void* h, int n_rows, int dim, float eps, void* stream) {
  HB_REQUIRE(n_rows > 0 && dim > 0 && ldy >= dim, "layernorm_residual: sizes must be positive and rows at least dim apart");
  if (dtype == HB_F32)
    hb_launch(layernorm_residual_kernel<float>, dim3(n_rows), dim3(ln_threads(dim)), 0, (cudaStream_t)stream, y, ldy, w, scale, x, (float*)h, dim, eps);
  else
    hb_launch(layernorm_residual_kernel<bf16>, dim3(n_rows), dim3(ln_threads(dim)), 0, (cudaStream_t)stream, y, ldy, w, scale, x, (bf16*)h, dim, eps);
  HB_CHECK_LAUNCH("layernorm_residual");
  return 0;
}
