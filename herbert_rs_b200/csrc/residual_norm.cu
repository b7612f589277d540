// The residual sum of a block whose sublayers' results are added with one factor, and the RMS norm
// that the next block begins with, in one pass over the row:
//   x[r, :] += mult * y[r, :]                                     (float)
//   h[r, :]  = x[r, :] / sqrt(mean(x[r, :]^2) + eps) * w          (if a next norm is given; h in T)
// One block per row; the updated row stays in registers between the sum and the norm when it is
// short enough, else it is read again.
#include "api.h"
#include "common.cuh"

#define RNORM_KEEP 8

template <typename T>
__global__ void scaled_residual_norm_kernel(const float* __restrict__ y, int ldy, float mult, float* __restrict__ x,
                                            const float* __restrict__ w, T* __restrict__ h, int dim, float eps) {
  __shared__ float red[32];
  pdl_wait();
  pdl_launch();
  const int r = blockIdx.x;
  const float* yr = y + (size_t)r * ldy;
  float* xr = x + (size_t)r * dim;
  float keep[RNORM_KEEP];
  float s = 0.0f;
  int n = 0;
  for (int i = threadIdx.x; i < dim; i += blockDim.x, ++n) {
    const float v = fmaf(mult, yr[i], xr[i]);
    xr[i] = v;
    if (n < RNORM_KEEP) keep[n] = v;
    s = fmaf(v, v, s);
  }
  if (h == nullptr) return;
  s = block_sum(s, red);
  const float inv = 1.0f / sqrtf(s / (float)dim + eps);
  T* hr = h + (size_t)r * dim;
  n = 0;
  for (int i = threadIdx.x; i < dim; i += blockDim.x, ++n) {
    const float v = n < RNORM_KEEP ? keep[n] : xr[i];
    hr[i] = from_f32<T>((v * inv) * w[i]);
  }
}

extern "C" int hb_scaled_residual_norm(int dtype, const float* y, int ldy, float mult, float* x, const float* w, void* h,
                                       int n_rows, int dim, float eps, void* stream) {
  HB_REQUIRE(n_rows > 0 && dim > 0 && ldy >= dim, "scaled_residual_norm: sizes must be positive and rows at least dim apart");
  HB_REQUIRE((w == nullptr) == (h == nullptr), "scaled_residual_norm: the next norm needs both a weight and an output");
  const int threads = dim >= 2048 ? 512 : (dim >= 512 ? 256 : 128);
  if (dtype == HB_F32)
    hb_launch(scaled_residual_norm_kernel<float>, dim3(n_rows), dim3(threads), 0, (cudaStream_t)stream, y, ldy, mult, x, w, (float*)h, dim, eps);
  else
    hb_launch(scaled_residual_norm_kernel<bf16>, dim3(n_rows), dim3(threads), 0, (cudaStream_t)stream, y, ldy, mult, x, w, (bf16*)h, dim, eps);
  HB_CHECK_LAUNCH("scaled_residual_norm");
  return 0;
}
