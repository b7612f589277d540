// A routed feed-forward: every token goes through `top` of E small feed-forwards.
//
//   z = R h (float);  s = softmax(z) over all E experts;  the `top` largest s are chosen
//   weights: the chosen s themselves, or (renorm) divided by their sum
//   y = sum over the chosen e of weight_e * Down_e act(Up_e h)      act: gelu (erf form) or silu
//
// Three launches, all reading the choice from device memory (nothing of it is known to the host, so
// a recorded step can be replayed): the router with softmax and choice; the chosen experts' first
// product with the activation; their second product with the weighted sum.  A warp computes one
// output number from one weight row read along its length, which is what a step of few tokens
// wants: every weight row of a chosen expert is read once per token that chose it.
#include "api.h"
#include "common.cuh"

#define MOE_WARPS 4

template <typename T>
__global__ void __launch_bounds__(MOE_WARPS * 32)
moe_route_kernel(const T* __restrict__ h, int ld, const T* __restrict__ wr, int* __restrict__ ids, float* __restrict__ wts,
                 int n_tokens, int D, int E, int top, int renorm) {
  extern __shared__ float sh[];  // [MOE_WARPS][E]
  pdl_wait();
  pdl_launch();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * MOE_WARPS + warp;
  if (t >= n_tokens) return;
  float* s = sh + (size_t)warp * E;
  const T* hr = h + (size_t)t * ld;
  for (int e = 0; e < E; ++e) {
    const T* w = wr + (size_t)e * D;
    float dot = 0.0f;
    for (int d = lane; d < D; d += 32) dot = fmaf(to_f32(hr[d]), to_f32(w[d]), dot);
    dot = warp_sum(dot);
    if (lane == 0) s[e] = dot;
  }
  __syncwarp();
  float mx = -INFINITY;
  for (int e = lane; e < E; e += 32) mx = fmaxf(mx, s[e]);
  mx = warp_max(mx);
  float sum = 0.0f;
  for (int e = lane; e < E; e += 32) sum += expf(s[e] - mx);
  sum = warp_sum(sum);
  for (int e = lane; e < E; e += 32) s[e] = expf(s[e] - mx) / sum;
  __syncwarp();
  float chosen_sum = 0.0f;
  for (int r = 0; r < top; ++r) {
    float best = -1.0f;
    int bi = E;
    for (int e = lane; e < E; e += 32)
      if (s[e] > best) { best = s[e]; bi = e; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if (lane == 0) {
      ids[(size_t)t * top + r] = bi;
      wts[(size_t)t * top + r] = best;
      s[bi] = -2.0f;  // taken
    }
    chosen_sum += best;
    __syncwarp();
  }
  if (renorm && lane == 0)
    for (int r = 0; r < top; ++r) wts[(size_t)t * top + r] /= chosen_sum;
}

extern "C" int hb_moe_route(int dtype, const void* h, int ld, const void* w_router, int* ids, float* weights, int n_tokens,
                            int D, int E, int top, int renorm, void* stream) {
  HB_REQUIRE(n_tokens > 0 && D > 0 && E > 0 && top > 0 && top <= E, "moe_route: bad sizes (experts %d, top %d)", E, top);
  const size_t smem = (size_t)MOE_WARPS * E * sizeof(float);
  HB_REQUIRE(smem <= 48 * 1024, "moe_route: %d experts exceed what a block keeps in shared memory", E);
  dim3 grid(ceil_div(n_tokens, MOE_WARPS));
  if (dtype == HB_F32)
    hb_launch(moe_route_kernel<float>, grid, dim3(MOE_WARPS * 32), smem, (cudaStream_t)stream, (const float*)h, ld, (const float*)w_router, ids, weights, n_tokens, D, E, top, renorm);
  else
    hb_launch(moe_route_kernel<bf16>, grid, dim3(MOE_WARPS * 32), smem, (cudaStream_t)stream, (const bf16*)h, ld, (const bf16*)w_router, ids, weights, n_tokens, D, E, top, renorm);
  HB_CHECK_LAUNCH("moe_route");
  return 0;
}

__device__ __forceinline__ float moe_act(float z, int act) {
  if (act == HB_ACT_GELU) return 0.5f * z * (1.0f + erff(z * 0.70710678118654752440f));
  if (act == HB_ACT_GELU_TANH) return 0.5f * z * (1.0f + tanhf(0.79788456080286535588f * (z + 0.044715f * z * z * z)));
  return z / (1.0f + expf(-z));
}

// mid[(t*top + r), f] = act(Up_e[f, :] . h[t, :]),  e = ids[t, r].  One warp per output.
template <typename T>
__global__ void __launch_bounds__(MOE_WARPS * 32)
moe_up_kernel(const T* __restrict__ h, int ld, const T* __restrict__ up, const int* __restrict__ ids, T* __restrict__ mid,
              int D, int F, int top, int act) {
  pdl_wait();
  pdl_launch();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int f = blockIdx.y * MOE_WARPS + warp, u = blockIdx.x;  // u = t*top + r
  if (f >= F) return;
  const int e = ids[u];
  const T* w = up + ((size_t)e * F + f) * D;
  const T* hr = h + (size_t)(u / top) * ld;
  float dot = 0.0f;
  for (int d = lane; d < D; d += 32) dot = fmaf(to_f32(hr[d]), to_f32(w[d]), dot);
  dot = warp_sum(dot);
  if (lane == 0) mid[(size_t)u * F + f] = from_f32<T>(moe_act(dot, act));
}

// y[t, d] (+)= sum_r wts[t, r] * Down_e[d, :] . mid[(t*top + r), :].  One warp per output.
template <typename T>
__global__ void __launch_bounds__(MOE_WARPS * 32)
moe_down_kernel(const T* __restrict__ mid, const T* __restrict__ down, const int* __restrict__ ids, const float* __restrict__ wts,
                float* __restrict__ y, int ldy, int D, int F, int top, int accumulate) {
  pdl_wait();
  pdl_launch();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int d = blockIdx.y * MOE_WARPS + warp, t = blockIdx.x;
  if (d >= D) return;
  float acc = 0.0f;
  for (int r = 0; r < top; ++r) {
    const int u = t * top + r;
    const T* w = down + ((size_t)ids[u] * D + d) * F;
    const T* m = mid + (size_t)u * F;
    float dot = 0.0f;
    for (int f = lane; f < F; f += 32) dot = fmaf(to_f32(m[f]), to_f32(w[f]), dot);
    acc = fmaf(wts[u], warp_sum(dot), acc);
  }
  if (lane == 0) {
    float* o = y + (size_t)t * ldy + d;
    *o = accumulate ? *o + acc : acc;
  }
}

extern "C" int hb_moe_experts(int dtype, const void* h, int ld, const void* up, const void* down, const int* ids,
                              const float* weights, void* mid, float* y, int ldy, int n_tokens, int D, int F, int top,
                              int act, int accumulate, void* stream) {
  HB_REQUIRE(n_tokens > 0 && D > 0 && F > 0 && top > 0, "moe_experts: sizes must be positive");
  HB_REQUIRE((long long)n_tokens * top < 2147483647LL && ceil_div(F, MOE_WARPS) <= 65535 && ceil_div(D, MOE_WARPS) <= 65535,
             "moe_experts: too many (token, choice) pairs or channels");
  cudaStream_t s = (cudaStream_t)stream;
  dim3 g1(n_tokens * top, ceil_div(F, MOE_WARPS)), g2(n_tokens, ceil_div(D, MOE_WARPS));
  if (dtype == HB_F32) {
    hb_launch(moe_up_kernel<float>, g1, dim3(MOE_WARPS * 32), 0, s, (const float*)h, ld, (const float*)up, ids, (float*)mid, D, F, top, act);
    hb_launch(moe_down_kernel<float>, g2, dim3(MOE_WARPS * 32), 0, s, (const float*)mid, (const float*)down, ids, weights, y, ldy, D, F, top, accumulate);
  } else {
    hb_launch(moe_up_kernel<bf16>, g1, dim3(MOE_WARPS * 32), 0, s, (const bf16*)h, ld, (const bf16*)up, ids, (bf16*)mid, D, F, top, act);
    hb_launch(moe_down_kernel<bf16>, g2, dim3(MOE_WARPS * 32), 0, s, (const bf16*)mid, (const bf16*)down, ids, weights, y, ldy, D, F, top, accumulate);
  }
  HB_CHECK_LAUNCH("moe_experts");
  return 0;
}
