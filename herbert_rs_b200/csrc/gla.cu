// Gated linear attention: a matrix of state per head that decays channel by channel.
//
//   a_t = sigmoid(z_t)^(1/tau),  z_t = W2 (W1 h_t) + b      one decay per key channel, in (0, 1)
//   S_t = diag(a_t) S_{t-1} + k_t v_t^T                      S: [key channels][value channels], float
//   o_t = S_t^T q_t                                          q already scaled
//   y_t = RMSNorm(o_t) * w * silu(g_t)                       per head, one weight vector for all heads
//
// The state of a sequence lives in its slot of the cache's state region ([slots][heads][dk][dv]
// floats, zero when the slot is handed out) and is carried from step to step: a step reads it,
// runs its tokens in order and writes it back, so a prompt cut into pieces, or decoded token by
// token, gives the state the whole prompt gives.  Decays, their logarithms, the state and the
// norm are float on both paths; q, k, v, g and W1 h come from the projection as floats.
#include "api.h"
#include "common.cuh"

// ---------------------------------------------------------------------------------------------
// a[t, c] = exp(logsigmoid(z) / tau),  z = b[c] + sum_r low[t, r] * W2[c, r].  A CTA takes GD_TOK tokens whose
// low-rank rows it keeps in shared memory, and a thread one channel: it reads its row of W2 once for all of them.
#define GD_TOK 8
#define GD_THREADS 128
template <typename T>
__global__ void __launch_bounds__(GD_THREADS)
gla_decay_kernel(const float* __restrict__ low, int ld, const T* __restrict__ w2, const float* __restrict__ bias,
                 float inv_tau, float* __restrict__ a, int n_tokens, int C, int R) {
  extern __shared__ float lows[];  // [GD_TOK][R]
  pdl_wait();
  pdl_launch();
  const int t0 = blockIdx.y * GD_TOK, c = blockIdx.x * GD_THREADS + threadIdx.x;
  const int nt = n_tokens - t0 < GD_TOK ? n_tokens - t0 : GD_TOK;
  for (int i = threadIdx.x; i < nt * R; i += GD_THREADS) lows[i] = low[(size_t)(t0 + i / R) * ld + i % R];
  __syncthreads();
  if (c >= C) return;
  const T* wr = w2 + (size_t)c * R;
  float z[GD_TOK];
  const float b = bias ? bias[c] : 0.0f;
#pragma unroll
  for (int i = 0; i < GD_TOK; ++i) z[i] = b;
  for (int r = 0; r < R; ++r) {
    const float w = to_f32(wr[r]);
#pragma unroll
    for (int i = 0; i < GD_TOK; ++i)
      if (i < nt) z[i] = fmaf(lows[i * R + r], w, z[i]);
  }
#pragma unroll
  for (int i = 0; i < GD_TOK; ++i)
    if (i < nt) {
      const float ls = fminf(z[i], 0.0f) - log1pf(expf(-fabsf(z[i])));  // log sigmoid(z)
      a[(size_t)(t0 + i) * C + c] = expf(ls * inv_tau);
    }
}

extern "C" int hb_gla_decay(int dtype, const float* low, int ld, const void* w2, const float* bias, float inv_tau, float* a,
                            int n_tokens, int channels, int low_rank, void* stream) {
  HB_REQUIRE(n_tokens > 0 && channels > 0 && low_rank > 0, "gla_decay: sizes must be positive");
  HB_REQUIRE(ceil_div(n_tokens, GD_TOK) <= 65535, "gla_decay: too many tokens per call");
  const size_t smem = (size_t)GD_TOK * low_rank * sizeof(float);
  HB_REQUIRE(smem <= 48 * 1024, "gla_decay: the decay's inner width %d exceeds what a block keeps in shared memory", low_rank);
  dim3 grid(ceil_div(channels, GD_THREADS), ceil_div(n_tokens, GD_TOK));
  if (dtype == HB_F32)
    hb_launch(gla_decay_kernel<float>, grid, dim3(GD_THREADS), smem, (cudaStream_t)stream, low, ld, (const float*)w2, bias, inv_tau, a, n_tokens, channels, low_rank);
  else
    hb_launch(gla_decay_kernel<bf16>, grid, dim3(GD_THREADS), smem, (cudaStream_t)stream, low, ld, (const bf16*)w2, bias, inv_tau, a, n_tokens, channels, low_rank);
  HB_CHECK_LAUNCH("gla_decay");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// The recurrence.  A block owns COLS (32, 16 or 8) value channels of one head of one sequence and walks
// that sequence's tokens of the step in order; thread (x, y) keeps RPT consecutive state rows of column x
// in registers, 128 / COLS groups of rows side by side (narrower blocks when a step has few sequences and
// heads, so that one long prompt still spreads over the GPU).  q, k, v and the decays of `chunk` tokens at a time are copied into shared memory
// asynchronously, the next chunk while this one is worked on, so the block meets at a barrier twice
// per chunk, not per token.  The tokens of a chunk are still taken one after another: the arithmetic
// is the recurrence's own, whatever the step was cut into.  (q's scale multiplies the sum at the end.)
#define GLA_THREADS 128
__device__ __forceinline__ void gla_copy4(float* smem, const float* gmem) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void gla_copy16(float* smem, const float* gmem) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem));
}

template <int RPT, int COLS>  // rows per thread: dk <= (128 / COLS) * RPT; up to 1,024 key channels with 8 columns
__global__ void __launch_bounds__(GLA_THREADS)
gla_scan_kernel(const float* __restrict__ proj, int ld, int q_off, int k_off, int v_off, const float* __restrict__ decay,
                float* __restrict__ state, const int* __restrict__ seq_slot, const int* __restrict__ seq_start,
                float* __restrict__ out, int ldo, int H, int dk, int dv, float qscale, int chunk, int wide) {
  constexpr int GLA_ROWGROUPS = GLA_THREADS / COLS;
  constexpr int DKP = GLA_ROWGROUPS * RPT;  // padded row count; rows past dk hold zeros and stay zero
  extern __shared__ __align__(16) float sh[];
  const int stage_floats = chunk * (3 * DKP + COLS);
  float* red = sh + 2 * stage_floats;        // [chunk][GLA_ROWGROUPS][COLS]
  pdl_wait();
  pdl_launch();
  const int b = blockIdx.x, h = blockIdx.y, x = threadIdx.x, y = threadIdx.y;
  const int col = blockIdx.z * COLS + x, tid = y * COLS + x;
  const int t0 = seq_start[b], t1 = seq_start[b + 1];
  float* S = state + (((size_t)seq_slot[b] * H + h) * dk) * (size_t)dv;
  float s[RPT];
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int r = y * RPT + i;
    s[i] = (r < dk && col < dv) ? S[(size_t)r * dv + col] : 0.0f;
  }
  for (int i = tid; i < 2 * stage_floats; i += GLA_THREADS) sh[i] = 0.0f;      // the padding stays zero from here on
  __syncthreads();

  auto stage = [&](int buf, int c0) {
    float* qs = sh + buf * stage_floats;
    float* ks = qs + chunk * DKP;
    float* as = ks + chunk * DKP;
    float* vs = as + chunk * DKP;
    const int n = t1 - c0 < chunk ? t1 - c0 : chunk;
    if (wide) {            // every row and offset starts on 16 bytes
      const int per = dk >> 2;
      for (int i = tid; i < n * per; i += GLA_THREADS) {
        const int tt = i / per, r = (i - tt * per) * 4;
        const float* row = proj + (size_t)(c0 + tt) * ld + h * dk + r;
        gla_copy16(qs + tt * DKP + r, row + q_off);
        gla_copy16(ks + tt * DKP + r, row + k_off);
        gla_copy16(as + tt * DKP + r, decay + (size_t)(c0 + tt) * H * dk + h * dk + r);
      }
    } else {
      for (int i = tid; i < n * dk; i += GLA_THREADS) {
        const int tt = i / dk, r = i - tt * dk;
        const float* row = proj + (size_t)(c0 + tt) * ld + h * dk + r;
        gla_copy4(qs + tt * DKP + r, row + q_off);
        gla_copy4(ks + tt * DKP + r, row + k_off);
        gla_copy4(as + tt * DKP + r, decay + (size_t)(c0 + tt) * H * dk + h * dk + r);
      }
    }
    for (int i = tid; i < n * COLS; i += GLA_THREADS) {
      const int tt = i / COLS, c = blockIdx.z * COLS + (i % COLS);
      if (c < dv) gla_copy4(vs + i, proj + (size_t)(c0 + tt) * ld + v_off + h * dv + c);
    }
    asm volatile("cp.async.commit_group;");
  };

  if (t0 < t1) stage(0, t0);
  int buf = 0;
  for (int c0 = t0; c0 < t1; c0 += chunk, buf ^= 1) {
    const int n = t1 - c0 < chunk ? t1 - c0 : chunk;
    if (c0 + chunk < t1) {
      stage(buf ^ 1, c0 + chunk);
      asm volatile("cp.async.wait_group 1;");
    } else {
      asm volatile("cp.async.wait_group 0;");
    }
    __syncthreads();
    const float* qs = sh + buf * stage_floats;
    const float* ks = qs + chunk * DKP;
    const float* as = ks + chunk * DKP;
    const float* vs = as + chunk * DKP;
    for (int tt = 0; tt < n; ++tt) {
      const float v = vs[tt * COLS + x];
      const float4* a4 = reinterpret_cast<const float4*>(as + tt * DKP + y * RPT);
      const float4* k4 = reinterpret_cast<const float4*>(ks + tt * DKP + y * RPT);
      const float4* q4 = reinterpret_cast<const float4*>(qs + tt * DKP + y * RPT);
      float c0a = 0.0f, c1a = 0.0f, c2a = 0.0f, c3a = 0.0f;
#pragma unroll
      for (int i = 0; i < RPT / 4; ++i) {
        const float4 a = a4[i], k = k4[i], q = q4[i];
        s[4 * i] = fmaf(a.x, s[4 * i], k.x * v);
        c0a = fmaf(s[4 * i], q.x, c0a);
        s[4 * i + 1] = fmaf(a.y, s[4 * i + 1], k.y * v);
        c1a = fmaf(s[4 * i + 1], q.y, c1a);
        s[4 * i + 2] = fmaf(a.z, s[4 * i + 2], k.z * v);
        c2a = fmaf(s[4 * i + 2], q.z, c2a);
        s[4 * i + 3] = fmaf(a.w, s[4 * i + 3], k.w * v);
        c3a = fmaf(s[4 * i + 3], q.w, c3a);
      }
      red[(tt * GLA_ROWGROUPS + y) * COLS + x] = (c0a + c1a) + (c2a + c3a);
    }
    __syncthreads();
    for (int i = tid; i < n * COLS; i += GLA_THREADS) {
      const int tt = i / COLS, xx = i % COLS, c = blockIdx.z * COLS + xx;
      if (c < dv) {
        float o = red[(tt * GLA_ROWGROUPS) * COLS + xx];
#pragma unroll
        for (int g = 1; g < GLA_ROWGROUPS; ++g) o += red[(tt * GLA_ROWGROUPS + g) * COLS + xx];
        out[(size_t)(c0 + tt) * ldo + h * dv + c] = o * qscale;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int r = y * RPT + i;
    if (r < dk && col < dv) S[(size_t)r * dv + col] = s[i];
  }
}

extern "C" int hb_gla_scan(const float* proj, int ld, int q_off, int k_off, int v_off, const float* decay, float* state,
                           const int* seq_slot, const int* seq_start, float* out, int ldo, int n_seqs, int heads, int dk,
                           int dv, float qscale, void* stream) {
  HB_REQUIRE(n_seqs > 0 && heads > 0 && dk > 0 && dv > 0, "gla_scan: sizes must be positive");
  HB_REQUIRE(dk <= 16 * 64, "gla_scan: %d key channels per head exceed the supported maximum 1024", dk);
  HB_REQUIRE(heads <= 65535 && ceil_div(dv, 8) <= 65535, "gla_scan: too many heads or value channels");
  cudaStream_t s = (cudaStream_t)stream;
  const int wide = dk % 4 == 0 && ld % 4 == 0 && q_off % 4 == 0 && k_off % 4 == 0 && (((uintptr_t)proj | (uintptr_t)decay) & 15) == 0;
  // the widest blocks that still give every SM one (a long prompt alone: narrower blocks, more of them)
  int sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int cols = dk > 512 ? 8 : dk > 256 ? 16 : 32;                    // at most 64 state rows per thread
  while (cols > 8 && (long long)n_seqs * heads * ceil_div(dv, cols) < sms) cols >>= 1;
  const int groups = GLA_THREADS / cols;
  int rpt = ceil_div(ceil_div(dk, groups), 4) * 4;                 // rows per thread, whole float4s
  rpt = rpt <= 4 ? 4 : rpt <= 8 ? 8 : rpt <= 16 ? 16 : rpt <= 32 ? 32 : 64;
  // tokens per stage: enough work per stage to cover the next stage's way from memory, within 100 KB of shared memory
  const size_t per_token = (size_t)(2 * (3 * groups * rpt + cols) + GLA_THREADS) * sizeof(float);
  const int chunk = (int)(100 * 1024 / per_token) >= 16 ? 16 : ((int)(100 * 1024 / per_token) < 1 ? 1 : (int)(100 * 1024 / per_token));
  dim3 grid(n_seqs, heads, ceil_div(dv, cols)), block(cols, groups);
  const size_t smem = (size_t)chunk * per_token;
#define GLA_GO(RPT, COLS)                                                                                                       \
  do {                                                                                                                          \
    if (smem > 48 * 1024) cudaFuncSetAttribute(gla_scan_kernel<RPT, COLS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    hb_launch(gla_scan_kernel<RPT, COLS>, grid, block, smem, s, proj, ld, q_off, k_off, v_off, decay, state, seq_slot, seq_start, \
              out, ldo, heads, dk, dv, qscale, chunk, wide);                                                                    \
  } while (0)
#define GLA_COLS(RPT)                                       \
  do {                                                      \
    if (cols == 32) GLA_GO(RPT, 32);                        \
    else if (cols == 16) GLA_GO(RPT, 16);                   \
    else GLA_GO(RPT, 8);                                    \
  } while (0)
  if (rpt == 4) GLA_COLS(4); else if (rpt == 8) GLA_COLS(8); else if (rpt == 16) GLA_COLS(16); else if (rpt == 32) GLA_COLS(32);
  else GLA_COLS(64);
#undef GLA_COLS
#undef GLA_GO
  HB_CHECK_LAUNCH("gla_scan");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// y[t, h, :] = o / sqrt(mean(o^2) + eps) * w * silu(g[t, h, :]).  One CTA of 128 threads per (token, head).
template <typename T>
__global__ void __launch_bounds__(128)
gla_output_kernel(const float* __restrict__ o, int ldo, const float* __restrict__ w, float eps, const float* __restrict__ gate,
                  int ldg, T* __restrict__ y, int ldy, int n_tokens, int H, int dv) {
  __shared__ float red[32];
  pdl_wait();
  pdl_launch();
  const int t = blockIdx.x / H, h = blockIdx.x % H;
  const float* orow = o + (size_t)t * ldo + (size_t)h * dv;
  float ss = 0.0f;
  for (int d = threadIdx.x; d < dv; d += blockDim.x) ss += orow[d] * orow[d];
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
  const float* g = gate + (size_t)t * ldg + (size_t)h * dv;
  T* yr = y + (size_t)t * ldy + (size_t)h * dv;
  for (int d = threadIdx.x; d < dv; d += blockDim.x) {
    const float gv = g[d];
    yr[d] = from_f32<T>(((orow[d] * inv) * w[d]) * (gv / (1.0f + expf(-gv))));
  }
}

extern "C" int hb_gla_output(int dtype, const float* o, int ldo, const float* w, float eps, const float* gate, int ldg,
                             void* y, int ldy, int n_tokens, int heads, int dv, void* stream) {
  HB_REQUIRE(n_tokens > 0 && heads > 0 && dv > 0, "gla_output: sizes must be positive");
  const long long blocks = (long long)n_tokens * heads;
  HB_REQUIRE(blocks < 2147483647LL, "gla_output: too many (token, head) pairs");
  const int threads = dv >= 128 ? 128 : (dv >= 64 ? 64 : 32);
  if (dtype == HB_F32)
    hb_launch(gla_output_kernel<float>, dim3((unsigned)blocks), dim3(threads), 0, (cudaStream_t)stream, o, ldo, w, eps, gate, ldg, (float*)y, ldy, n_tokens, heads, dv);
  else
    hb_launch(gla_output_kernel<bf16>, dim3((unsigned)blocks), dim3(threads), 0, (cudaStream_t)stream, o, ldo, w, eps, gate, ldg, (bf16*)y, ldy, n_tokens, heads, dv);
  HB_CHECK_LAUNCH("gla_output");
  return 0;
}
