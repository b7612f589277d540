// Attention over a cached latent: every token stores one vector [c | r] (c: `rank` numbers, normed;
// r: `rot` numbers, rotated by position) from which all heads' keys and values follow
// (k_h = [Uk_h c | r], v_h = Uv_h c).  The kernels never build k or v.  With q_h = [a_h | b_h]:
//
//   score(t, j) = a_h . (Uk_h c_j) + b_h . r_j = (Uk_h^T a_h) . c_j + b_h . r_j
//   out_h       = Uv_h (sum_j p_j c_j)
//
// so a query becomes one vector of rank + rot numbers (`hb_headwise_gemm` makes Uk_h^T a_h,
// `hb_rotate_heads` the rotated part), attention runs with ONE key/value "head" shared by all query
// heads and returns sum_j p_j c_j, and `hb_headwise_gemm` again lifts that to the value size.
//
//   softmax     p_j = exp(s_j) / (sum_i exp(s_i) + exp(sink_h)): the sink has no key and no value
//   range       keys lo..p of the query at position p, lo = max(0, p - window + 1) (window 0: all)
//   rotation    pair (i, i + rot/2) at position p turns by a = p * f_i; cos a and sin a are both
//               multiplied by one constant m (frequency scaling folds into f and m on the host)
//   cache       one plane [pages][page_size][rank + rot] in the activation dtype
//
// Scores, softmax, angles and the norm of c are float on both paths.
#include "api.h"
#include "common.cuh"
#include "mma_utils.cuh"

// ---------------------------------------------------------------------------------------------
// One warp per token: c = RMSNorm(kv[:rank]) * w, r = rotate(kv[rank:]), both into the cache.
template <typename T>
__global__ void latent_kv_store_kernel(const float* __restrict__ kv, int ld, const float* __restrict__ nw, float eps,
                                       const float* __restrict__ freq, float mscale, int rank, int rot,
                                       const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                       const int* __restrict__ seq_pages, int pages_stride, T* __restrict__ cache,
                                       int n_tokens, int page_size) {
  pdl_wait();
  pdl_launch();
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= n_tokens) return;
  const float* row = kv + (size_t)t * ld;
  float ss = 0.0f;
  for (int i = lane; i < rank; i += 32) ss += row[i] * row[i];
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)rank + eps);
  const int p = tok_pos[t], b = tok_seq[t];
  const int page = seq_pages[(size_t)b * pages_stride + p / page_size];
  T* dst = cache + ((size_t)page * page_size + (p % page_size)) * (size_t)(rank + rot);
  for (int i = lane; i < rank; i += 32) dst[i] = from_f32<T>((row[i] * inv) * nw[i]);
  const int half = rot >> 1;
  for (int i = lane; i < half; i += 32) {
    float s, c;
    sincosf((float)p * freq[i], &s, &c);
    s *= mscale;
    c *= mscale;
    const float u = row[rank + i], v = row[rank + half + i];
    dst[rank + i] = from_f32<T>(u * c - v * s);
    dst[rank + half + i] = from_f32<T>(v * c + u * s);
  }
}

extern "C" int hb_latent_kv_store(int dtype, const float* kv, int ld, const float* norm_w, float eps, const float* freq,
                                  float mscale, int rank, int rot, const int* tok_seq, const int* tok_pos,
                                  const int* seq_pages, int pages_stride, void* cache, int n_tokens, int page_size,
                                  void* stream) {
  HB_REQUIRE(n_tokens > 0 && rank > 0 && rot >= 0 && rot % 2 == 0 && page_size > 0, "latent_kv_store: bad sizes");
  HB_REQUIRE(ld >= rank + rot, "latent_kv_store: rows are shorter than rank + rot");
  const int warps = 4;
  dim3 grid(ceil_div(n_tokens, warps));
  if (dtype == HB_F32)
    hb_launch(latent_kv_store_kernel<float>, grid, dim3(warps * 32), 0, (cudaStream_t)stream, kv, ld, norm_w, eps, freq, mscale, rank,
              rot, tok_seq, tok_pos, seq_pages, pages_stride, (float*)cache, n_tokens, page_size);
  else
    hb_launch(latent_kv_store_kernel<bf16>, grid, dim3(warps * 32), 0, (cudaStream_t)stream, kv, ld, norm_w, eps, freq, mscale, rank,
              rot, tok_seq, tok_pos, seq_pages, pages_stride, (bf16*)cache, n_tokens, page_size);
  HB_CHECK_LAUNCH("latent_kv_store");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// The rotated part of every head of every token: in[t, h*in_hs + in_off + ..rot] -> out[t, h*out_hs + out_off + ..rot],
// rotated at the token's position and multiplied by `scale`.  One thread per pair.
__global__ void rotate_heads_kernel(const float* __restrict__ in, int ld_in, int in_hs, int in_off, float* __restrict__ out,
                                    int ld_out, int out_hs, int out_off, const float* __restrict__ freq, float mscale,
                                    const int* __restrict__ tok_pos, int n_tokens, int H, int rot, float scale) {
  pdl_wait();
  pdl_launch();
  const int half = rot >> 1;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)n_tokens * H * half) return;
  const int i = (int)(idx % half), h = (int)((idx / half) % H), t = (int)(idx / ((long long)half * H));
  float s, c;
  sincosf((float)tok_pos[t] * freq[i], &s, &c);
  s *= mscale;
  c *= mscale;
  const float* src = in + (size_t)t * ld_in + (size_t)h * in_hs + in_off;
  float* dst = out + (size_t)t * ld_out + (size_t)h * out_hs + out_off;
  const float u = src[i], v = src[half + i];
  dst[i] = (u * c - v * s) * scale;
  dst[half + i] = (v * c + u * s) * scale;
}

extern "C" int hb_rotate_heads(const float* in, int ld_in, int in_head_stride, int in_offset, float* out, int ld_out,
                               int out_head_stride, int out_offset, const float* freq, float mscale, const int* tok_pos,
                               int n_tokens, int heads, int rot, float scale, void* stream) {
  HB_REQUIRE(n_tokens > 0 && heads > 0 && rot >= 0 && rot % 2 == 0, "rotate_heads: bad sizes");
  if (rot == 0) return 0;
  const long long n = (long long)n_tokens * heads * (rot / 2);
  hb_launch(rotate_heads_kernel, dim3((unsigned)ceil_div_ll(n, 256)), dim3(256), 0, (cudaStream_t)stream, in, ld_in, in_head_stride,
            in_offset, out, ld_out, out_head_stride, out_offset, freq, mscale, tok_pos, n_tokens, heads, rot, scale);
  HB_CHECK_LAUNCH("rotate_heads");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// A product per head:  out[t, h*out_hs + n] = scale * sum_k in[t, h*in_hs + k] * W[h][n][k]   (n < N, k < K)
// optionally times sigmoid(gate[t, h*N + n]).  W is [H][N][K] with k innermost.
//  * few tokens: a warp per (head, n) reads its weight row once, 16 bytes per lane and step, against up to
//    HW_TT tokens' input rows;
//  * many tokens, bfloat16: tiles of 64 tokens x 64 outputs of one head on the tensor cores (mma.sync), the
//    float inputs rounded to bfloat16 on their way into shared memory, as a product's inputs are.
#define HW_TT 8
#define HW_WARPS 4
__device__ __forceinline__ void hw_load8(const float* p, float* v) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void hw_load8(const bf16* p, float* v) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __bfloat1622float2(h2[j]);
    v[2 * j] = f.x;
    v[2 * j + 1] = f.y;
  }
}

template <typename TW, typename TO>
__global__ void __launch_bounds__(HW_WARPS * 32)
headwise_dot_kernel(const float* __restrict__ in, int ld_in, int in_hs, const TW* __restrict__ w, TO* __restrict__ out,
                    int ld_out, int out_hs, const float* __restrict__ gate, int ld_gate, int n_tokens, int K, int N,
                    float scale, int vec) {
  pdl_wait();
  pdl_launch();
  const int lane = threadIdx.x & 31, n = blockIdx.x * HW_WARPS + (threadIdx.x >> 5), h = blockIdx.y, t0 = blockIdx.z * HW_TT;
  if (n >= N) return;
  const TW* wr = w + ((size_t)h * N + n) * K;
  const float* a0 = in + (size_t)t0 * ld_in + (size_t)h * in_hs;
  const int nt = n_tokens - t0 < HW_TT ? n_tokens - t0 : HW_TT;
  float acc[HW_TT];
#pragma unroll
  for (int i = 0; i < HW_TT; ++i) acc[i] = 0.0f;
  if (vec) {
    for (int k = lane * 8; k < K; k += 256) {
      float wv[8], av[8];
      hw_load8(wr + k, wv);
#pragma unroll
      for (int i = 0; i < HW_TT; ++i)
        if (i < nt) {
          hw_load8(a0 + (size_t)i * ld_in + k, av);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[i] = fmaf(av[j], wv[j], acc[i]);
        }
    }
  } else {
    for (int k = lane; k < K; k += 32) {
      const float wv = to_f32(wr[k]);
#pragma unroll
      for (int i = 0; i < HW_TT; ++i)
        if (i < nt) acc[i] = fmaf(a0[(size_t)i * ld_in + k], wv, acc[i]);
    }
  }
#pragma unroll
  for (int i = 0; i < HW_TT; ++i) {
    const float v = warp_sum(acc[i]) * scale;
    if (lane == 0 && i < nt) {
      const int t = t0 + i;
      float r = v;
      if (gate) r *= 1.0f / (1.0f + expf(-gate[(size_t)t * ld_gate + (size_t)h * N + n]));
      out[(size_t)t * ld_out + (size_t)h * out_hs + n] = from_f32<TO>(r);
    }
  }
}

#define HM_TM 64
#define HM_TN 64
#define HM_TK 32
template <typename TO>
__global__ void __launch_bounds__(128)
headwise_mma_kernel(const float* __restrict__ in, int ld_in, int in_hs, const bf16* __restrict__ w, TO* __restrict__ out,
                    int ld_out, int out_hs, const float* __restrict__ gate, int ld_gate, int n_tokens, int K, int N,
                    float scale) {
  __shared__ __align__(16) bf16 As[2][HM_TM][HM_TK + 8];
  __shared__ __align__(16) bf16 Ws[2][HM_TN][HM_TK + 8];
  pdl_wait();
  pdl_launch();
  const int t0 = blockIdx.x * HM_TM, h = blockIdx.y, n0 = blockIdx.z * HM_TN;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const bf16* wh = w + (size_t)h * N * K;
  const float* ah = in + (size_t)h * in_hs;

  auto load = [&](int buf, int k0) {
    for (int i = tid; i < HM_TN * (HM_TK / 8); i += 128) {       // weights: 16-byte pieces, asynchronously
      const int r = i >> 2, c = (i & 3) * 8;
      if (n0 + r < N && k0 + c < K) cp_async16(&Ws[buf][r][c], wh + (size_t)(n0 + r) * K + k0 + c);
      else *reinterpret_cast<uint4*>(&Ws[buf][r][c]) = make_uint4(0, 0, 0, 0);
    }
    cp_async_commit();
    for (int i = tid; i < HM_TM * (HM_TK / 4); i += 128) {       // inputs: four floats become four bfloat16
      const int r = i >> 3, c = (i & 7) * 4;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (t0 + r < n_tokens && k0 + c < K) v = *reinterpret_cast<const float4*>(ah + (size_t)(t0 + r) * ld_in + k0 + c);
      *reinterpret_cast<__nv_bfloat162*>(&As[buf][r][c]) = __floats2bfloat162_rn(v.x, v.y);
      *reinterpret_cast<__nv_bfloat162*>(&As[buf][r][c + 2]) = __floats2bfloat162_rn(v.z, v.w);
    }
  };

  float acc[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[i][c] = 0.0f;
  const int nk = (K + HM_TK - 1) / HM_TK;
  load(0, 0);
  for (int kb = 0; kb < nk; ++kb) {
    if (kb + 1 < nk) {
      load((kb + 1) & 1, (kb + 1) * HM_TK);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int buf = kb & 1;
#pragma unroll
    for (int ks = 0; ks < HM_TK / 16; ++ks) {
      unsigned a0, a1, a2, a3;
      ldmatrix_x4(a0, a1, a2, a3, &As[buf][warp * 16 + (lane & 15)][ks * 16 + (lane >> 4) * 8]);
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        unsigned b0, b1, b2, b3;
        ldmatrix_x4(b0, b1, b2, b3, &Ws[buf][np * 16 + (lane & 7) + ((lane >> 4) << 3)][ks * 16 + ((lane >> 3) & 1) * 8]);
        mma16816(acc[2 * np], a0, a1, a2, a3, b0, b1);
        mma16816(acc[2 * np + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int tk = t0 + warp * 16 + g + half * 8;
    if (tk >= n_tokens) continue;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int n = n0 + nt * 8 + 2 * t + c;
        if (n >= N) continue;
        float v = acc[nt][half * 2 + c] * scale;
        if (gate) v *= 1.0f / (1.0f + expf(-gate[(size_t)tk * ld_gate + (size_t)h * N + n]));
        out[(size_t)tk * ld_out + (size_t)h * out_hs + n] = from_f32<TO>(v);
      }
  }
}

extern "C" int hb_headwise_gemm(int dtype, int out_dtype, const float* in, int ld_in, int in_head_stride, const void* w,
                                void* out, int ld_out, int out_head_stride, const float* gate, int ld_gate, int n_tokens,
                                int heads, int K, int N, float scale, void* stream) {
  HB_REQUIRE(n_tokens > 0 && heads > 0 && K > 0 && N > 0, "headwise_gemm: sizes must be positive");
  HB_REQUIRE(heads <= 65535 && ceil_div(n_tokens, HW_TT) <= 65535 && ceil_div(N, HM_TN) <= 65535, "headwise_gemm: too many heads, tokens or outputs");
  cudaStream_t s = (cudaStream_t)stream;
  HB_REQUIRE(dtype != HB_F32 || out_dtype == HB_F32, "headwise_gemm: the 32-bit path writes floats");
  // 16-byte loads need rows that start on 16 bytes: every stride a multiple of 8 elements (of 4 for the float inputs of the tiles)
  const bool in4 = ld_in % 4 == 0 && in_head_stride % 4 == 0 && ((uintptr_t)in & 15) == 0;
  const bool vec = K % 8 == 0 && ld_in % 8 == 0 && in_head_stride % 8 == 0 && ((uintptr_t)in & 31) == 0 && ((uintptr_t)w & 15) == 0;
  if (dtype == HB_BF16 && n_tokens >= 32 && K % 8 == 0 && in4 && ((uintptr_t)w & 15) == 0) {
    dim3 grid(ceil_div(n_tokens, HM_TM), heads, ceil_div(N, HM_TN));
    if (out_dtype == HB_F32)
      hb_launch(headwise_mma_kernel<float>, grid, dim3(128), 0, s, in, ld_in, in_head_stride, (const bf16*)w, (float*)out, ld_out,
                out_head_stride, gate, ld_gate, n_tokens, K, N, scale);
    else
      hb_launch(headwise_mma_kernel<bf16>, grid, dim3(128), 0, s, in, ld_in, in_head_stride, (const bf16*)w, (bf16*)out, ld_out,
                out_head_stride, gate, ld_gate, n_tokens, K, N, scale);
    HB_CHECK_LAUNCH("headwise_gemm");
    return 0;
  }
  dim3 grid(ceil_div(N, HW_WARPS), heads, ceil_div(n_tokens, HW_TT));
#define HW_GO(TW, TO)                                                                                                          \
  hb_launch(headwise_dot_kernel<TW, TO>, grid, dim3(HW_WARPS * 32), 0, s, in, ld_in, in_head_stride, (const TW*)w, (TO*)out, ld_out, \
            out_head_stride, gate, ld_gate, n_tokens, K, N, scale, vec ? 1 : 0)
  if (dtype == HB_F32) HW_GO(float, float);
  else if (out_dtype == HB_F32) HW_GO(bf16, float);
  else HW_GO(bf16, bf16);
#undef HW_GO
  HB_CHECK_LAUNCH("headwise_gemm");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// One warp per (token, head), 32 keys at a time (a lane per key for the scores, a lane per channel
// for the sum).  q: [T][H][rank + rot] floats, already scaled.  out: [T][H][rank] floats.  The online
// softmax starts from the sink as if it were a first key with value zero: m = sink, l = 1.
#define LA_WARPS 4
template <typename T, int CH>  // CH = ceil(rank / 32)
__global__ void __launch_bounds__(LA_WARPS * 32)
latent_attention_kernel(const float* __restrict__ q, int ldq, float* __restrict__ out, int ldo, const T* __restrict__ cache,
                        const float* __restrict__ sink, const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                        const int* __restrict__ seq_pages, int pages_stride, int n_tokens, int H, int rank, int rot,
                        int page_size, int window) {
  extern __shared__ float qs[];  // [LA_WARPS][rank + rot]
  pdl_wait();
  pdl_launch();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, W = rank + rot;
  const long long unit = (long long)blockIdx.x * LA_WARPS + warp;
  if (unit >= (long long)n_tokens * H) return;
  const int t = (int)(unit / H), h = (int)(unit % H);
  const int p = tok_pos[t], b = tok_seq[t];
  const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
  float* qw = qs + (size_t)warp * W;
  const float* qp = q + (size_t)t * ldq + (size_t)h * W;
  for (int d = lane; d < W; d += 32) qw[d] = qp[d];
  __syncwarp();
  const int* pages = seq_pages + (size_t)b * pages_stride;

  float m = sink ? sink[h] : -INFINITY, l = sink ? 1.0f : 0.0f;
  float o[CH];
#pragma unroll
  for (int i = 0; i < CH; ++i) o[i] = 0.0f;

  for (int j0 = lo; j0 <= p; j0 += 32) {
    const int j = j0 + lane;
    float s = -INFINITY;
    if (j <= p) {
      const T* kr = cache + ((size_t)pages[j / page_size] * page_size + (j % page_size)) * (size_t)W;
      float dot = 0.0f;
      for (int d = 0; d < W; ++d) dot = fmaf(qw[d], to_f32(kr[d]), dot);
      s = dot;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float corr = expf(m - m_new);
    const float pj = (j <= p) ? expf(s - m_new) : 0.0f;
    l = l * corr + warp_sum(pj);
    m = m_new;
#pragma unroll
    for (int i = 0; i < CH; ++i) o[i] *= corr;
    const int nk = (p - j0 + 1 < 32) ? p - j0 + 1 : 32;
    for (int k = 0; k < nk; ++k) {
      const float pk = __shfl_sync(0xffffffffu, pj, k);
      const int jk = j0 + k;
      const T* vr = cache + ((size_t)pages[jk / page_size] * page_size + (jk % page_size)) * (size_t)W;
#pragma unroll
      for (int i = 0; i < CH; ++i) {
        const int d = lane + 32 * i;
        if (d < rank) o[i] = fmaf(pk, to_f32(vr[d]), o[i]);
      }
    }
  }
  const float inv = l > 0.0f ? 1.0f / l : 0.0f;
  float* op = out + (size_t)t * ldo + (size_t)h * rank;
#pragma unroll
  for (int i = 0; i < CH; ++i) {
    const int d = lane + 32 * i;
    if (d < rank) op[d] = o[i] * inv;
  }
}

extern "C" int hb_latent_attention(int dtype, const float* q, int ldq, float* out, int ldo, const void* cache,
                                   const float* sink, const int* tok_seq, const int* tok_pos, const int* seq_pages,
                                   int pages_stride, int n_tokens, int heads, int rank, int rot, int page_size, int window,
                                   void* stream) {
  HB_REQUIRE(n_tokens > 0 && heads > 0 && rank > 0 && rot >= 0 && page_size > 0 && window >= 0, "latent_attention: bad sizes");
  HB_REQUIRE(rank <= 1024, "latent_attention: latent size %d exceeds the supported maximum 1024", rank);
  const size_t smem = (size_t)LA_WARPS * (rank + rot) * sizeof(float);
  HB_REQUIRE(smem <= 48 * 1024, "latent_attention: rank + rot = %d exceeds what a block keeps in shared memory", rank + rot);
  const long long blocks = ceil_div_ll((long long)n_tokens * heads, LA_WARPS);
  HB_REQUIRE(blocks < 2147483647LL, "latent_attention: too many (token, head) pairs");
  cudaStream_t s = (cudaStream_t)stream;
#define LA_GO(T, CH)                                                                                                              \
  hb_launch(latent_attention_kernel<T, CH>, dim3((unsigned)blocks), dim3(LA_WARPS * 32), smem, s, q, ldq, out, ldo, (const T*)cache, \
            sink, tok_seq, tok_pos, seq_pages, pages_stride, n_tokens, heads, rank, rot, page_size, window)
  const int ch = ceil_div(rank, 32);
  if (dtype == HB_F32) {
    if (ch <= 2) LA_GO(float, 2); else if (ch <= 4) LA_GO(float, 4); else if (ch <= 8) LA_GO(float, 8);
    else if (ch <= 16) LA_GO(float, 16); else LA_GO(float, 32);
  } else {
    if (ch <= 2) LA_GO(bf16, 2); else if (ch <= 4) LA_GO(bf16, 4); else if (ch <= 8) LA_GO(bf16, 8);
    else if (ch <= 16) LA_GO(bf16, 16); else LA_GO(bf16, 32);
  }
#undef LA_GO
  HB_CHECK_LAUNCH("latent_attention");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// The same attention on the tensor cores (bfloat16 cache, mma.sync m16n8k16), flash form.  Since all
// heads share one cached vector per token, the rows of the score matrix are (token, head) pairs, head
// fastest: a CTA takes 32 consecutive pairs of one sequence (with 16 heads: two tokens; a decode step:
// all heads of the one token) against 64 keys at a time.
//   phase 1: S = Q K^T, 32 x 64 over W = rank + rot: warp w owns rows 16 (w & 1).., keys 8 (w >> 1)..
//   softmax: per-row maxima and sums meet in shared memory; P (bfloat16) goes to shared memory
//   phase 2: O += P C, 32 x rank: the key tile's first `rank` columns are the values; warp w owns the
//            16-column groups w, w + 16, ... of O for all 32 rows
// Key tiles go global -> shared with cp.async, two buffers; a row of a tile finds its own page, so any
// page size serves.  Masked scores never enter a maximum or a sum; the sink starts m and l.
#define LM_ROWS 32
#define LM_KEYS 64
#define LM_WARPS 16
#define LM_KG 8            // key groups of 8 keys per round of 64
#define LM_THREADS (LM_WARPS * 32)
#define LM_NEG (-1.0e30f)

struct LatentMmaArgs {
  const float* q;
  int ldq;
  float* out;
  int ldo;
  const bf16* cache;
  const float* sink;
  const int* seq_start;
  const int* seq_pos0;
  const int* seq_pages;
  int pages_stride;
  int H, rank, rot, page_size, window;
  int nsplit;      // key ranges per row tile; > 1: partial results go to `part` and a second kernel joins them
  float* part;     // [seq][row tile][split][32 rows][rank + 2]: unnormalised sums, then m and l
  int row_tiles;
};

template <int NPW>  // 16-column groups of O per warp: rank <= 256 * NPW
__global__ void __launch_bounds__(LM_THREADS) latent_attention_mma_kernel(LatentMmaArgs a) {
  extern __shared__ __align__(16) unsigned char smem[];
  pdl_wait();
  pdl_launch();
  const int W = a.rank + a.rot, rb = W * 2 + 16, pb = LM_KEYS * 2 + 16;
  unsigned char* qs = smem;
  unsigned char* kbuf = qs + LM_ROWS * rb;
  unsigned char* ps = kbuf + 2 * LM_KEYS * rb;
  float* smax = (float*)(ps + LM_ROWS * pb);   // [32][LM_KG]
  float* ssum = smax + LM_ROWS * LM_KG;        // [32][LM_KG]
  float* mrow = ssum + LM_ROWS * LM_KG;        // [32]
  float* lrow = mrow + LM_ROWS;                // [32]
  int* rowp = (int*)(lrow + LM_ROWS);          // [32] position of the row's token (-1: no row)
  int* rowlo = rowp + LM_ROWS;                 // [32] first key the row sees

  const int b = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int tok0 = a.seq_start[b], nrows = (a.seq_start[b + 1] - tok0) * a.H, r0 = blockIdx.x * LM_ROWS;
  if (r0 >= nrows) return;
  const int pos0 = a.seq_pos0[b];
  if (tid < LM_ROWS) {
    const int r = r0 + tid;
    const bool valid = r < nrows;
    const int p = valid ? pos0 + r / a.H : -1;
    rowp[tid] = p;
    rowlo[tid] = (valid && a.window > 0 && p - a.window + 1 > 0) ? p - a.window + 1 : 0;
    const bool sunk = valid && a.sink && blockIdx.z == 0;      // the sink counts once: in the first key range
    mrow[tid] = sunk ? a.sink[r % a.H] : LM_NEG;
    lrow[tid] = sunk ? 1.0f : 0.0f;
  }
  for (int rr = warp; rr < LM_ROWS; rr += LM_WARPS) {      // a row per warp and turn: no division per element
    const int r = r0 + rr;
    const float* src = r < nrows ? a.q + (size_t)(tok0 + r / a.H) * a.ldq + (size_t)(r % a.H) * W : nullptr;
    bf16* dst = (bf16*)(qs + rr * rb);
    for (int d = lane; d < W; d += 32) dst[d] = __float2bfloat16_rn(src ? src[d] : 0.0f);
  }
  __syncthreads();
  const int last = (nrows - r0 < LM_ROWS ? nrows - r0 : LM_ROWS) - 1;
  const int jmin = rowlo[0], jmax = rowp[last];
  const int k0 = (jmin / LM_KEYS) * LM_KEYS, ntiles = (jmax - k0) / LM_KEYS + 1;
  const int per_split = (ntiles + a.nsplit - 1) / a.nsplit;
  const int it0 = blockIdx.z * per_split, it1 = it0 + per_split < ntiles ? it0 + per_split : ntiles;
  const int* pages = a.seq_pages + (size_t)b * a.pages_stride;
  const int chunks = W >> 3;  // 16-byte pieces of a row

  const bool whole_pages = a.page_size % LM_KEYS == 0;     // then a tile of keys lies inside one page
  auto load_tile = [&](int it) {
    unsigned char* dst = kbuf + (it & 1) * LM_KEYS * rb;
    const int base = k0 + it * LM_KEYS;
    int pi0 = base / a.page_size;
    if (pi0 >= a.pages_stride) pi0 = a.pages_stride - 1;    // beyond the table: masked anyway
    const bf16* tile0 = a.cache + ((size_t)pages[pi0] * a.page_size + (base % a.page_size)) * (size_t)W;
    for (int kr = warp; kr < LM_KEYS; kr += LM_WARPS) {     // a key row per warp and turn
      const bf16* src = tile0 + (size_t)kr * W;
      if (!whole_pages) {
        const int j = base + kr;
        int pi = j / a.page_size;
        if (pi >= a.pages_stride) pi = a.pages_stride - 1;
        src = a.cache + ((size_t)pages[pi] * a.page_size + (j % a.page_size)) * (size_t)W;
      }
      for (int c = lane; c < chunks; c += 32) cp_async16(dst + kr * rb + c * 16, src + c * 8);
    }
    cp_async_commit();
  };

  float acc[2][NPW][2][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < NPW; ++j)
#pragma unroll
      for (int k = 0; k < 2; ++k)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[i][j][k][c] = 0.0f;
  const int npairs = a.rank >> 4;
  const int mt = warp & 1, kg = warp >> 1;
  auto row_max = [&](int r) {       // the row's maximum so far and over this round's key groups
    float m = mrow[r];
#pragma unroll
    for (int k = 0; k < LM_KG; ++k) m = fmaxf(m, smax[r * LM_KG + k]);
    return m;
  };

  if (it0 < it1) load_tile(it0);
  for (int it = it0; it < it1; ++it) {
    if (it + 1 < it1) {
      load_tile(it + 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const unsigned char* kt = kbuf + (it & 1) * LM_KEYS * rb;
    // ---- phase 1: scores of rows 16 mt.. against keys 8 kg..; four sets of partial sums over k, so that
    // four instructions per score tile are in flight, not one after the other
    float s[4], sp[4][4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int c = 0; c < 4; ++c) sp[u][c] = 0.0f;
    {
      const unsigned char* qa = qs + (mt * 16 + (lane & 15)) * rb + (lane >> 4) * 16;
      const unsigned char* kb = kt + (kg * 8 + (lane & 7)) * rb + (lane >> 3) * 16;   // one load: these 8 keys, 32 of k
      const int nks = W >> 4;
      int ks = 0;
      for (; ks + 4 <= nks; ks += 4) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          unsigned a0, a1, a2, a3, b0, b1, b2, b3;
          ldmatrix_x4(b0, b1, b2, b3, kb + (ks + 2 * u) * 32);
          ldmatrix_x4(a0, a1, a2, a3, qa + (ks + 2 * u) * 32);
          mma16816(sp[2 * u], a0, a1, a2, a3, b0, b1);
          ldmatrix_x4(a0, a1, a2, a3, qa + (ks + 2 * u + 1) * 32);
          mma16816(sp[2 * u + 1], a0, a1, a2, a3, b2, b3);
        }
      }
      for (; ks < nks; ++ks) {      // what is left, a step of 16 at a time (the load's upper half is not used)
        unsigned a0, a1, a2, a3, b0, b1, b2, b3;
        ldmatrix_x4(b0, b1, b2, b3, kb + ks * 32);
        ldmatrix_x4(a0, a1, a2, a3, qa + ks * 32);
        mma16816(sp[0], a0, a1, a2, a3, b0, b1);
      }
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) s[c] = (sp[0][c] + sp[1][c]) + (sp[2][c] + sp[3][c]);
    const int jb = k0 + it * LM_KEYS + kg * 8 + 2 * t;
    const int ra = mt * 16 + g, rbw = ra + 8;
    const int pa = rowp[ra], la = rowlo[ra], pbv = rowp[rbw], lb = rowlo[rbw];
    bool ok[4];
    float mxa = LM_NEG, mxb = LM_NEG;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int j = jb + (c & 1);
      const bool o = c < 2 ? (j >= la && j <= pa) : (j >= lb && j <= pbv);
      ok[c] = o;
      if (o) {
        if (c < 2) mxa = fmaxf(mxa, s[c]); else mxb = fmaxf(mxb, s[c]);
      }
    }
    mxa = fmaxf(mxa, __shfl_xor_sync(0xffffffffu, mxa, 1));
    mxa = fmaxf(mxa, __shfl_xor_sync(0xffffffffu, mxa, 2));
    mxb = fmaxf(mxb, __shfl_xor_sync(0xffffffffu, mxb, 1));
    mxb = fmaxf(mxb, __shfl_xor_sync(0xffffffffu, mxb, 2));
    if (t == 0) {
      smax[ra * LM_KG + kg] = mxa;
      smax[rbw * LM_KG + kg] = mxb;
    }
    __syncthreads();
    const float ma = row_max(ra), mb = row_max(rbw);
    float sa, sb;
    {
      const float p0 = ok[0] ? expf(s[0] - ma) : 0.0f, p1 = ok[1] ? expf(s[1] - ma) : 0.0f;
      const float p2 = ok[2] ? expf(s[2] - mb) : 0.0f, p3 = ok[3] ? expf(s[3] - mb) : 0.0f;
      // the sums take the rounded weights, the ones the product below uses
      const __nv_bfloat162 ua = __floats2bfloat162_rn(p0, p1), ub = __floats2bfloat162_rn(p2, p3);
      sa = __bfloat162float(ua.x) + __bfloat162float(ua.y);
      sb = __bfloat162float(ub.x) + __bfloat162float(ub.y);
      const int col = kg * 8 + 2 * t;
      *(__nv_bfloat162*)(ps + ra * pb + col * 2) = ua;
      *(__nv_bfloat162*)(ps + rbw * pb + col * 2) = ub;
    }
    sa += __shfl_xor_sync(0xffffffffu, sa, 1);
    sa += __shfl_xor_sync(0xffffffffu, sa, 2);
    sb += __shfl_xor_sync(0xffffffffu, sb, 1);
    sb += __shfl_xor_sync(0xffffffffu, sb, 2);
    if (t == 0) {
      ssum[ra * LM_KG + kg] = sa;
      ssum[rbw * LM_KG + kg] = sb;
    }
    __syncthreads();
    // ---- phase 2: O = O * corr + P C for this warp's column groups, both row tiles
#pragma unroll
    for (int m2 = 0; m2 < 2; ++m2) {
      const int r1 = m2 * 16 + g, r2 = r1 + 8;
      const float c1 = expf(mrow[r1] - row_max(r1)), c2 = expf(mrow[r2] - row_max(r2));
#pragma unroll
      for (int j = 0; j < NPW; ++j)
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          acc[m2][j][k][0] *= c1;
          acc[m2][j][k][1] *= c1;
          acc[m2][j][k][2] *= c2;
          acc[m2][j][k][3] *= c2;
        }
    }
#pragma unroll
    for (int kk = 0; kk < LM_KEYS / 16; ++kk) {
      unsigned pa0[4], pa1[4];
      ldmatrix_x4(pa0[0], pa0[1], pa0[2], pa0[3], ps + (lane & 15) * pb + kk * 32 + (lane >> 4) * 16);
      ldmatrix_x4(pa1[0], pa1[1], pa1[2], pa1[3], ps + (16 + (lane & 15)) * pb + kk * 32 + (lane >> 4) * 16);
      const unsigned char* vb = kt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * rb + (lane >> 4) * 16;
#pragma unroll
      for (int j = 0; j < NPW; ++j) {
        const int pair = warp + LM_WARPS * j;
        if (pair < npairs) {
          unsigned b0, b1, b2, b3;
          ldmatrix_x4_trans(b0, b1, b2, b3, vb + pair * 32);
          mma16816(acc[0][j][0], pa0[0], pa0[1], pa0[2], pa0[3], b0, b1);
          mma16816(acc[0][j][1], pa0[0], pa0[1], pa0[2], pa0[3], b2, b3);
          mma16816(acc[1][j][0], pa1[0], pa1[1], pa1[2], pa1[3], b0, b1);
          mma16816(acc[1][j][1], pa1[0], pa1[1], pa1[2], pa1[3], b2, b3);
        }
      }
    }
    __syncthreads();
    if (tid < LM_ROWS) {
      const float mo = mrow[tid], mn = row_max(tid);
      float sum = 0.0f;
#pragma unroll
      for (int k = 0; k < LM_KG; ++k) sum += ssum[tid * LM_KG + k];
      lrow[tid] = lrow[tid] * expf(mo - mn) + sum;
      mrow[tid] = mn;
    }
  }
  __syncthreads();
  float* pbase = a.nsplit > 1 ? a.part + ((((size_t)b * a.row_tiles + blockIdx.x) * a.nsplit + blockIdx.z) * LM_ROWS) * (size_t)(a.rank + 2)
                              : nullptr;
  if (pbase && tid < LM_ROWS) {
    pbase[(size_t)tid * (a.rank + 2) + a.rank] = mrow[tid];
    pbase[(size_t)tid * (a.rank + 2) + a.rank + 1] = lrow[tid];
  }
#pragma unroll
  for (int m2 = 0; m2 < 2; ++m2)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int rr = m2 * 16 + g + half * 8, r = r0 + rr;
      if (r >= nrows) continue;
      const float l = lrow[rr], inv = pbase ? 1.0f : (l > 0.0f ? 1.0f / l : 0.0f);
      float* op = pbase ? pbase + (size_t)rr * (a.rank + 2)
                        : a.out + (size_t)(tok0 + r / a.H) * a.ldo + (size_t)(r % a.H) * a.rank;
#pragma unroll
      for (int j = 0; j < NPW; ++j) {
        const int pair = warp + LM_WARPS * j;
        if (pair >= npairs) continue;
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const int col = pair * 16 + k * 8 + 2 * t;
          op[col] = acc[m2][j][k][half * 2] * inv;
          op[col + 1] = acc[m2][j][k][half * 2 + 1] * inv;
        }
      }
    }
}

// Joins the key ranges of a row: M = max m_s, out = sum_s e^{m_s - M} O_s / sum_s e^{m_s - M} l_s.  One CTA per
// row; its threads share the ranges' factors and take the row's columns side by side.
#define LJ_THREADS 128
__global__ void __launch_bounds__(LJ_THREADS)
latent_attention_join_kernel(const float* __restrict__ part, float* __restrict__ out, int ldo, const int* __restrict__ seq_start,
                             int H, int rank, int nsplit, int row_tiles) {
  __shared__ float f[64];
  pdl_wait();
  pdl_launch();
  const int b = blockIdx.y, rl = blockIdx.x;      // row within the sequence
  const int tok0 = seq_start[b], nrows = (seq_start[b + 1] - tok0) * H;
  if (rl >= nrows) return;
  const int tile = rl / LM_ROWS, rr = rl % LM_ROWS;
  const float* p0 = part + ((((size_t)b * row_tiles + tile) * nsplit) * LM_ROWS + rr) * (size_t)(rank + 2);
  const size_t step = (size_t)LM_ROWS * (rank + 2);
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    float m0 = lane < nsplit ? p0[lane * step + rank] : LM_NEG, m1 = lane + 32 < nsplit ? p0[(lane + 32) * step + rank] : LM_NEG;
    const float M = warp_max(fmaxf(m0, m1));
    const float e0 = lane < nsplit ? expf(m0 - M) : 0.0f, e1 = lane + 32 < nsplit ? expf(m1 - M) : 0.0f;
    float L = (lane < nsplit ? e0 * p0[lane * step + rank + 1] : 0.0f) + (lane + 32 < nsplit ? e1 * p0[(lane + 32) * step + rank + 1] : 0.0f);
    L = warp_sum(L);
    const float inv = L > 0.0f ? 1.0f / L : 0.0f;
    f[lane] = e0 * inv;
    f[lane + 32] = e1 * inv;
  }
  __syncthreads();
  float* op = out + (size_t)(tok0 + rl / H) * ldo + (size_t)(rl % H) * rank;
  for (int d = threadIdx.x; d < rank; d += LJ_THREADS) {
    float o = 0.0f;
    for (int s = 0; s < nsplit; ++s) o = fmaf(f[s], p0[s * step + d], o);
    op[d] = o;
  }
}

static size_t latent_mma_smem(int W) {
  const size_t rb = (size_t)W * 2 + 16;
  return (LM_ROWS + 2 * LM_KEYS) * rb + LM_ROWS * (LM_KEYS * 2 + 16) + LM_ROWS * (2 * LM_KG + 4) * sizeof(float);
}

// Whether the tensor-core kernel serves these sizes (else the any-shape kernel does).
extern "C" int hb_latent_attention_mma_ok(int rank, int rot) {
  return rank > 0 && rank % 16 == 0 && rot % 16 == 0 && rank <= 512 && latent_mma_smem(rank + rot) <= 220 * 1024;
}

// Floats of scratch that `nsplit` key ranges need.
extern "C" long long hb_latent_attention_mma_scratch_floats(int n_seqs, int max_q_len, int heads, int rank, int nsplit) {
  return (long long)n_seqs * ceil_div_ll((long long)max_q_len * heads, LM_ROWS) * nsplit * LM_ROWS * (rank + 2);
}

extern "C" int hb_latent_attention_mma_bf16(const float* q, int ldq, float* out, int ldo, const void* cache, const float* sink,
                                            const int* seq_start, const int* seq_pos0, const int* seq_pages, int pages_stride,
                                            int n_seqs, int max_q_len, int heads, int rank, int rot, int page_size, int window,
                                            int nsplit, float* scratch, void* stream) {
  HB_REQUIRE(n_seqs > 0 && max_q_len > 0 && heads > 0 && page_size > 0 && window >= 0 && pages_stride > 0, "latent_attention_mma: bad sizes");
  HB_REQUIRE(hb_latent_attention_mma_ok(rank, rot), "latent_attention_mma: rank %d and rot %d must be multiples of 16, rank at most 512", rank, rot);
  HB_REQUIRE(n_seqs <= 65535, "latent_attention_mma: at most 65535 sequences per step");
  HB_REQUIRE(nsplit >= 1 && nsplit <= 64 && (nsplit == 1 || scratch != nullptr), "latent_attention_mma: 1 to 64 key ranges, with scratch beyond one");
  const size_t smem = latent_mma_smem(rank + rot);
  const int row_tiles = (int)ceil_div_ll((long long)max_q_len * heads, LM_ROWS);
  LatentMmaArgs a{q, ldq, out, ldo, (const bf16*)cache, sink, seq_start, seq_pos0, seq_pages, pages_stride, heads, rank, rot, page_size, window,
                  nsplit, scratch, row_tiles};
  dim3 grid((unsigned)row_tiles, n_seqs, nsplit);
  cudaStream_t s = (cudaStream_t)stream;
#define LM_GO(NPW)                                                                                                     \
  do {                                                                                                                 \
    cudaFuncSetAttribute(latent_attention_mma_kernel<NPW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
    hb_launch(latent_attention_mma_kernel<NPW>, grid, dim3(LM_THREADS), smem, s, a);                                   \
  } while (0)
  if (rank <= 256) LM_GO(1); else LM_GO(2);
#undef LM_GO
  if (nsplit > 1)
    hb_launch(latent_attention_join_kernel, dim3(max_q_len * heads, n_seqs), dim3(LJ_THREADS), 0, s, (const float*)scratch, out, ldo,
              seq_start, heads, rank, nsplit, row_tiles);
  HB_CHECK_LAUNCH("latent_attention_mma");
  return 0;
}
