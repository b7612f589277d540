// What lies between the q/k(/v) product and attention for a mixer that neither norms nor rotates its
// heads: the projections' biases, a query temperature that grows with the position, and the cache
// write.  The product's rows arrive as floats [q heads | k heads | v heads], so each number is
// rounded to the storage type once, after bias and temperature:
//   q[t, h, :] = (q + bq) * (1 + coef * ln(floor((p_t + 1) / every) + 1))     -> q_out, type T
//   k[t, g, :] = k + bk -> the key plane of the paged cache at the token's place
//   v[t, g, :] = v + bv -> the value plane, if the mixer has one (a mixer whose values are its keys
//                          keeps one plane and the row has no v part)
// One warp per (token, head) over all heads of the row.
#include "api.h"
#include "common.cuh"

struct QkPrepArgs {
  const float* qkv;
  int ld;
  const float* bias;   // [nh*hd + nkv*hd (+ nkv*hd)] in the row's layout, or null
  void* q_out;
  int ldq;
  float temp_coef;
  int temp_every;      // 0: no temperature
  const int* tok_seq;
  const int* tok_pos;
  const int* seq_pages;
  int pages_stride;
  void* kcache;
  void* vcache;        // null: the row has no v part
  int n_tokens, nh, nkv, hd, page_size, write_cache;
};

template <typename T>
__global__ void __launch_bounds__(128) qk_prepare_cache_kernel(QkPrepArgs a) {
  pdl_wait();
  pdl_launch();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = a.nh + a.nkv * (a.vcache ? 2 : 1);
  const long long unit = (long long)blockIdx.x * 4 + warp;
  if (unit >= (long long)a.n_tokens * heads) return;
  const int t = (int)(unit / heads), u = (int)(unit % heads);
  const int p = a.tok_pos[t];
  const float* src = a.qkv + (size_t)t * a.ld + (size_t)u * a.hd;
  const float* b = a.bias ? a.bias + (size_t)u * a.hd : nullptr;
  if (u < a.nh) {
    float f = 1.0f;
    if (a.temp_every > 0) f = 1.0f + a.temp_coef * logf((float)((p + 1) / a.temp_every + 1));
    T* dst = (T*)a.q_out + (size_t)t * a.ldq + (size_t)u * a.hd;
    for (int d = lane; d < a.hd; d += 32) dst[d] = from_f32<T>((src[d] + (b ? b[d] : 0.0f)) * f);
    return;
  }
  if (!a.write_cache) return;
  const int g = (u - a.nh) % a.nkv;
  T* plane = (T*)((u - a.nh) < a.nkv ? a.kcache : a.vcache);
  const int page = a.seq_pages[(size_t)a.tok_seq[t] * a.pages_stride + p / a.page_size];
  T* dst = plane + (((size_t)page * a.nkv + g) * a.page_size + (size_t)(p % a.page_size)) * a.hd;
  for (int d = lane; d < a.hd; d += 32) dst[d] = from_f32<T>(src[d] + (b ? b[d] : 0.0f));
}

extern "C" int hb_qk_prepare_cache(int dtype, const float* qkv, int ld, const float* bias, void* q_out, int ldq,
                                   float temp_coef, int temp_every, const int* tok_seq, const int* tok_pos,
                                   const int* seq_pages, int pages_stride, void* kcache, void* vcache, int n_tokens,
                                   int nh, int nkv, int hd, int page_size, int write_cache, void* stream) {
  HB_REQUIRE(n_tokens > 0 && nh > 0 && nkv > 0 && hd > 0 && page_size > 0, "qk_prepare_cache: sizes must be positive");
  HB_REQUIRE(temp_every >= 0, "qk_prepare_cache: the temperature's period must be >= 0");
  HB_REQUIRE(ld >= (nh + nkv * (vcache ? 2 : 1)) * hd && ldq >= nh * hd, "qk_prepare_cache: rows are shorter than their heads");
  QkPrepArgs a{qkv, ld, bias, q_out, ldq, temp_coef, temp_every, tok_seq, tok_pos, seq_pages, pages_stride, kcache, vcache,
               n_tokens, nh, nkv, hd, page_size, write_cache};
  const long long blocks = ceil_div_ll((long long)n_tokens * (nh + nkv * (vcache ? 2 : 1)), 4);
  HB_REQUIRE(blocks < 2147483647LL, "qk_prepare_cache: too many (token, head) pairs");
  if (dtype == HB_F32)
    hb_launch(qk_prepare_cache_kernel<float>, dim3((unsigned)blocks), dim3(128), 0, (cudaStream_t)stream, a);
  else
    hb_launch(qk_prepare_cache_kernel<bf16>, dim3((unsigned)blocks), dim3(128), 0, (cudaStream_t)stream, a);
  HB_CHECK_LAUNCH("qk_prepare_cache");
  return 0;
}
