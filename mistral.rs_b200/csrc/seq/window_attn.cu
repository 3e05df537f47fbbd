// window_attn.cu — softmax attention over a paged cache for layers whose scores carry no position signal: per-head
// RMS norm of queries and keys, a sliding window (or full causal reach), grouped key/value heads, and key / value
// head sizes that need not match.  The new tokens' keys and values are stored first; the attention kernel then reads
// every key of a query, old or new, from the pages — one code path for a prompt portion and for a decoded token.
#include "seq_common.cuh"

namespace seq {

// one warp per (token, head) for q; warps past the q heads take the k heads (norm + store) and the v heads (store)
template <typename T>
__global__ void qk_norm_store_kernel(T *__restrict__ q, int64_t q_ld, const T *__restrict__ k, int64_t k_ld, const T *__restrict__ v,
                                     int64_t v_ld, const float *__restrict__ q_norm_w, const float *__restrict__ k_norm_w,
                                     float eps, int heads, int kv_heads, int dk, int dv, T *__restrict__ k_cache,
                                     T *__restrict__ v_cache, const int64_t *__restrict__ slot_of_tok) {
  const int t = blockIdx.x, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int64_t slot = slot_of_tok[t];
  for (int job = threadIdx.x >> 5; job < heads + 2 * kv_heads; job += nw) {
    if (job < heads + kv_heads) {
      const bool is_q = job < heads;
      const int hh = is_q ? job : job - heads;
      const T *src = is_q ? q + (int64_t)t * q_ld + hh * dk : k + (int64_t)t * k_ld + hh * dk;
      const float *w = is_q ? q_norm_w : k_norm_w;
      float ss = 0.0f;
      for (int d = lane; d < dk; d += 32) {
        const float x = to_f32<T>(src[d]);
        ss = fmaf(x, x, ss);
      }
      const float inv = w ? rsqrtf_exact(warp_sum(ss) / (float)dk + eps) : 1.0f;
      T *dst = is_q ? q + (int64_t)t * q_ld + hh * dk : (slot >= 0 ? k_cache + (slot * kv_heads + hh) * dk : nullptr);
      if (dst)
        for (int d = lane; d < dk; d += 32) dst[d] = from_f32<T>(w ? to_f32<T>(src[d]) * inv * w[d] : to_f32<T>(src[d]));
    } else if (slot >= 0) {
      const int hh = job - heads - kv_heads;
      const T *src = v + (int64_t)t * v_ld + hh * dv;
      T *dst = v_cache + (slot * kv_heads + hh) * dv;
      for (int d = lane; d < dv; d += 32) dst[d] = src[d];
    }
  }
}

// One warp per (token, head).  32 keys per round: lane j scores key j against the whole query (held in shared
// memory as f32, pre-scaled), the round's maximum and sum go through the warp, then every lane accumulates its
// value columns over the round's keys.  Softmax statistics and the output accumulate in f32.
template <typename T, int MAX_VCOLS>   // MAX_VCOLS * 32 >= value head size
__global__ void __launch_bounds__(128) window_attention_kernel(const T *__restrict__ q, int64_t q_ld, const T *__restrict__ k_cache,
                                                               const T *__restrict__ v_cache, int heads, int kv_heads, int dk, int dv,
                                                               float scale, int window, const int32_t *__restrict__ pages,
                                                               int pages_ld, int page_size, const int32_t *__restrict__ seq_of_tok,
                                                               const int32_t *__restrict__ pos_of_tok, int n_tok, T *__restrict__ out,
                                                               int64_t out_ld, float out_scale) {
  extern __shared__ __align__(16) float qsm[];   // [warps][dk]
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const int64_t job = (int64_t)blockIdx.x * (blockDim.x >> 5) + wib;
  if (job >= (int64_t)n_tok * heads) return;
  const int t = (int)(job / heads), h = (int)(job % heads), g = h / (heads / kv_heads);
  const int s = seq_of_tok[t], pos = pos_of_tok[t];
  float *qv = qsm + wib * dk;
  for (int d = lane; d < dk; d += 32) qv[d] = to_f32<T>(q[(int64_t)t * q_ld + h * dk + d]) * scale;
  __syncwarp();
  const int32_t *table = pages + (int64_t)s * pages_ld;
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  float m = -INFINITY, l = 0.0f, acc[MAX_VCOLS];
#pragma unroll
  for (int c = 0; c < MAX_VCOLS; c++) acc[c] = 0.0f;
  for (int j0 = lo; j0 <= pos; j0 += 32) {
    const int j = j0 + lane;
    float sc = -INFINITY;
    int64_t slot = 0;
    if (j <= pos) {
      slot = (int64_t)table[j / page_size] * page_size + j % page_size;
      const T *kr = k_cache + (slot * kv_heads + g) * dk;
      float a0 = 0.0f, a1 = 0.0f;
      int d = 0;
      for (; d + 1 < dk; d += 2) {
        a0 = fmaf(qv[d], to_f32<T>(kr[d]), a0);
        a1 = fmaf(qv[d + 1], to_f32<T>(kr[d + 1]), a1);
      }
      if (d < dk) a0 = fmaf(qv[d], to_f32<T>(kr[d]), a0);
      sc = a0 + a1;
    }
    const float m_new = fmaxf(m, warp_max(sc));      // the round always holds key j0 <= pos: m_new is finite
    const float p = j <= pos ? expf(sc - m_new) : 0.0f;
    const float corr = expf(m - m_new);               // exp(-inf) = 0 on the first round
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int c = 0; c < MAX_VCOLS; c++) acc[c] *= corr;
    const int n = min(32, pos - j0 + 1);
    for (int i = 0; i < n; i++) {
      const float pi = __shfl_sync(0xffffffffu, p, i);
      const int64_t si = __shfl_sync(0xffffffffu, slot, i);
      const T *vr = v_cache + (si * kv_heads + g) * dv;
#pragma unroll
      for (int c = 0; c < MAX_VCOLS; c++)
        if (c * 32 + lane < dv) acc[c] = fmaf(pi, to_f32<T>(vr[c * 32 + lane]), acc[c]);
    }
    m = m_new;
  }
  const float inv = out_scale / l;
#pragma unroll
  for (int c = 0; c < MAX_VCOLS; c++)
    if (c * 32 + lane < dv) out[(int64_t)t * out_ld + h * dv + c * 32 + lane] = from_f32<T>(acc[c] * inv);
}

}  // namespace seq

using namespace seq;

extern "C" int mrs_seq_qk_norm_store(void *q, int64_t q_ld, const void *k, int64_t k_ld, const void *v, int64_t v_ld, int dtype,
                                     const float *q_norm_w, const float *k_norm_w, float eps, int heads, int kv_heads, int dk, int dv,
                                     void *k_cache, void *v_cache, const int64_t *slot_of_tok, int n_tok, int64_t stream) {
  if (n_tok <= 0) return 0;
  const int jobs = heads + 2 * kv_heads, warps = jobs < 8 ? jobs : 8;
  SEQ_DISPATCH_DTYPE(dtype, (qk_norm_store_kernel<T><<<n_tok, warps * 32, 0, (cudaStream_t)stream>>>(
                                (T *)q, q_ld, (const T *)k, k_ld, (const T *)v, v_ld, q_norm_w, k_norm_w, eps, heads, kv_heads, dk, dv,
                                (T *)k_cache, (T *)v_cache, slot_of_tok)));
  return launch_status();
}

extern "C" int mrs_seq_window_attention(const void *q, int64_t q_ld, const void *k_cache, const void *v_cache, int dtype, int heads,
                                        int kv_heads, int dk, int dv, float scale, int window, const int32_t *pages, int pages_ld,
                                        int page_size, const int32_t *seq_of_tok, const int32_t *pos_of_tok, int n_tok, void *out,
                                        int64_t out_ld, float out_scale, int64_t stream) {
  if (n_tok <= 0) return 0;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || dv > 512 || dk > 1024) return -2;
  const int warps = 4;
  const int64_t jobs = (int64_t)n_tok * heads;
#define SEQ_ATTN_LAUNCH(VC)                                                                                              \
  window_attention_kernel<T, VC><<<(unsigned)((jobs + warps - 1) / warps), warps * 32, warps * dk * sizeof(float),          \
                                   (cudaStream_t)stream>>>((const T *)q, q_ld, (const T *)k_cache, (const T *)v_cache, heads, \
                                                           kv_heads, dk, dv, scale, window, pages, pages_ld, page_size,      \
                                                           seq_of_tok, pos_of_tok, n_tok, (T *)out, out_ld, out_scale)
  SEQ_DISPATCH_DTYPE(dtype, {
    if (dv <= 64) SEQ_ATTN_LAUNCH(2);
    else if (dv <= 128) SEQ_ATTN_LAUNCH(4);
    else if (dv <= 256) SEQ_ATTN_LAUNCH(8);
    else SEQ_ATTN_LAUNCH(16);
  });
#undef SEQ_ATTN_LAUNCH
  return launch_status();
}
