// mlstm.cu — what surrounds the linear scan when it runs a stabilised matrix memory (the mLSTM of xLSTM):
//
//   m_t = max(f_t + m_(t-1), i_t)                     running maximum of the log gates, from 0
//   S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T        (n_t likewise, with k_t alone)
//   y_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
//
// The recurrence itself is mrs_seq_linear_scan with per-token decay and input scale; the normaliser n rides along as
// one more value column that is constantly 1.  Here: the gate kernel (soft cap, log-sigmoid, the running maximum as a
// scan over blocks of 32 tokens side by side, carried per sequence), the ones column, and the output stage (denominator, unit
// RMS per head, weight, sigmoid gate).  Everything is f32 except the value copy and the gate / output activations.
#include "seq_common.cuh"

namespace seq {

__device__ __forceinline__ float log_sigmoid_f(float z) { return fminf(z, 0.0f) - log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float soft_cap_f(float z, float cap) { return cap > 0.0f ? cap * tanhf(z / cap) : z; }

// One CTA of GATE_WARPS warps per (sequence, head); every warp takes a block of 32 tokens, GATE_WARPS blocks per round.
// Inside a block with inclusive prefix sums F of f:  m_l = F_l + max(m_start, max_{j <= l}(i_j - F_j)), which equals the
// token-by-token rule; a block's effect on the running maximum is the pair (F_31, max_j(i_j - F_j)), so the warps compute
// their blocks side by side and then fold the pairs of the blocks before theirs.  keep / take are formed from the m
// values actually stored, so they stay consistent with them whatever the rounding of the scan.
constexpr int GATE_WARPS = 8;
__global__ void __launch_bounds__(GATE_WARPS * 32) mlstm_gates_kernel(const float *__restrict__ raw_in, const float *__restrict__ raw_forget, int64_t raw_ld,
                                   float cap, int heads, float *__restrict__ m_state, const int32_t *__restrict__ cu_tok,
                                   const int32_t *__restrict__ past, const int32_t *__restrict__ slot, float *__restrict__ keep,
                                   float *__restrict__ take, float *__restrict__ m_tok) {
  __shared__ float tot_f[GATE_WARPS], top_g[GATE_WARPS];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const int b = blockIdx.x / heads, h = blockIdx.x % heads;
  const int t_begin = cu_tok[b], t_end = cu_tok[b + 1];
  if (t_end <= t_begin) return;
  float *ms = m_state + (int64_t)slot[b] * heads + h;
  float m_round = past[b] > 0 ? *ms : 0.0f;          // the running maximum before this round
  for (int r0 = t_begin; r0 < t_end; r0 += GATE_WARPS * 32) {
    const int t = r0 + wib * 32 + lane;
    const bool live = t < t_end;
    const float f = live ? log_sigmoid_f(soft_cap_f(raw_forget[(int64_t)t * raw_ld + h], cap)) : 0.0f;
    const float i = live ? soft_cap_f(raw_in[(int64_t)t * raw_ld + h], cap) : -INFINITY;
    float F = f;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const float o = __shfl_up_sync(0xffffffffu, F, d);
      if (lane >= d) F += o;
    }
    float G = i - F;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const float o = __shfl_up_sync(0xffffffffu, G, d);
      if (lane >= d) G = fmaxf(G, o);
    }
    if (lane == 31) { tot_f[wib] = F; top_g[wib] = G; }
    __syncthreads();
    float m_start = m_round;                          // fold the blocks before this warp's (a dead block: F = 0, G = -inf)
    for (int w = 0; w < wib; w++) m_start = tot_f[w] + fmaxf(m_start, top_g[w]);
    const float m = F + fmaxf(m_start, G);
    float before = __shfl_up_sync(0xffffffffu, m, 1);
    if (lane == 0) before = m_start;
    if (live) {
      const int64_t at = (int64_t)t * heads + h;
      keep[at] = expf(f + before - m);
      take[at] = expf(i - m);
      m_tok[at] = m;
    }
    for (int w = wib; w < GATE_WARPS; w++) m_start = tot_f[w] + fmaxf(m_start, top_g[w]);
    m_round = m_start;                                // every warp arrives at the same value
    __syncthreads();
  }
  if (threadIdx.x == 0) *ms = m_round;
}

template <typename T>
__global__ void append_ones_kernel(const T *__restrict__ v, int64_t v_ld, int heads, int dv, int dvp, T *__restrict__ vaug) {
  const int t = blockIdx.x, n = heads * dvp;
  for (int e = threadIdx.x; e < n; e += blockDim.x) {
    const int h = e / dvp, c = e % dvp;
    vaug[(int64_t)t * n + e] = c < dv ? v[(int64_t)t * v_ld + h * dv + c] : from_f32<T>(c == dv ? 1.0f : 0.0f);
  }
}

// one warp per (token, head)
template <typename T>
__global__ void mlstm_out_norm_kernel(const float *__restrict__ o, int dvp, const float *__restrict__ m_tok, float q_scale,
                                      const T *__restrict__ gate, int64_t gate_ld, const float *__restrict__ weight, float eps, int heads,
                                      int dv, T *__restrict__ out, int64_t out_ld, int n_tok) {
  const int lane = threadIdx.x & 31;
  const int64_t job = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (job >= (int64_t)n_tok * heads) return;
  const int t = (int)(job / heads), h = (int)(job % heads);
  const float *row = o + ((int64_t)t * heads + h) * dvp;
  const float den = fmaxf(fabsf(q_scale * row[dv]), expf(-m_tok[(int64_t)t * heads + h])) + 1e-6f;
  const float mul = q_scale / den;
  float ss = 0.0f;
  for (int c = lane; c < dv; c += 32) {
    const float y = row[c] * mul;
    ss = fmaf(y, y, ss);
  }
  const float inv = rsqrtf_exact(warp_sum(ss) / (float)dv + eps);
  const T *g = gate + (int64_t)t * gate_ld + h * dv;
  const float *w = weight + h * dv;
  T *dst = out + (int64_t)t * out_ld + h * dv;
  for (int c = lane; c < dv; c += 32) dst[c] = from_f32<T>(row[c] * mul * inv * w[c] * sigmoid_f(to_f32<T>(g[c])));
}

}  // namespace seq

using namespace seq;

extern "C" int mrs_seq_mlstm_gates(const float *raw_in, const float *raw_forget, int64_t raw_ld, float cap, int heads, float *m_state,
                                   const int32_t *cu_tok, const int32_t *past, const int32_t *slot, int n_seq, int n_tok, float *keep,
                                   float *take, float *m_tok, int64_t stream) {
  if (n_tok <= 0 || n_seq <= 0) return 0;
  if (heads <= 0 || !raw_in || !raw_forget || !m_state || !keep || !take || !m_tok) return -2;
  mlstm_gates_kernel<<<n_seq * heads, GATE_WARPS * 32, 0, (cudaStream_t)stream>>>(raw_in, raw_forget, raw_ld, cap, heads, m_state, cu_tok, past,
                                                                                  slot, keep, take, m_tok);
  return launch_status();
}

extern "C" int mrs_seq_append_ones(const void *v, int64_t v_ld, int dtype, int heads, int dv, int dvp, int n_tok, void *vaug,
                                   int64_t stream) {
  if (n_tok <= 0) return 0;
  if (heads <= 0 || dv <= 0 || dvp <= dv) return -2;
  SEQ_DISPATCH_DTYPE(dtype, (append_ones_kernel<T><<<n_tok, 256, 0, (cudaStream_t)stream>>>((const T *)v, v_ld, heads, dv, dvp, (T *)vaug)));
  return launch_status();
}

extern "C" int mrs_seq_mlstm_out_norm(const float *o, int dvp, const float *m_tok, float q_scale, const void *gate, int64_t gate_ld,
                                      const float *weight, float eps, int heads, int dv, void *out, int64_t out_ld, int dtype, int n_tok,
                                      int64_t stream) {
  if (n_tok <= 0) return 0;
  if (heads <= 0 || dv <= 0 || dvp <= dv) return -2;
  const int warps = 4;
  const int64_t jobs = (int64_t)n_tok * heads;
  SEQ_DISPATCH_DTYPE(dtype, (mlstm_out_norm_kernel<T><<<(unsigned)((jobs + warps - 1) / warps), warps * 32, 0, (cudaStream_t)stream>>>(
                                o, dvp, m_tok, q_scale, (const T *)gate, gate_ld, weight, eps, heads, dv, (T *)out, out_ld, n_tok)));
  return launch_status();
}
