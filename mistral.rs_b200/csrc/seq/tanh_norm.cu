// tanh_norm.cu — a single f32 residual whose norms are Dynamic Tanh (tanh(alpha z) * weight + bias: no mean, no
// variance, so no reduction and no row-wide dependency).  A layer with a norm before AND after each sublayer becomes
// one elementwise pass per sublayer: add the normed sublayer output to the residual, optionally add a second f32
// tensor (the embedding output re-entering before a repeated pass over a range of layers), and produce the next
// sublayer's normed input.  The residual never leaves f32.
#include "seq_common.cuh"

namespace seq {

template <typename T, int VEC>
__global__ void __launch_bounds__(256) tanh_norm_rows_kernel(const float *__restrict__ x, const int32_t *__restrict__ rows,
                                                             const float *__restrict__ alpha, const float *__restrict__ weight,
                                                             const float *__restrict__ bias, T *__restrict__ out, int width) {
  const int r = blockIdx.x, t = rows ? rows[r] : r;
  const float a = *alpha;
  const float *src = x + (int64_t)t * width;
  T *dst = out + (int64_t)r * width;
  for (int c = (blockIdx.y * blockDim.x + threadIdx.x) * VEC; c < width; c += gridDim.y * blockDim.x * VEC) {
    if (VEC == 4) {
      const float4 v = *(const float4 *)(src + c), w = *(const float4 *)(weight + c), b = *(const float4 *)(bias + c);
      store4<T>(dst + c, make_float4(fmaf(tanhf(a * v.x), w.x, b.x), fmaf(tanhf(a * v.y), w.y, b.y), fmaf(tanhf(a * v.z), w.z, b.z),
                                     fmaf(tanhf(a * v.w), w.w, b.w)));
    } else {
      dst[c] = from_f32<T>(fmaf(tanhf(a * src[c]), weight[c], bias[c]));
    }
  }
}

template <typename T, int VEC>
__global__ void __launch_bounds__(256) residual_tanh_norm_kernel(float *__restrict__ x, const T *__restrict__ y,
                                                                 const float *__restrict__ post_alpha, const float *__restrict__ post_w,
                                                                 const float *__restrict__ post_b, const float *__restrict__ extra,
                                                                 const float *__restrict__ next_alpha, const float *__restrict__ next_w,
                                                                 const float *__restrict__ next_b, T *__restrict__ next_out, int width) {
  const int t = blockIdx.x;
  const float pa = y ? *post_alpha : 0.0f, na = next_out ? *next_alpha : 0.0f;
  float *xr = x + (int64_t)t * width;
  for (int c = (blockIdx.y * blockDim.x + threadIdx.x) * VEC; c < width; c += gridDim.y * blockDim.x * VEC) {
    float v[VEC];
    if (VEC == 4) { const float4 q = *(const float4 *)(xr + c); v[0] = q.x; v[1 % VEC] = q.y; v[2 % VEC] = q.z; v[3 % VEC] = q.w; }
    else v[0] = xr[c];
    if (y) {
      float yv[VEC];
      if (VEC == 4) { const float4 q = load4<T>(y + (int64_t)t * width + c); yv[0] = q.x; yv[1 % VEC] = q.y; yv[2 % VEC] = q.z; yv[3 % VEC] = q.w; }
      else yv[0] = to_f32<T>(y[(int64_t)t * width + c]);
#pragma unroll
      for (int e = 0; e < VEC; e++) v[e] += fmaf(tanhf(pa * yv[e]), post_w[c + e], post_b[c + e]);
    }
    if (extra) {
#pragma unroll
      for (int e = 0; e < VEC; e++) v[e] += extra[(int64_t)t * width + c + e];
    }
    if (y || extra) {
      if (VEC == 4) *(float4 *)(xr + c) = make_float4(v[0], v[1 % VEC], v[2 % VEC], v[3 % VEC]);
      else xr[c] = v[0];
    }
    if (next_out) {
      float o[VEC];
#pragma unroll
      for (int e = 0; e < VEC; e++) o[e] = fmaf(tanhf(na * v[e]), next_w[c + e], next_b[c + e]);
      if (VEC == 4) store4<T>(next_out + (int64_t)t * width + c, make_float4(o[0], o[1 % VEC], o[2 % VEC], o[3 % VEC]));
      else next_out[(int64_t)t * width + c] = from_f32<T>(o[0]);
    }
  }
}

static inline bool aligned16(const void *p) { return ((uintptr_t)p & 15) == 0; }

}  // namespace seq

using namespace seq;

extern "C" int mrs_seq_tanh_norm_rows(const float *x, const int32_t *rows, const float *alpha, const float *weight, const float *bias,
                                      void *out, int dtype, int n_rows, int width, int64_t stream) {
  if (n_rows <= 0 || width <= 0) return 0;
  if (!x || !alpha || !weight || !bias || !out) return -2;
  const bool vec = width % 4 == 0 && aligned16(x) && aligned16(weight) && aligned16(bias) && aligned16(out);
  const int per = vec ? 1024 : 256, by = (width + per - 1) / per;
  const dim3 grid(n_rows, by < 32 ? by : 32);
  SEQ_DISPATCH_DTYPE(dtype, {
    if (vec) tanh_norm_rows_kernel<T, 4><<<grid, 256, 0, (cudaStream_t)stream>>>(x, rows, alpha, weight, bias, (T *)out, width);
    else tanh_norm_rows_kernel<T, 1><<<grid, 256, 0, (cudaStream_t)stream>>>(x, rows, alpha, weight, bias, (T *)out, width);
  });
  return launch_status();
}

extern "C" int mrs_seq_residual_tanh_norm(float *x, const void *y, int dtype, const float *post_alpha, const float *post_weight,
                                          const float *post_bias, const float *extra, const float *next_alpha, const float *next_weight,
                                          const float *next_bias, void *next_out, int n_tok, int width, int64_t stream) {
  if (n_tok <= 0 || width <= 0) return 0;
  if (!x || (y && (!post_alpha || !post_weight || !post_bias)) || (next_out && (!next_alpha || !next_weight || !next_bias))) return -2;
  const bool vec = width % 4 == 0 && aligned16(x) && aligned16(y) && aligned16(extra) && aligned16(next_out) && aligned16(post_weight) &&
                   aligned16(post_bias) && aligned16(next_weight) && aligned16(next_bias);
  const int per = vec ? 1024 : 256, by = (width + per - 1) / per;
  const dim3 grid(n_tok, by < 32 ? by : 32);
  SEQ_DISPATCH_DTYPE(dtype, {
    if (vec)
      residual_tanh_norm_kernel<T, 4><<<grid, 256, 0, (cudaStream_t)stream>>>(x, (const T *)y, post_alpha, post_weight, post_bias, extra,
                                                                             next_alpha, next_weight, next_bias, (T *)next_out, width);
    else
      residual_tanh_norm_kernel<T, 1><<<grid, 256, 0, (cudaStream_t)stream>>>(x, (const T *)y, post_alpha, post_weight, post_bias, extra,
                                                                             next_alpha, next_weight, next_bias, (T *)next_out, width);
  });
  return launch_status();
}
