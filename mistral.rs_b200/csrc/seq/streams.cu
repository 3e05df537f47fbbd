// streams.cu — multi-stream residual (hyper-connections): the model keeps `n_streams` f32 copies of the residual per
// token.  A sublayer reads a weighted sum of them (fused here with its RMS norm) and writes back a mix of the old
// streams plus its scaled output (fused with the NEXT sublayer's read + norm, the way add + RMSNorm are one kernel in
// the single-stream decoder).  One CTA per token; the streams never leave f32.
#include "seq_common.cuh"

namespace seq {

constexpr int MAX_STREAMS = 16;

template <typename T>
__global__ void embed_streams_kernel(const T *__restrict__ table, const int32_t *__restrict__ ids, float *__restrict__ streams,
                                     int n_streams, int width) {
  const int t = blockIdx.x;
  const T *row = table + (int64_t)ids[t] * width;
  float *dst = streams + (int64_t)t * n_streams * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = to_f32<T>(row[c]);
    for (int s = 0; s < n_streams; s++) dst[(int64_t)s * width + c] = v;
  }
}

// NS: the stream count as a compile-time constant (1..4, loops fully unrolled) or 0 for any count up to MAX_STREAMS.
template <int NS> struct StreamCount {
  static constexpr int CAP = NS ? NS : MAX_STREAMS;
  static __device__ __forceinline__ int n(int runtime) { return NS ? NS : runtime; }
};

// u = sum_s w_in[s] x_s ; out = u / sqrt(mean(u^2) + eps) * (unit_offset + w)
template <typename T, int NS>
__global__ void __launch_bounds__(1024) streams_read_norm_kernel(const float *__restrict__ streams, const float *__restrict__ w_in,
                                         const float *__restrict__ norm_w, float eps, float unit_offset,
                                         const int32_t *__restrict__ rows, T *__restrict__ out, int n_streams, int width) {
  __shared__ float red[33];
  const int ns = StreamCount<NS>::n(n_streams);
  const int r = blockIdx.x;
  const int t = rows ? rows[r] : r;
  const float *src = streams + (int64_t)t * ns * width;
  float win[StreamCount<NS>::CAP];
#pragma unroll
  for (int s = 0; s < StreamCount<NS>::CAP; s++) win[s] = s < ns ? (w_in ? w_in[s] : 1.0f) : 0.0f;
  float ss = 0.0f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float u = 0.0f;
#pragma unroll
    for (int s = 0; s < StreamCount<NS>::CAP; s++)
      if (s < ns) u = fmaf(win[s], src[(int64_t)s * width + c], u);
    ss = fmaf(u, u, ss);
  }
  const float inv = rsqrtf_exact(block_sum(ss, red) / (float)width + eps);
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float u = 0.0f;
#pragma unroll
    for (int s = 0; s < StreamCount<NS>::CAP; s++)
      if (s < ns) u = fmaf(win[s], src[(int64_t)s * width + c], u);
    out[(int64_t)r * width + c] = from_f32<T>(u * inv * (unit_offset + norm_w[c]));
  }
}

// x_r <- sum_s mix[s][r] x_s + w_out[r] y, every r from the old x; then (optionally) the next read + norm.
// VEC = 4: four neighbouring columns per thread (16-byte stream accesses) when the width allows; VEC = 1 otherwise.
template <typename T, int VEC, int NS>
__global__ void __launch_bounds__(1024) streams_write_kernel(float *__restrict__ streams, const float *__restrict__ w_mix, const float *__restrict__ w_out,
                                     const T *__restrict__ y, int n_streams, int width, const float *__restrict__ next_in,
                                     const float *__restrict__ next_norm_w, float eps, float unit_offset, T *__restrict__ next_out) {
  constexpr int CAP = StreamCount<NS>::CAP;
  __shared__ float red[33];
  __shared__ float mix[MAX_STREAMS * MAX_STREAMS], wout[MAX_STREAMS], nin[MAX_STREAMS];
  const int ns = StreamCount<NS>::n(n_streams);
  const int t = blockIdx.x;
  for (int e = threadIdx.x; e < ns * ns; e += blockDim.x) mix[e] = w_mix[e];
  if (threadIdx.x < ns) {
    wout[threadIdx.x] = w_out[threadIdx.x];
    nin[threadIdx.x] = next_in ? next_in[threadIdx.x] : 0.0f;
  }
  __syncthreads();
  float *x = streams + (int64_t)t * ns * width;
  float ss = 0.0f;
  for (int c = threadIdx.x * VEC; c < width; c += blockDim.x * VEC) {
    float old[CAP][VEC], yv[VEC], u[VEC];
#pragma unroll
    for (int s = 0; s < CAP; s++)
      if (s < ns) {
        if (VEC == 4) { const float4 v = *(const float4 *)(x + (int64_t)s * width + c); old[s][0] = v.x; old[s][1 % VEC] = v.y; old[s][2 % VEC] = v.z; old[s][3 % VEC] = v.w; }
        else old[s][0] = x[(int64_t)s * width + c];
      }
    if (VEC == 4) { const float4 v = load4<T>(y + (int64_t)t * width + c); yv[0] = v.x; yv[1 % VEC] = v.y; yv[2 % VEC] = v.z; yv[3 % VEC] = v.w; }
    else yv[0] = to_f32<T>(y[(int64_t)t * width + c]);
#pragma unroll
    for (int e = 0; e < VEC; e++) u[e] = 0.0f;
#pragma unroll
    for (int r = 0; r < CAP; r++) {
      if (r < ns) {
        float acc[VEC];
#pragma unroll
        for (int e = 0; e < VEC; e++) {
          acc[e] = wout[r] * yv[e];
#pragma unroll
          for (int s = 0; s < CAP; s++)
            if (s < ns) acc[e] = fmaf(mix[s * ns + r], old[s][e], acc[e]);
          u[e] = fmaf(nin[r], acc[e], u[e]);
        }
        if (VEC == 4) *(float4 *)(x + (int64_t)r * width + c) = make_float4(acc[0], acc[1 % VEC], acc[2 % VEC], acc[3 % VEC]);
        else x[(int64_t)r * width + c] = acc[0];
      }
    }
#pragma unroll
    for (int e = 0; e < VEC; e++) ss = fmaf(u[e], u[e], ss);
  }
  if (next_out == nullptr) return;
  const float inv = rsqrtf_exact(block_sum(ss, red) / (float)width + eps);
  for (int c = threadIdx.x * VEC; c < width; c += blockDim.x * VEC) {   // the thread re-reads the columns it wrote itself
    float u[VEC];
#pragma unroll
    for (int e = 0; e < VEC; e++) u[e] = 0.0f;
#pragma unroll
    for (int r = 0; r < CAP; r++)
      if (r < ns) {
#pragma unroll
        for (int e = 0; e < VEC; e++) u[e] = fmaf(nin[r], x[(int64_t)r * width + c + e], u[e]);
      }
    if (VEC == 4) {
      const float4 w = *(const float4 *)(next_norm_w + c);
      store4<T>(next_out + (int64_t)t * width + c, make_float4(u[0] * inv * (unit_offset + w.x), u[1 % VEC] * inv * (unit_offset + w.y),
                                                               u[2 % VEC] * inv * (unit_offset + w.z), u[3 % VEC] * inv * (unit_offset + w.w)));
    } else {
      next_out[(int64_t)t * width + c] = from_f32<T>(u[0] * inv * (unit_offset + next_norm_w[c]));
    }
  }
}

static int threads_for(int width, int n_rows = 1 << 30) {
  if (n_rows <= 64) return width >= 1024 ? 1024 : (width >= 512 ? 512 : (width >= 256 ? 256 : (width >= 128 ? 128 : 64)));   // short batches: latency, not occupancy
  return width >= 1024 ? 256 : (width >= 256 ? 128 : 64);
}

}  // namespace seq

using namespace seq;

extern "C" int mrs_seq_embed_streams(const void *table, int dtype, const int32_t *ids, float *streams, int n_tok, int n_streams,
                                     int width, int64_t stream) {
  if (n_tok <= 0) return 0;
  if (n_streams < 1 || n_streams > MAX_STREAMS) return -2;
  SEQ_DISPATCH_DTYPE(dtype, (embed_streams_kernel<T><<<n_tok, threads_for(width), 0, (cudaStream_t)stream>>>(
                                (const T *)table, ids, streams, n_streams, width)));
  return launch_status();
}

extern "C" int mrs_seq_streams_read_norm(const float *streams, const float *w_in, const float *norm_w, float eps, float unit_offset,
                                         const int32_t *rows, void *out, int dtype, int n_rows, int n_streams, int width,
                                         int64_t stream) {
  if (n_rows <= 0) return 0;
  if (n_streams < 1 || n_streams > MAX_STREAMS) return -2;
#define SEQ_READ(NS) streams_read_norm_kernel<T, NS><<<n_rows, threads_for(width, n_rows), 0, (cudaStream_t)stream>>>( \
      streams, w_in, norm_w, eps, unit_offset, rows, (T *)out, n_streams, width)
  SEQ_DISPATCH_DTYPE(dtype, {
    switch (n_streams) {
      case 1: SEQ_READ(1); break;
      case 2: SEQ_READ(2); break;
      case 3: SEQ_READ(3); break;
      case 4: SEQ_READ(4); break;
      default: SEQ_READ(0);
    }
  });
#undef SEQ_READ
  return launch_status();
}

extern "C" int mrs_seq_streams_write(float *streams, const float *w_mix, const float *w_out, const void *y, int dtype, int n_tok,
                                     int n_streams, int width, const float *next_in, const float *next_norm_w, float eps,
                                     float unit_offset, void *next_out, int64_t stream) {
  if (n_tok <= 0) return 0;
  if (n_streams < 1 || n_streams > MAX_STREAMS) return -2;
  const bool vec = width % 4 == 0 && (uintptr_t)streams % 16 == 0 && (uintptr_t)y % 16 == 0 && (uintptr_t)next_out % 16 == 0 &&
                   (uintptr_t)next_norm_w % 16 == 0;
  int th = vec ? (width >= 4096 ? 256 : (width >= 512 ? 128 : 64)) : threads_for(width);
  if (n_tok <= 64) {   // short batches: one vector item per thread where possible
    const int items = vec ? width / 4 : width;
    while (th < 1024 && th < items) th *= 2;
  }
#define SEQ_WRITE(V, NS) streams_write_kernel<T, V, NS><<<n_tok, th, 0, (cudaStream_t)stream>>>( \
      streams, w_mix, w_out, (const T *)y, n_streams, width, next_in, next_norm_w, eps, unit_offset, (T *)next_out)
  SEQ_DISPATCH_DTYPE(dtype, {
    if (vec) {
      switch (n_streams) {
        case 1: SEQ_WRITE(4, 1); break;
        case 2: SEQ_WRITE(4, 2); break;
        case 3: SEQ_WRITE(4, 3); break;
        case 4: SEQ_WRITE(4, 4); break;
        default: SEQ_WRITE(1, 0);
      }
    } else {
      switch (n_streams) {
        case 1: SEQ_WRITE(1, 1); break;
        case 2: SEQ_WRITE(1, 2); break;
        case 3: SEQ_WRITE(1, 3); break;
        case 4: SEQ_WRITE(1, 4); break;
        default: SEQ_WRITE(1, 0);
      }
    }
  });
#undef SEQ_WRITE
  return launch_status();
}
