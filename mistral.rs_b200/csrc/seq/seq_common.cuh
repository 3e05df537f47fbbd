// seq_common.cuh — helpers shared by the sequence-mixer kernels (libmrs_b200_seq.so): activation storage
// types (bf16 or f32, picked by the dtype code of the C ABI), exact f32 activations, block reductions and the
// per-step batch description.  Everything that the kernels accumulate, normalise or carry from token to token is
// f32; only tensors that a matrix product reads or writes take the activation type.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../../include/mrs_b200_seq.h"

namespace seq {

// ---- storage types ----------------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// ---- exact activations (no fast-math intrinsics: the f32 mode is held to f32 rounding) ----------------
__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
__device__ __forceinline__ float rsqrtf_exact(float x) { return 1.0f / sqrtf(x); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.0f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float apply_act(float z, int act) {
  switch (act) {
    case MRS_SEQ_ACT_SILU: return silu_f(z);
    case MRS_SEQ_ACT_GELU_TANH: return gelu_tanh_f(z);
    case MRS_SEQ_ACT_SIGMOID: return sigmoid_f(z);
    default: return z;
  }
}

// ---- reductions -------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) x += __shfl_xor_sync(0xffffffffu, x, m);
  return x;
}
__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, m));
  return x;
}
// sum over the block; `red` is 33 floats of shared memory; every thread gets the result
__device__ __forceinline__ float block_sum(float x, float *red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  x = warp_sum(x);
  __syncthreads();   // `red` may still be read from an earlier call
  if (lane == 0) red[w] = x;
  __syncthreads();
  if (w == 0) {
    float y = lane < nw ? red[lane] : 0.0f;
    y = warp_sum(y);
    if (lane == 0) red[32] = y;
  }
  __syncthreads();
  return red[32];
}

// launch helper: a C-ABI function returns the CUDA error of its launches as an int (0 = ok)
inline int launch_status() { return (int)cudaGetLastError(); }

}  // namespace seq

#define SEQ_DISPATCH_DTYPE(dtype, ...)                                    \
  do {                                                                    \
    if ((dtype) == MRS_SEQ_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
    else if ((dtype) == MRS_SEQ_F32) { using T = float; __VA_ARGS__; }     \
    else return -1;                                                       \
  } while (0)
