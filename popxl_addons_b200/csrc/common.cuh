// Shared device helpers for the sm_100a kernels of this package: dtype dispatch, 16-byte vector access, block
// reductions. Launchers are plain `extern "C"` functions taking raw device pointers and a stream, so the library has no
// dependency on torch headers and is loaded from Python with ctypes.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define XL_API extern "C" __attribute__((visibility("default")))

enum XlDtype : int { XL_F32 = 0, XL_F16 = 1, XL_BF16 = 2 };

template <typename T> struct XlVec;  // 16 bytes worth of T
template <> struct XlVec<float> { static constexpr int N = 4; };
template <> struct XlVec<__half> { static constexpr int N = 8; };
template <> struct XlVec<__nv_bfloat16> { static constexpr int N = 8; };

__device__ __forceinline__ float xl_to_float(float v) { return v; }
__device__ __forceinline__ float xl_to_float(__half v) { return __half2float(v); }
__device__ __forceinline__ float xl_to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T xl_from_float(float v);
template <> __device__ __forceinline__ float xl_from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __half xl_from_float<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 xl_from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// Load / store N = 16/sizeof(T) consecutive elements through one 128-bit access. `p` must be 16-byte aligned.
template <typename T> __device__ __forceinline__ void xl_load16(const T* __restrict__ p, float (&out)[XlVec<T>::N]) {
  constexpr int N = XlVec<T>::N;
  uint4 raw = *reinterpret_cast<const uint4*>(p);
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < N; ++i) out[i] = xl_to_float(e[i]);
}
template <typename T> __device__ __forceinline__ void xl_store16(T* __restrict__ p, const float (&in)[XlVec<T>::N]) {
  constexpr int N = XlVec<T>::N;
  uint4 raw;
  T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
  for (int i = 0; i < N; ++i) e[i] = xl_from_float<T>(in[i]);
  *reinterpret_cast<uint4*>(p) = raw;
}

__device__ __forceinline__ float xl_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float xl_warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Block-wide sum; `smem` holds >= 32 floats. All threads get the result.
__device__ __forceinline__ float xl_block_sum(float v, float* smem) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = xl_warp_sum(v);
  __syncthreads();
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  float r = (lane < nwarps) ? smem[lane] : 0.f;
  return xl_warp_sum(r);
}
__device__ __forceinline__ float xl_block_max(float v, float* smem) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = xl_warp_max(v);
  __syncthreads();
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  float r = (lane < nwarps) ? smem[lane] : -INFINITY;
  return xl_warp_max(r);
}

#define XL_DISPATCH_DTYPE(dtype, T, ...)                                     \
  switch (dtype) {                                                           \
    case XL_F32: { using T = float; __VA_ARGS__; break; }                    \
    case XL_F16: { using T = __half; __VA_ARGS__; break; }                   \
    case XL_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; }           \
    default: return (int)cudaErrorInvalidValue;                              \
  }

static inline int xl_grid_for(long long n_items, int per_block, int max_blocks = 148 * 16) {
  long long b = (n_items + per_block - 1) / per_block;
  if (b < 1) b = 1;
  if (b > max_blocks) b = max_blocks;
  return (int)b;
}
