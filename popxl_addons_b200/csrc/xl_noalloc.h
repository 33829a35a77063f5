// Allocation-free entry point of libxlb200.so. It has no counterpart in the reference (popxl_addons); it exists for
// callers of this library that are not allowed to allocate device memory.
//
// Who cannot allocate: code that runs while a stream is being captured into a CUDA graph (cudaMalloc is illegal
// there), plug-ins that are handed a fixed memory budget by their host application, and services that pre-allocate
// everything at start-up and treat a later allocation as a fault. The regular entry point xl_grad_sumsq needs a scratch
// buffer for its per-block partial sums, which such a caller would have to provide; this one needs nothing but the
// input and the output.
//
//   int xl_grad_sumsq_noalloc(const void* x, int dtype, const float* scale, float* out, long long n, cudaStream_t s)
//
//   *out = (sum over the n elements of x of x_i^2) * (*scale if scale != NULL else 1), in fp32.
//   x      device pointer, dtype 0 = float, 1 = half, 2 = bfloat16
//   scale  device pointer to one float, or NULL
//   out    device pointer to one float
//   n      1 .. XL_NOALLOC_SUMSQ_MAX_ELEMS; larger inputs are refused with XL_NOALLOC_TOO_LARGE
//   Returns 0, a cudaError_t value, or one of the negative codes below. The work is enqueued on stream s.
//
// The partial sums go into a fixed array of XL_NOALLOC_SUMSQ_PARTS floats (1 KiB) that is part of the library image:
// every GPU that loads the library holds that array until the process exits. Consequences for the caller:
//   * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
//     current). Make that first call before any stream capture begins on the device.
//   * All calls on one device share the array. Two calls whose kernels can overlap on the GPU (different streams
//     without an ordering between them) race on it; calls ordered on one stream are safe, and a call never reads what
//     an earlier call left behind.
//   * The array that is used belongs to the device that is current when the call is made, so that device must be the
//     one stream s was created on (cudaSetDevice first in a multi-GPU process); the entry point does not check this,
//     and a stream of another device makes the launch fail or use the wrong device's array.
//   * The looked-up address is cached per device in plain host memory without a lock. Two host threads that make the
//     first call on a device at the same time both look it up and both store the same value, which is harmless.
//   * The entry point itself never calls cudaMalloc, cudaFree or any allocating library routine.
#pragma once
#include <cuda_runtime.h>

#define XL_NOALLOC_SUMSQ_PARTS 256
#define XL_NOALLOC_SUMSQ_MAX_ELEMS (1LL << 32)
#define XL_NOALLOC_MAX_DEVICES 64
#define XL_NOALLOC_BAD_ARGUMENT (-1)
#define XL_NOALLOC_TOO_LARGE (-2)

#ifdef __cplusplus
extern "C"
#endif
int xl_grad_sumsq_noalloc(const void* x, int dtype, const float* scale, float* out, long long n, cudaStream_t s);
