// Smaller device ops of the add-on layer:
//   xl_pow2_cast_to_fp8 / xl_pow2_cast_from_fp8   power-of-two scaled casts between 16/32-bit floats and e4m3 / e5m2
//   xl_fp8_mse_scale                              power-of-two scale that minimises the squared quantisation error
//   xl_dense_csr_matmul                           dense x constant CSR matrix
//   xl_gather_rows / xl_scatter_add_rows          embedding lookup (rows out of range give zeros) and its gradient
//   xl_row_stats / xl_ce_shard_*                  row statistics of hidden-sharded LayerNorm and vocabulary-sharded
//                                                 cross-entropy (the pieces between the small all-reduces)
#include "common.cuh"

#include <cuda_fp8.h>
#include <math.h>

// ------------------------------------------------------------------------------------------------------------------
// FP8 casts. log2_scale is a device scalar (int32 or fp32); y = saturate(x * 2^s) in the 8-bit format, and back.
// ------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float load_log2(const void* p, int is_int) {
  return is_int ? (float)(*(const int*)p) : *(const float*)p;
}

template <typename T>
__global__ void __launch_bounds__(256)
    pow2_cast_to_fp8_kernel(const T* __restrict__ x, const void* __restrict__ log2_scale, int log2_is_int,
                            uint8_t* __restrict__ y, long long n, int e5m2) {
  const float s = exp2f(load_log2(log2_scale, log2_is_int));
  const __nv_fp8_interpretation_t fmt = e5m2 ? __NV_E5M2 : __NV_E4M3;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    y[i] = (uint8_t)__nv_cvt_float_to_fp8(xl_to_float(x[i]) * s, __NV_SATFINITE, fmt);
}

template <typename T>
__global__ void __launch_bounds__(256)
    pow2_cast_from_fp8_kernel(const uint8_t* __restrict__ x, const void* __restrict__ log2_scale, int log2_is_int,
                              T* __restrict__ y, long long n, int e5m2) {
  const float s = exp2f(load_log2(log2_scale, log2_is_int));
  const __nv_fp8_interpretation_t fmt = e5m2 ? __NV_E5M2 : __NV_E4M3;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)x[i], fmt);
    y[i] = xl_from_float<T>(__half2float(__half(h)) * s);
  }
}

XL_API int xl_pow2_cast_to_fp8(const void* x, int dtype, const void* log2_scale, int log2_is_int, void* y, long long n,
                               int e5m2, cudaStream_t s) {
  const int grid = xl_grid_for(n, 256 * 4);
  XL_DISPATCH_DTYPE(dtype, T, {
    pow2_cast_to_fp8_kernel<T><<<grid, 256, 0, s>>>((const T*)x, log2_scale, log2_is_int, (uint8_t*)y, n, e5m2);
  });
  return (int)cudaGetLastError();
}

XL_API int xl_pow2_cast_from_fp8(const void* x, const void* log2_scale, int log2_is_int, void* y, int dtype, long long n,
                                 int e5m2, cudaStream_t s) {
  const int grid = xl_grid_for(n, 256 * 4);
  XL_DISPATCH_DTYPE(dtype, T, {
    pow2_cast_from_fp8_kernel<T><<<grid, 256, 0, s>>>((const uint8_t*)x, log2_scale, log2_is_int, (T*)y, n, e5m2);
  });
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------------------------
// Best power-of-two scale for an 8-bit format by squared error (the algorithm of ops/fp8_mse_scale.py):
// histogram of |x| over the 254 octaves of normal fp32 numbers (shared-memory atomics, then global atomics); the last
// block to finish evaluates the 62 candidate shifts in double precision, writes the result and leaves the scratch
// (254 counters + ticket) zeroed.
// ------------------------------------------------------------------------------------------------------------------
constexpr int MSE_BINS = 254;
constexpr int MSE_CANDIDATES = 62;

template <typename T>
__global__ void __launch_bounds__(256)
    fp8_mse_scale_kernel(const T* __restrict__ x, long long n, unsigned int* __restrict__ scratch, int lo, int span,
                         double qerr, int* __restrict__ out) {
  __shared__ unsigned int hist[MSE_BINS];
  __shared__ double cost[MSE_CANDIDATES];
  __shared__ unsigned int last;
  for (int i = threadIdx.x; i < MSE_BINS; i += blockDim.x) hist[i] = 0;
  __syncthreads();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const unsigned int e = (__float_as_uint(fabsf(xl_to_float(x[i]))) >> 23) & 0xFFu;  // biased exponent
    if (e >= 1 && e <= 254) atomicAdd(&hist[e - 1], 1u);  // zeros and subnormals are not counted; inf / nan ignored
  }
  __syncthreads();
  for (int i = threadIdx.x; i < MSE_BINS; i += blockDim.x)
    if (hist[i]) atomicAdd(&scratch[i], hist[i]);
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) last = atomicAdd(&scratch[MSE_BINS], 1u) == gridDim.x - 1;
  __syncthreads();
  if (!last) return;
  __threadfence();
  if (threadIdx.x < MSE_CANDIDATES) {
    const int c = threadIdx.x;
    const int first = lo - 31 + 126;  // bin of the lowest covered octave for the first candidate shift (-31)
    const int start = first + c, stop = first + c + span;
    const int top_bin = min(max(stop - 1, 0), MSE_BINS - 1);
    const double top = exp2((double)(top_bin - 126));
    const double inv_n = 1.0 / (double)(n > 0 ? n : 1);
    double acc_under = 0.0, acc_in = 0.0, acc_over = 0.0;
    for (int b = 0; b < MSE_BINS; ++b) {
      const double h = (double)__ldcg(&scratch[b]) * inv_n;
      const double v = exp2((double)(b - 126));
      if (b < start) { if (b >= 1) acc_under += h * v * v; }
      else if (b < stop) acc_in += h * v * v * qerr;
      else acc_over += h * (v - top) * (v - top);
    }
    cost[c] = acc_under + acc_in + acc_over;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    double best = cost[0];
    int arg = 0;
    for (int c = 1; c < MSE_CANDIDATES; ++c)
      if (cost[c] < best) { best = cost[c]; arg = c; }
    int ties = 0;
    for (int c = 0; c < MSE_CANDIDATES; ++c) ties += cost[c] == best;
    *out = -(arg + ties / 2 - 31);
  }
  __syncthreads();
  for (int i = threadIdx.x; i <= MSE_BINS; i += blockDim.x) scratch[i] = 0;
}

// scratch: 255 zero-initialised words (left zeroed). lo / span: lowest octave covered by the format and the number of
// octaves it covers; qerr = 2^(-2 * (source mantissa bits - format mantissa bits)).
XL_API int xl_fp8_mse_scale(const void* x, int dtype, long long n, unsigned int* scratch, int lo, int span, double qerr,
                            int* out, cudaStream_t s) {
  const int grid = xl_grid_for(n, 256 * 8, 148 * 4);
  XL_DISPATCH_DTYPE(dtype, T, {
    fp8_mse_scale_kernel<T><<<grid, 256, 0, s>>>((const T*)x, n, scratch, lo, span, qerr, out);
  });
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------------------------
// y (M, N) = x (M, K) @ S, S a constant K x N matrix in CSR form (indptr K+1, indices, values). One CTA per output row:
// the row is accumulated in shared memory (fp32); threads walk the non-zeros, the CSR row of a non-zero is found by
// bisection of indptr. N * 4 bytes must fit in 48 KB of shared memory.
// ------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
    dense_csr_matmul_kernel(const T* __restrict__ x, const int* __restrict__ indptr, const int* __restrict__ indices,
                            const float* __restrict__ values, T* __restrict__ y, int K, int N, int nnz) {
  extern __shared__ float acc[];
  const int m = blockIdx.x;
  for (int i = threadIdx.x; i < N; i += blockDim.x) acc[i] = 0.f;
  __syncthreads();
  const T* xr = x + (long long)m * K;
  for (int idx = threadIdx.x; idx < nnz; idx += blockDim.x) {
    int lo = 0, hi = K;  // largest k with indptr[k] <= idx
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (indptr[mid] <= idx) lo = mid;
      else hi = mid;
    }
    atomicAdd(&acc[indices[idx]], xl_to_float(xr[lo]) * values[idx]);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < N; i += blockDim.x) y[(long long)m * N + i] = xl_from_float<T>(acc[i]);
}

XL_API int xl_dense_csr_matmul(const void* x, int dtype, const int* indptr, const int* indices, const float* values, void* y,
                               int M, int K, int N, int nnz, cudaStream_t s) {
  if (M < 1 || N < 1 || (long long)N * 4 > 48 * 1024) return -1;
  XL_DISPATCH_DTYPE(dtype, T, {
    dense_csr_matmul_kernel<T><<<M, 256, N * 4, s>>>((const T*)x, indptr, indices, values, (T*)y, K, N, nnz);
  });
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------------------------
// Embedding lookup on a vocabulary shard: out[i, :] = table[idx[i], :] if 0 <= idx[i] < rows else 0 (zero_oor), and the
// gradient scatter-add into an fp32 or 16-bit table gradient. cols % 8 == 0 for the vector path of 16-bit tables.
// ------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
    gather_rows_kernel(const T* __restrict__ table, const int* __restrict__ idx, T* __restrict__ out, long long n_idx,
                       int rows, int cols) {
  const long long i = blockIdx.x;
  if (i >= n_idx) return;
  const int r = idx[i];
  const bool ok = r >= 0 && r < rows;
  const T* src = table + (long long)(ok ? r : 0) * cols;
  T* dst = out + i * cols;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) dst[c] = ok ? src[c] : xl_from_float<T>(0.f);
}

template <typename T, typename G>
__global__ void __launch_bounds__(256)
    scatter_add_rows_kernel(const G* __restrict__ grad_out, const int* __restrict__ idx, T* __restrict__ grad_table,
                            long long n_idx, int rows, int cols) {
  const long long i = blockIdx.x;
  if (i >= n_idx) return;
  const int r = idx[i];
  if (r < 0 || r >= rows) return;
  const G* src = grad_out + i * cols;
  T* dst = grad_table + (long long)r * cols;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) atomicAdd(dst + c, (T)xl_to_float(src[c]));
}

XL_API int xl_gather_rows(const void* table, int dtype, const int* idx, void* out, long long n_idx, int rows, int cols,
                          cudaStream_t s) {
  if (n_idx < 1) return 0;
  XL_DISPATCH_DTYPE(dtype, T, {
    gather_rows_kernel<T><<<(unsigned)n_idx, 256, 0, s>>>((const T*)table, idx, (T*)out, n_idx, rows, cols);
  });
  return (int)cudaGetLastError();
}

// grad_table: fp32 (rows, cols), accumulated into (not zeroed here); grad_out: (n_idx, cols) of dtype.
XL_API int xl_scatter_add_rows(const void* grad_out, int dtype, const int* idx, float* grad_table, long long n_idx, int rows,
                               int cols, cudaStream_t s) {
  if (n_idx < 1) return 0;
  XL_DISPATCH_DTYPE(dtype, G, {
    scatter_add_rows_kernel<float, G><<<(unsigned)n_idx, 256, 0, s>>>((const G*)grad_out, idx, grad_table, n_idx, rows,
                                                                      cols);
  });
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------------------------
// Row statistics for ops whose rows are sharded over ranks: per row (sum, sum of squares) for the hidden-sharded
// LayerNorm's forward pass (its backward pass and the vocabulary-sharded cross-entropy are in sharded_ops.cu). The tiny
// per-row results are all-reduced by the caller between the kernels. One CTA per row.
// ------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float block_sum_256(float v, float* red) {
  v = xl_warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < 8; ++i) t += red[i];
  return t;
}
__device__ __forceinline__ float block_max_256(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = -INFINITY;
  for (int i = 0; i < 8; ++i) t = fmaxf(t, red[i]);
  return t;
}

// stats: (2, rows) fp32 = [sum | sum of squares]
template <typename T>
__global__ void __launch_bounds__(256) row_sum_sumsq_kernel(const T* __restrict__ x, float* __restrict__ stats, int rows, int cols) {
  __shared__ float red[8];
  const int r = blockIdx.x;
  float s = 0.f, q = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    const float v = xl_to_float(x[(long long)r * cols + c]);
    s += v;
    q += v * v;
  }
  s = block_sum_256(s, red);
  q = block_sum_256(q, red);
  if (threadIdx.x == 0) { stats[r] = s; stats[rows + r] = q; }
}

// y = (x - mean) * rstd * w + b with mean / rstd from the all-reduced stats over `hidden` = full width
template <typename T>
__global__ void __launch_bounds__(256)
    ln_apply_stats_kernel(const T* __restrict__ x, const float* __restrict__ stats, const T* __restrict__ w,
                          const T* __restrict__ b, T* __restrict__ y, float* __restrict__ mean_out,
                          float* __restrict__ rstd_out, int rows, int cols, float hidden, float eps) {
  const int r = blockIdx.x;
  const float mean = stats[r] / hidden;
  const float var = fmaxf(stats[rows + r] / hidden - mean * mean, 0.f);
  const float rstd = rsqrtf(var + eps);
  if (threadIdx.x == 0) { mean_out[r] = mean; rstd_out[r] = rstd; }
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    const float v = (xl_to_float(x[(long long)r * cols + c]) - mean) * rstd;
    y[(long long)r * cols + c] = xl_from_float<T>(v * xl_to_float(w[c]) + xl_to_float(b[c]));
  }
}

XL_API int xl_row_sum_sumsq(const void* x, int dtype, float* stats, int rows, int cols, cudaStream_t s) {
  XL_DISPATCH_DTYPE(dtype, T, { row_sum_sumsq_kernel<T><<<rows, 256, 0, s>>>((const T*)x, stats, rows, cols); });
  return (int)cudaGetLastError();
}
XL_API int xl_ln_apply_stats(const void* x, int dtype, const float* stats, const void* w, const void* b, void* y,
                             float* mean_out, float* rstd_out, int rows, int cols, float hidden, float eps,
                             cudaStream_t s) {
  XL_DISPATCH_DTYPE(dtype, T, {
    ln_apply_stats_kernel<T><<<rows, 256, 0, s>>>((const T*)x, stats, (const T*)w, (const T*)b, (T*)y, mean_out, rstd_out,
                                                 rows, cols, hidden, eps);
  });
  return (int)cudaGetLastError();
}
