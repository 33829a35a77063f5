// Memory-bound kernels: activations, normalisation, optimizer steps, rotary embedding, int4 group de-quantisation,
// softmax for attention, fused cross-entropy. All are single-pass over HBM with 128-bit accesses, fp32 arithmetic in
// registers; grids are sized as multiples of the 148 SMs for grid-stride kernels or one CTA per row for row kernels.
#include "common.cuh"

#include <math.h>

// ------------------------------------------------------------------------------------------------------------------
// generic 1-/2-/3-operand elementwise driver
// ------------------------------------------------------------------------------------------------------------------
constexpr int EW_UNROLL = 4;  // 16-byte vectors per thread and iteration: keeps ~64 B per thread in flight

template <typename T, typename F>
__global__ void __launch_bounds__(256) ew_unary_kernel(const T* __restrict__ x, T* __restrict__ y, long long n, F f) {
  constexpr int N = XlVec<T>::N;
  const long long nvec = n / N;
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  for (; i + (EW_UNROLL - 1) * stride < nvec; i += EW_UNROLL * stride) {
    float a[EW_UNROLL][N];
#pragma unroll
    for (int u = 0; u < EW_UNROLL; ++u) xl_load16(x + (i + u * stride) * N, a[u]);
#pragma unroll
    for (int u = 0; u < EW_UNROLL; ++u) {
#pragma unroll
      for (int k = 0; k < N; ++k) a[u][k] = f(a[u][k]);
      xl_store16(y + (i + u * stride) * N, a[u]);
    }
  }
  for (; i < nvec; i += stride) {
    float a[N];
    xl_load16(x + i * N, a);
#pragma unroll
    for (int k = 0; k < N; ++k) a[k] = f(a[k]);
    xl_store16(y + i * N, a);
  }
  for (long long j = nvec * N + blockIdx.x * (long long)blockDim.x + threadIdx.x; j < n; j += stride)
    y[j] = xl_from_float<T>(f(xl_to_float(x[j])));
}

template <typename T, typename F>
__global__ void __launch_bounds__(256)
    ew_binary_kernel(const T* __restrict__ x, const T* __restrict__ g, T* __restrict__ y, long long n, F f) {
  constexpr int N = XlVec<T>::N;
  const long long nvec = n / N;
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  for (; i + (EW_UNROLL - 1) * stride < nvec; i += EW_UNROLL * stride) {
    float a[EW_UNROLL][N], b[EW_UNROLL][N];
#pragma unroll
    for (int u = 0; u < EW_UNROLL; ++u) {
      xl_load16(x + (i + u * stride) * N, a[u]);
      xl_load16(g + (i + u * stride) * N, b[u]);
    }
#pragma unroll
    for (int u = 0; u < EW_UNROLL; ++u) {
#pragma unroll
      for (int k = 0; k < N; ++k) a[u][k] = f(a[u][k], b[u][k]);
      xl_store16(y + (i + u * stride) * N, a[u]);
    }
  }
  for (; i < nvec; i += stride) {
    float a[N], b[N];
    xl_load16(x + i * N, a);
    xl_load16(g + i * N, b);
#pragma unroll
    for (int k = 0; k < N; ++k) a[k] = f(a[k], b[k]);
    xl_store16(y + i * N, a);
  }
  for (long long j = nvec * N + blockIdx.x * (long long)blockDim.x + threadIdx.x; j < n; j += stride)
    y[j] = xl_from_float<T>(f(xl_to_float(x[j]), xl_to_float(g[j])));
}

// ---- GELU ---------------------------------------------------------------------------------------------------------
// erf by the Abramowitz-Stegun 7.1.26 rational approximation (|error| < 1.5e-7): ~10 instructions instead of ~30 for
// erff, which otherwise makes the 16-bit GELU kernels compute-bound instead of bandwidth-bound.
__device__ __forceinline__ float xl_fast_erf(float x) {
  const float ax = fabsf(x);
  const float t = __fdividef(1.f, fmaf(0.3275911f, ax, 1.f));
  const float poly = t * fmaf(t, fmaf(t, fmaf(t, fmaf(t, 1.061405429f, -1.453152027f), 1.421413741f), -0.284496736f), 0.254829592f);
  const float r = 1.f - poly * __expf(-ax * ax);
  return copysignf(r, x);
}
struct GeluErf {
  __device__ __forceinline__ float operator()(float x) const { return 0.5f * x * (1.f + erff(x * 0.70710678118654752f)); }
};
struct GeluErfFast {
  __device__ __forceinline__ float operator()(float x) const { return 0.5f * x * (1.f + xl_fast_erf(x * 0.70710678118654752f)); }
};
struct GeluErfGradFast {
  __device__ __forceinline__ float operator()(float x, float g) const {
    const float cdf = 0.5f * (1.f + xl_fast_erf(x * 0.70710678118654752f));
    const float pdf = 0.3989422804014327f * __expf(-0.5f * x * x);
    return g * (cdf + x * pdf);
  }
};
struct GeluTanh {
  __device__ __forceinline__ float operator()(float x) const {
    const float k = 0.7978845608028654f;
    return 0.5f * x * (1.f + tanhf(k * (x + 0.044715f * x * x * x)));
  }
};
struct GeluErfGrad {
  __device__ __forceinline__ float operator()(float x, float g) const {
    const float cdf = 0.5f * (1.f + erff(x * 0.70710678118654752f));
    const float pdf = 0.3989422804014327f * __expf(-0.5f * x * x);
    return g * (cdf + x * pdf);
  }
};
struct GeluTanhGrad {
  __device__ __forceinline__ float operator()(float x, float g) const {
    const float k = 0.7978845608028654f;
    const float t = tanhf(k * (x + 0.044715f * x * x * x));
    return g * (0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * k * (1.f + 3.f * 0.044715f * x * x));
  }
};
struct SiluGrad {
  __device__ __forceinline__ float operator()(float x, float g) const {
    const float s = 1.f / (1.f + __expf(-x));
    return g * s * (1.f + x * (1.f - s));
  }
};
struct Silu {
  __device__ __forceinline__ float operator()(float x) const { return x / (1.f + __expf(-x)); }
};
struct SwiGlu {
  __device__ __forceinline__ float operator()(float gate, float up) const { return gate / (1.f + __expf(-gate)) * up; }
};

XL_API int xl_gelu_fwd(const void* x, void* y, long long n, int dtype, int tanh_approx, cudaStream_t s) {
  const int grid = xl_grid_for(n, 256 * 8);
  XL_DISPATCH_DTYPE(dtype, T, {
    if (tanh_approx) ew_unary_kernel<T><<<grid, 256, 0, s>>>((const T*)x, (T*)y, n, GeluTanh());
    else if (sizeof(T) == 2) ew_unary_kernel<T><<<grid, 256, 0, s>>>((const T*)x, (T*)y, n, GeluErfFast());
    else ew_unary_kernel<T><<<grid, 256, 0, s>>>((const T*)x, (T*)y, n, GeluErf());
  });
  return (int)cudaGetLastError();
}
XL_API int xl_gelu_bwd(const void* x, const void* g, void* dx, long long n, int dtype, int tanh_approx, cudaStream_t s) {
  const int grid = xl_grid_for(n, 256 * 8);
  XL_DISPATCH_DTYPE(dtype, T, {
    if (tanh_approx) ew_binary_kernel<T><<<grid, 256, 0, s>>>((const T*)x, (const T*)g, (T*)dx, n, GeluTanhGrad());
    else if (sizeof(T) == 2) ew_binary_kernel<T><<<grid, 256, 0, s>>>((const T*)x, (const T*)g, (T*)dx, n, GeluErfGradFast());
    else ew_binary_kernel<T><<<grid, 256, 0, s>>>((const T*)x, (const T*)g, (T*)dx, n, GeluErfGrad());
  });
  return (int)cudaGetLastError();
}
XL_API int xl_silu_fwd(const void* x, void* y, long long n, int dtype, cudaStream_t s) {
  const int grid = xl_grid_for(n, 256 * 8);
  XL_DISPATCH_DTYPE(dtype, T, { ew_unary_kernel<T><<<grid, 256, 0, s>>>((const T*)x, (T*)y, n, Silu()); });
  return (int)cudaGetLastError();
}
XL_API int xl_silu_bwd(const void* x, const void* g, void* dx, long long n, int dtype, cudaStream_t s) {
  const int grid = xl_grid_for(n, 256 * 8);
  XL_DISPATCH_DTYPE(dtype, T, { ew_binary_kernel<T><<<grid, 256, 0, s>>>((const T*)x, (const T*)g, (T*)dx, n, SiluGrad()); });
  return (int)cudaGetLastError();
}
XL_API int xl_swiglu_fwd(const void* gate, const void* up, void* y, long long n, int dtype, cudaStream_t s) {
  const int grid = xl_grid_for(n, 256 * 8);
  XL_DISPATCH_DTYPE(dtype, T, { ew_binary_kernel<T><<<grid, 256, 0, s>>>((const T*)gate, (const T*)up, (T*)y, n, SwiGlu()); });
  return (int)cudaGetLastError();
}

template <typename T>
__global__ void __launch_bounds__(256) swiglu_bwd_kernel(const T* __restrict__ gate, const T* __restrict__ up,
                                                        const T* __restrict__ g, T* __restrict__ dgate,
                                                        T* __restrict__ dup, long long n) {
  constexpr int N = XlVec<T>::N;
  const long long nvec = n / N;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float a[N], u[N], d[N], da[N], du[N];
    xl_load16(gate + i * N, a);
    xl_load16(up + i * N, u);
    xl_load16(g + i * N, d);
#pragma unroll
    for (int k = 0; k < N; ++k) {
      const float sg = 1.f / (1.f + __expf(-a[k]));
      da[k] = d[k] * u[k] * sg * (1.f + a[k] * (1.f - sg));
      du[k] = d[k] * a[k] * sg;
    }
    xl_store16(dgate + i * N, da);
    xl_store16(dup + i * N, du);
  }
  for (long long i = nvec * N + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float a = xl_to_float(gate[i]), u = xl_to_float(up[i]), d = xl_to_float(g[i]);
    const float sg = 1.f / (1.f + __expf(-a));
    dgate[i] = xl_from_float<T>(d * u * sg * (1.f + a * (1.f - sg)));
    dup[i] = xl_from_float<T>(d * a * sg);
  }
}
XL_API int xl_swiglu_bwd(const void* gate, const void* up, const void* g, void* dgate, void* dup, long long n,
                         int dtype, cudaStream_t s) {
  const int grid = xl_grid_for(n, 256 * 8);
  XL_DISPATCH_DTYPE(dtype, T, {
    swiglu_bwd_kernel<T><<<grid, 256, 0, s>>>((const T*)gate, (const T*)up, (const T*)g, (T*)dgate, (T*)dup, n);
  });
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------------------------
// LayerNorm / RMSNorm. One CTA per row, the row lives in registers (cols <= 256 threads * 8 iters * vec width).
// ------------------------------------------------------------------------------------------------------------------
constexpr int NORM_THREADS = 256;
constexpr int NORM_MAX_ITERS = 8;

template <typename T, bool RMS, int ITERS>
__global__ void __launch_bounds__(NORM_THREADS)
    norm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ b, T* __restrict__ y,
                    float* __restrict__ mean_out, float* __restrict__ rstd_out, int cols, float eps) {
  constexpr int N = XlVec<T>::N;
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const T* xr = x + row * cols;
  T* yr = y + row * cols;
  const int nvec = cols / N;
  float v[ITERS][N];
  float sum = 0.f;
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int i = threadIdx.x + it * NORM_THREADS;
    if (i < nvec) {
      xl_load16(xr + i * N, v[it]);
#pragma unroll
      for (int k = 0; k < N; ++k) sum += RMS ? v[it][k] * v[it][k] : v[it][k];
    }
  }
  float mean = 0.f, rstd;
  if (RMS) {
    const float ms = xl_block_sum(sum, red) / cols;
    rstd = rsqrtf(ms + eps);
  } else {
    mean = xl_block_sum(sum, red) / cols;
    float sq = 0.f;
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      const int i = threadIdx.x + it * NORM_THREADS;
      if (i < nvec) {
#pragma unroll
        for (int k = 0; k < N; ++k) { const float d = v[it][k] - mean; sq += d * d; }
      }
    }
    const float var = xl_block_sum(sq, red) / cols;
    rstd = rsqrtf(var + eps);
  }
  if (threadIdx.x == 0) {
    if (!RMS) mean_out[row] = mean;
    rstd_out[row] = rstd;
  }
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int i = threadIdx.x + it * NORM_THREADS;
    if (i < nvec) {
      float ww[N], bb[N], o[N];
      xl_load16(w + i * N, ww);
      if (!RMS) xl_load16(b + i * N, bb);
#pragma unroll
      for (int k = 0; k < N; ++k) o[k] = RMS ? v[it][k] * rstd * ww[k] : (v[it][k] - mean) * rstd * ww[k] + bb[k];
      xl_store16(yr + i * N, o);
    }
  }
}

// Smallest register tiling (vectors per thread) that covers a row, or 0 if the row is too long / not vectorisable.
static inline int norm_iters(int cols, int dtype, int max_iters) {
  const int n = dtype == XL_F32 ? 4 : 8;
  if (cols % n != 0) return 0;
  const int nvec = cols / n;
  for (int it = 1; it <= max_iters; it *= 2)
    if (nvec <= NORM_THREADS * it) return it;
  return 0;
}
#define XL_DISPATCH_ITERS(iters, IT, ...)                 \
  switch (iters) {                                        \
    case 1: { constexpr int IT = 1; __VA_ARGS__; break; } \
    case 2: { constexpr int IT = 2; __VA_ARGS__; break; } \
    case 4: { constexpr int IT = 4; __VA_ARGS__; break; } \
    case 8: { constexpr int IT = 8; __VA_ARGS__; break; } \
    default: return -1;                                   \
  }

XL_API int xl_layer_norm_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd,
                             long long rows, int cols, float eps, int dtype, cudaStream_t s) {
  const int iters = norm_iters(cols, dtype, NORM_MAX_ITERS);
  if (!iters) return -1;
  XL_DISPATCH_DTYPE(dtype, T, XL_DISPATCH_ITERS(iters, IT, {
    norm_fwd_kernel<T, false, IT><<<(unsigned)rows, NORM_THREADS, 0, s>>>((const T*)x, (const T*)w, (const T*)b, (T*)y,
                                                                           mean, rstd, cols, eps);
  }));
  return (int)cudaGetLastError();
}
XL_API int xl_rms_norm_fwd(const void* x, const void* w, void* y, float* rstd, long long rows, int cols, float eps,
                           int dtype, cudaStream_t s) {
  const int iters = norm_iters(cols, dtype, NORM_MAX_ITERS);
  if (!iters) return -1;
  XL_DISPATCH_DTYPE(dtype, T, XL_DISPATCH_ITERS(iters, IT, {
    norm_fwd_kernel<T, true, IT><<<(unsigned)rows, NORM_THREADS, 0, s>>>((const T*)x, (const T*)w, nullptr, (T*)y,
                                                                          nullptr, rstd, cols, eps);
  }));
  return (int)cudaGetLastError();
}

// Backward: each CTA walks rows blockIdx.x, +gridDim.x, ...; dx is written per row, the per-column sums for dw/db are
// kept in registers and written once per CTA into the scratch `partial` ([gridDim.x][2][cols] fp32), which the finish
// kernel reduces in a fixed order (deterministic).
template <typename T, bool RMS, int ITERS>
__global__ void __launch_bounds__(NORM_THREADS)
    norm_bwd_kernel(const T* __restrict__ x, const T* __restrict__ w, const float* __restrict__ mean,
                    const float* __restrict__ rstd, const T* __restrict__ g, T* __restrict__ dx,
                    float* __restrict__ partial, long long rows, int cols) {
  constexpr int N = XlVec<T>::N;
  __shared__ float red[32];
  const int nvec = cols / N;
  float ww[ITERS][N], dw[ITERS][N], db[ITERS][N];
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int i = threadIdx.x + it * NORM_THREADS;
#pragma unroll
    for (int k = 0; k < N; ++k) { dw[it][k] = 0.f; db[it][k] = 0.f; ww[it][k] = 0.f; }
    if (i < nvec) xl_load16(w + i * N, ww[it]);
  }
  // The next row's loads are issued before the current row's two block reductions: with two CTAs of 8 warps per SM the
  // row-by-row chain load -> reduce -> store would otherwise leave the memory system idle most of the time.
  // (only while the extra registers keep two CTAs per SM: up to 16 values per array and thread)
  constexpr bool AHEAD = ITERS * N <= 16;
  uint4 nx[ITERS], ng[ITERS];
  float n_mu = 0.f, n_rs = 0.f;
  auto request = [&](long long row) {
    if (row >= rows) return;
    n_mu = RMS ? 0.f : mean[row];
    n_rs = rstd[row];
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      const int i = threadIdx.x + it * NORM_THREADS;
      if (i < nvec) {
        nx[it] = *reinterpret_cast<const uint4*>(x + row * cols + i * N);
        ng[it] = *reinterpret_cast<const uint4*>(g + row * cols + i * N);
      }
    }
  };
  request(blockIdx.x);
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    if (!AHEAD && row != (long long)blockIdx.x) request(row);
    const float mu = n_mu, rs = n_rs;
    uint4 cx[ITERS], cg[ITERS];
#pragma unroll
    for (int it = 0; it < ITERS; ++it) { cx[it] = nx[it]; cg[it] = ng[it]; }
    if (AHEAD) request(row + gridDim.x);
    float xh[ITERS][N], gw[ITERS][N];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      const int i = threadIdx.x + it * NORM_THREADS;
      if (i < nvec) {
        const T* xe = reinterpret_cast<const T*>(&cx[it]);
        const T* ge = reinterpret_cast<const T*>(&cg[it]);
#pragma unroll
        for (int k = 0; k < N; ++k) {
          const float xv = xl_to_float(xe[k]), gv = xl_to_float(ge[k]);
          xh[it][k] = (xv - mu) * rs;
          gw[it][k] = gv * ww[it][k];
          s1 += gw[it][k];
          s2 += gw[it][k] * xh[it][k];
          dw[it][k] += gv * xh[it][k];
          db[it][k] += gv;
        }
      }
    }
    const float c2 = xl_block_sum(s2, red) / cols;
    const float c1 = RMS ? 0.f : xl_block_sum(s1, red) / cols;
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      const int i = threadIdx.x + it * NORM_THREADS;
      if (i < nvec) {
        float o[N];
#pragma unroll
        for (int k = 0; k < N; ++k) o[k] = (gw[it][k] - c1 - xh[it][k] * c2) * rs;
        xl_store16(dx + row * cols + i * N, o);
      }
    }
  }
  float* pw = partial + (long long)blockIdx.x * 2 * cols;
  float* pb = pw + cols;
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int i = threadIdx.x + it * NORM_THREADS;
    if (i < nvec) {
#pragma unroll
      for (int k = 0; k < N; ++k) {
        pw[i * N + k] = dw[it][k];
        if (!RMS) pb[i * N + k] = db[it][k];
      }
    }
  }
}

// One CTA per 32 columns: 8 groups of 32 threads walk the per-CTA partial rows with stride 8 (coalesced 128-byte reads),
// then the 8 group sums are added in a fixed order (deterministic).
template <typename T>
__global__ void __launch_bounds__(256)
    norm_bwd_finish_kernel(const float* __restrict__ partial, T* __restrict__ dw, T* __restrict__ db, int nparts, int cols) {
  __shared__ float sw[8][33], sb[8][33];
  const int lane = threadIdx.x & 31, grp = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  float aw = 0.f, ab = 0.f;
  if (c < cols) {
    for (int p = grp; p < nparts; p += 8) {
      aw += partial[(long long)p * 2 * cols + c];
      if (db) ab += partial[(long long)p * 2 * cols + cols + c];
    }
  }
  sw[grp][lane] = aw;
  sb[grp][lane] = ab;
  __syncthreads();
  if (grp == 0 && c < cols) {
    float tw = 0.f, tb = 0.f;
#pragma unroll
    for (int g = 0; g < 8; ++g) { tw += sw[g][lane]; tb += sb[g][lane]; }
    dw[c] = xl_from_float<T>(tw);
    if (db) db[c] = xl_from_float<T>(tb);
  }
}

// Number of CTAs (= rows of the scratch buffer) the backward kernels use for `rows` rows.
XL_API int xl_norm_bwd_parts(long long rows) { return (int)(rows < 296 ? rows : 296); }

template <bool RMS>
static int norm_bwd_launch(const void* x, const void* w, const float* mean, const float* rstd, const void* g, void* dx,
                           void* dw, void* db, float* partial, long long rows, int cols, int dtype, cudaStream_t s) {
  // the backward keeps 5 row-sized arrays in registers: at most 16 values per array and thread
  const int iters = norm_iters(cols, dtype, dtype == XL_F32 ? 4 : 2);
  if (!iters) return -1;
  const int parts = xl_norm_bwd_parts(rows);
  XL_DISPATCH_DTYPE(dtype, T, XL_DISPATCH_ITERS(iters, IT, {
    norm_bwd_kernel<T, RMS, IT><<<parts, NORM_THREADS, 0, s>>>((const T*)x, (const T*)w, mean, rstd, (const T*)g,
                                                              (T*)dx, partial, rows, cols);
    norm_bwd_finish_kernel<T><<<(cols + 31) / 32, 256, 0, s>>>(partial, (T*)dw, (T*)db, parts, cols);
  }));
  return (int)cudaGetLastError();
}
XL_API int xl_layer_norm_bwd(const void* x, const void* w, const float* mean, const float* rstd, const void* g,
                             void* dx, void* dw, void* db, float* scratch, long long rows, int cols, int dtype,
                             cudaStream_t s) {
  return norm_bwd_launch<false>(x, w, mean, rstd, g, dx, dw, db, scratch, rows, cols, dtype, s);
}
XL_API int xl_rms_norm_bwd(const void* x, const void* w, const float* rstd, const void* g, void* dx, void* dw,
                           float* scratch, long long rows, int cols, int dtype, cudaStream_t s) {
  return norm_bwd_launch<true>(x, w, nullptr, rstd, g, dx, dw, nullptr, scratch, rows, cols, dtype, s);
}

// ------------------------------------------------------------------------------------------------------------------
// Column sums of a row-major matrix (bias gradients: sum over the token rows)
// ------------------------------------------------------------------------------------------------------------------
constexpr int COLSUM_THREADS = 256;

// grid (column tiles of 32 lanes x N columns, row parts): the 8 warps of a CTA take every 8th row of the part, four
// rows in flight per warp; the warps' sums are added through shared memory in a fixed order and written to
// `partial[part][cols]`; the finish kernel adds the parts in a fixed order (deterministic).
template <typename T>
__global__ void __launch_bounds__(COLSUM_THREADS)
    col_sum_kernel(const T* __restrict__ x, float* __restrict__ partial, long long rows, int cols, long long rows_per_part) {
  constexpr int N = XlVec<T>::N;
  __shared__ float red[COLSUM_THREADS / 32][32 * N + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c0 = (blockIdx.x * 32 + lane) * N;
  const long long r_begin = blockIdx.y * rows_per_part;
  const long long r_end = r_begin + rows_per_part < rows ? r_begin + rows_per_part : rows;
  float acc[N];
#pragma unroll
  for (int k = 0; k < N; ++k) acc[k] = 0.f;
  if (c0 < cols) {
    constexpr int WARPS = COLSUM_THREADS / 32;
    long long r = r_begin + warp;
    for (; r + 3 * WARPS < r_end; r += 4 * WARPS) {
      float v[4][N];
#pragma unroll
      for (int u = 0; u < 4; ++u) xl_load16(x + (r + u * WARPS) * cols + c0, v[u]);
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int k = 0; k < N; ++k) acc[k] += v[u][k];
    }
    for (; r < r_end; r += WARPS) {
      float v[N];
      xl_load16(x + r * cols + c0, v);
#pragma unroll
      for (int k = 0; k < N; ++k) acc[k] += v[k];
    }
  }
#pragma unroll
  for (int k = 0; k < N; ++k) red[warp][lane * N + k] = acc[k];
  __syncthreads();
  for (int i = threadIdx.x; i < 32 * N; i += COLSUM_THREADS) {
    const int c = blockIdx.x * 32 * N + i;
    if (c < cols) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < COLSUM_THREADS / 32; ++w) t += red[w][i];
      partial[(long long)blockIdx.y * cols + c] = t;
    }
  }
}
template <typename T>
__global__ void __launch_bounds__(256) col_sum_finish_kernel(const float* __restrict__ partial, T* __restrict__ out, int parts, int cols) {
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c >= cols) return;
  float t = 0.f;
  for (int p = 0; p < parts; ++p) t += partial[(long long)p * cols + c];
  out[c] = xl_from_float<T>(t);
}

// Row parts (= rows of the fp32 scratch `partial`, parts x cols) that xl_col_sum uses for this shape.
XL_API int xl_col_sum_parts(long long rows, int cols, int dtype) {
  const int n = dtype == XL_F32 ? 4 : 8;
  const long long tiles = (cols + 32 * n - 1) / (32 * n);
  long long parts = (4 * 148 + tiles - 1) / tiles;  // about four CTAs per SM in total
  const long long max_parts = (rows + 31) / 32;     // at least 32 rows per part
  if (parts > max_parts) parts = max_parts;
  if (parts > 256) parts = 256;
  return (int)(parts < 1 ? 1 : parts);
}
// out[c] = sum over rows of x[r][c]; x row-major (rows x cols) with cols a multiple of 16 bytes, 16-byte aligned.
XL_API int xl_col_sum(const void* x, void* out, float* partial, long long rows, int cols, int dtype, cudaStream_t s) {
  const int n = dtype == XL_F32 ? 4 : 8;
  if (rows <= 0 || cols <= 0 || (cols % n) || (((uintptr_t)x) & 15)) return -1;
  const int parts = xl_col_sum_parts(rows, cols, dtype);
  const long long rows_per_part = (rows + parts - 1) / parts;
  dim3 grid((cols + 32 * n - 1) / (32 * n), parts);
  XL_DISPATCH_DTYPE(dtype, T, {
    col_sum_kernel<T><<<grid, COLSUM_THREADS, 0, s>>>((const T*)x, partial, rows, cols, rows_per_part);
    col_sum_finish_kernel<T><<<(cols + 255) / 256, 256, 0, s>>>(partial, (T*)out, parts, cols);
  });
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------------------------
// AdamW / SGD / running-mean accumulation
// ------------------------------------------------------------------------------------------------------------------
struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay, grad_scale;
  int bias_correction;
};

__global__ void step_increment_kernel(float* step) { *step += 1.f; }

template <typename TW, typename TG, typename TM>
__global__ void __launch_bounds__(256)
    adam_kernel(TW* __restrict__ w, const TG* __restrict__ g, TM* __restrict__ m, float* __restrict__ v,
                float* __restrict__ master, const float* __restrict__ step, AdamArgs a, long long n) {
  float c1 = 1.f, c2 = 1.f;
  if (step != nullptr && a.bias_correction) {
    const float t = *step;
    c1 = 1.f / (1.f - powf(a.beta1, t));
    c2 = 1.f / (1.f - powf(a.beta2, t));
  }
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float gf = xl_to_float(g[i]) * a.grad_scale;
    const float mf = xl_to_float(m[i]) * a.beta1 + gf * (1.f - a.beta1);
    const float vf = v[i] * a.beta2 + gf * gf * (1.f - a.beta2);
    const TM mq = xl_from_float<TM>(mf);
    m[i] = mq;
    v[i] = vf;
    const float wf = master ? master[i] : xl_to_float(w[i]);
    const float upd = (xl_to_float(mq) * c1) / (sqrtf(vf * c2) + a.eps) + wf * a.weight_decay;
    const float wn = wf - a.lr * upd;
    if (master) master[i] = wn;
    w[i] = xl_from_float<TW>(wn);
  }
}

template <typename TW, typename TG>
static int adam_launch_m(void* w, const void* g, void* m, int m_dtype, float* v, float* master, float* step,
                         AdamArgs a, long long n, cudaStream_t s) {
  const int grid = xl_grid_for(n, 256 * 4);
  switch (m_dtype) {
    case XL_F32: adam_kernel<TW, TG, float><<<grid, 256, 0, s>>>((TW*)w, (const TG*)g, (float*)m, v, master, step, a, n); break;
    case XL_F16: adam_kernel<TW, TG, __half><<<grid, 256, 0, s>>>((TW*)w, (const TG*)g, (__half*)m, v, master, step, a, n); break;
    case XL_BF16: adam_kernel<TW, TG, __nv_bfloat16><<<grid, 256, 0, s>>>((TW*)w, (const TG*)g, (__nv_bfloat16*)m, v, master, step, a, n); break;
    default: return (int)cudaErrorInvalidValue;
  }
  return (int)cudaGetLastError();
}

// One AdamW step over `n` elements. `step` (device float, may be null) is incremented first and used for bias
// correction; `master` (fp32, may be null) carries the full-precision weights when `w` is 16-bit.
XL_API int xl_adam_step(void* w, int w_dtype, const void* g, int g_dtype, void* m, int m_dtype, float* v, float* master,
                        float* step, float lr, float beta1, float beta2, float eps, float weight_decay,
                        float grad_scale, int bias_correction, long long n, cudaStream_t s) {
  AdamArgs a{lr, beta1, beta2, eps, weight_decay, grad_scale, bias_correction};
  if (step) step_increment_kernel<<<1, 1, 0, s>>>(step);
  if (g_dtype != w_dtype && g_dtype != XL_F32) return -1;
  XL_DISPATCH_DTYPE(w_dtype, TW, {
    if (g_dtype == XL_F32) return adam_launch_m<TW, float>(w, g, m, m_dtype, v, master, step, a, n, s);
    return adam_launch_m<TW, TW>(w, g, m, m_dtype, v, master, step, a, n, s);
  });
  return (int)cudaGetLastError();
}

template <typename TW, typename TG>
__global__ void __launch_bounds__(256)
    sgd_kernel(TW* __restrict__ w, const TG* __restrict__ g, float* __restrict__ buf, float lr, float momentum,
               float weight_decay, float grad_scale, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float wf = xl_to_float(w[i]);
    float gf = xl_to_float(g[i]) * grad_scale + wf * weight_decay;
    if (buf) { gf = buf[i] * momentum + gf; buf[i] = gf; }
    w[i] = xl_from_float<TW>(wf - lr * gf);
  }
}
XL_API int xl_sgd_step(void* w, int w_dtype, const void* g, int g_dtype, float* buf, float lr, float momentum,
                       float weight_decay, float grad_scale, long long n, cudaStream_t s) {
  const int grid = xl_grid_for(n, 256 * 4);
  if (g_dtype != w_dtype && g_dtype != XL_F32) return -1;
  XL_DISPATCH_DTYPE(w_dtype, TW, {
    if (g_dtype == XL_F32) sgd_kernel<TW, float><<<grid, 256, 0, s>>>((TW*)w, (const float*)g, buf, lr, momentum, weight_decay, grad_scale, n);
    else sgd_kernel<TW, TW><<<grid, 256, 0, s>>>((TW*)w, (const TW*)g, buf, lr, momentum, weight_decay, grad_scale, n);
  });
  return (int)cudaGetLastError();
}

// acc = acc * step/(step+1) + x/(step+1), `step` read on the device.
template <typename TA, typename TX>
__global__ void __launch_bounds__(256)
    accumulate_mean_kernel(TA* __restrict__ acc, const TX* __restrict__ x, const float* __restrict__ step, long long n) {
  const float t = *step;
  const float a = t / (t + 1.f), b = 1.f / (t + 1.f);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    acc[i] = xl_from_float<TA>(xl_to_float(acc[i]) * a + xl_to_float(x[i]) * b);
}
XL_API int xl_accumulate_mean(void* acc, int acc_dtype, const void* x, int x_dtype, const float* step, long long n,
                              cudaStream_t s) {
  const int grid = xl_grid_for(n, 256 * 4);
  XL_DISPATCH_DTYPE(acc_dtype, TA, {
    if (x_dtype == acc_dtype) accumulate_mean_kernel<TA, TA><<<grid, 256, 0, s>>>((TA*)acc, (const TA*)x, step, n);
    else if (x_dtype == XL_BF16) accumulate_mean_kernel<TA, __nv_bfloat16><<<grid, 256, 0, s>>>((TA*)acc, (const __nv_bfloat16*)x, step, n);
    else if (x_dtype == XL_F16) accumulate_mean_kernel<TA, __half><<<grid, 256, 0, s>>>((TA*)acc, (const __half*)x, step, n);
    else accumulate_mean_kernel<TA, float><<<grid, 256, 0, s>>>((TA*)acc, (const float*)x, step, n);
  });
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------------------------
// sum of squares (gradient norm): per-CTA partials in scratch, then a single CTA adds them in index order
// ------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) sumsq_partial_kernel(const T* __restrict__ x, float* __restrict__ partial, long long n) {
  __shared__ float red[32];
  float acc = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float v = xl_to_float(x[i]);
    acc += v * v;
  }
  acc = xl_block_sum(acc, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = acc;
}
__global__ void sumsq_finish_kernel(const float* __restrict__ partial, int nparts, const float* __restrict__ scale,
                                    float* __restrict__ out) {
  __shared__ float red[32];
  float acc = 0.f;
  for (int i = threadIdx.x; i < nparts; i += blockDim.x) acc += partial[i];
  acc = xl_block_sum(acc, red);
  if (threadIdx.x == 0) *out = acc * (scale ? *scale : 1.f);
}
XL_API int xl_sumsq_parts(long long n) { return xl_grid_for(n, 256 * 16, 1024); }
XL_API int xl_grad_sumsq(const void* x, int dtype, const float* scale, float* out, float* scratch, long long n,
                         cudaStream_t s) {
  const int parts = xl_sumsq_parts(n);
  XL_DISPATCH_DTYPE(dtype, T, { sumsq_partial_kernel<T><<<parts, 256, 0, s>>>((const T*)x, scratch, n); });
  sumsq_finish_kernel<<<1, 256, 0, s>>>(scratch, parts, scale, out);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------------------------
// Rotary position embedding on interleaved pairs. x: (B, H, S, D); sin/cos: (Bs, S, R/2) with Bs in {1, B}.
// ------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
    rotary_kernel(const T* __restrict__ x, const T* __restrict__ sin_t, const T* __restrict__ cos_t, T* __restrict__ y,
                  long long total_pairs, int H, int S, int D, int R, int sin_batch, float sign, long long xb,
                  long long xh, long long xs, long long yb, long long yh, long long ys) {
  // in place only the rotated pairs are touched; out of place the pass-through features are copied as well
  const int pairs_per_row = (x == y) ? R / 2 : D / 2;
  for (long long p = blockIdx.x * (long long)blockDim.x + threadIdx.x; p < total_pairs; p += (long long)gridDim.x * blockDim.x) {
    const int j = (int)(p % pairs_per_row);
    long long row = p / pairs_per_row;  // (b*H + h)*S + s
    const int sidx = (int)(row % S);
    row /= S;
    const int h = (int)(row % H);
    const long long b = row / H;
    const T* xp = x + b * xb + h * xh + sidx * xs + 2 * j;
    T* yp = y + b * yb + h * yh + sidx * ys + 2 * j;
    const float a0 = xl_to_float(xp[0]), a1 = xl_to_float(xp[1]);
    if (2 * j < R) {
      const long long t = ((sin_batch > 1 ? b : 0) * S + sidx) * (long long)(R / 2) + j;
      const float sn = xl_to_float(sin_t[t]) * sign, cs = xl_to_float(cos_t[t]);
      yp[0] = xl_from_float<T>(a0 * cs - a1 * sn);
      yp[1] = xl_from_float<T>(a1 * cs + a0 * sn);
    } else if (yp != xp) {
      yp[0] = xp[0];
      yp[1] = xp[1];
    }
  }
}
// Strides (in elements) of the batch, head and sequence axes are explicit so that head-interleaved layouts such as a
// packed (tokens, 3*heads*head_dim) qkv matrix can be rotated in place; the feature axis must be contiguous.
XL_API int xl_rotary(const void* x, const void* sin_t, const void* cos_t, void* y, long long B, int H, int S, int D,
                     int R, int sin_batch, int inverse, int dtype, long long xb, long long xh, long long xs,
                     long long yb, long long yh, long long ys, cudaStream_t s) {
  const long long pairs = B * H * S * (long long)((x == y ? R : D) / 2);
  if (pairs == 0) return 0;
  const int grid = xl_grid_for(pairs, 256 * 4);
  XL_DISPATCH_DTYPE(dtype, T, {
    rotary_kernel<T><<<grid, 256, 0, s>>>((const T*)x, (const T*)sin_t, (const T*)cos_t, (T*)y, pairs, H, S, D, R,
                                          sin_batch, inverse ? -1.f : 1.f, xb, xh, xs, yb, yh, ys);
  });
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------------------------
// int4 group de-quantisation. packed: (rows, groups, gs/4) u16, first element in the top nibble. One thread -> two
// words -> eight outputs (one 16-byte store for 16-bit outputs).
// ------------------------------------------------------------------------------------------------------------------
template <typename T, typename S>
__global__ void __launch_bounds__(256)
    gq_decompress_kernel(const uint16_t* __restrict__ packed, const S* __restrict__ scale, const S* __restrict__ bias,
                         T* __restrict__ out, long long n_pairs, int words_per_group) {
  for (long long p = blockIdx.x * (long long)blockDim.x + threadIdx.x; p < n_pairs; p += (long long)gridDim.x * blockDim.x) {
    const uint32_t two = *reinterpret_cast<const uint32_t*>(packed + 2 * p);
    const long long group = (2 * p) / words_per_group;
    const float sc = xl_to_float(scale[group]), bi = xl_to_float(bias[group]);
    const uint32_t w0 = two & 0xffffu, w1 = two >> 16;
    T o[8];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      o[k] = xl_from_float<T>((float)((w0 >> (12 - 4 * k)) & 0xfu) * sc + bi);
      o[4 + k] = xl_from_float<T>((float)((w1 >> (12 - 4 * k)) & 0xfu) * sc + bi);
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) out[8 * p + k] = o[k];
  }
}
// `dtype`: type of the output; `scale_dtype`: type of the per-group scale and bias (may differ, e.g. fp16 scales with a
// bf16 model).
XL_API int xl_gq_decompress(const void* packed, const void* scale, const void* bias, void* out, long long n_words,
                            int words_per_group, int dtype, int scale_dtype, cudaStream_t s) {
  if ((n_words & 1) || (words_per_group & 1)) return -1;
  const long long pairs = n_words / 2;
  const int grid = xl_grid_for(pairs, 256 * 4);
  XL_DISPATCH_DTYPE(dtype, T, {
    XL_DISPATCH_DTYPE(scale_dtype, S, {
      gq_decompress_kernel<T, S><<<grid, 256, 0, s>>>((const uint16_t*)packed, (const S*)scale, (const S*)bias, (T*)out,
                                                     pairs, words_per_group);
    });
  });
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------------------------
// Softmax over attention scores, in place. s: (batch, Sq, Sk); row r of a batch may attend to columns
// <= r + (Sk - Sq) when causal. Writes probabilities (zeros in the masked part) and the row log-sum-exp.
// ------------------------------------------------------------------------------------------------------------------
constexpr int SM_THREADS = 128;
constexpr int SM_MAX_ITERS = 8;

template <typename T, int ITERS>
__global__ void __launch_bounds__(SM_THREADS)
    attn_softmax_fwd_kernel(T* __restrict__ s, float* __restrict__ lse, int Sq, int Sk, float scale, int causal) {
  constexpr int N = XlVec<T>::N;
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const int r = (int)(row % Sq);
  const int limit = causal ? min(Sk, r + (Sk - Sq) + 1) : Sk;  // valid columns: [0, limit)
  T* sr = s + row * Sk;
  const int nvec = Sk / N;
  float v[ITERS][N];
  float mx = -INFINITY;
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int i = threadIdx.x + it * SM_THREADS;
    if (i < nvec && i * N < limit) {
      xl_load16(sr + i * N, v[it]);
#pragma unroll
      for (int k = 0; k < N; ++k) {
        v[it][k] = (i * N + k < limit) ? v[it][k] * scale : -INFINITY;
        mx = fmaxf(mx, v[it][k]);
      }
    } else {
#pragma unroll
      for (int k = 0; k < N; ++k) v[it][k] = -INFINITY;
    }
  }
  mx = xl_block_max(mx, red);
  float sum = 0.f;
#pragma unroll
  for (int it = 0; it < ITERS; ++it)
#pragma unroll
    for (int k = 0; k < N; ++k) {
      v[it][k] = __expf(v[it][k] - mx);
      sum += v[it][k];
    }
  sum = xl_block_sum(sum, red);
  const float inv = 1.f / sum;
  if (threadIdx.x == 0) lse[row] = mx + logf(sum);
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int i = threadIdx.x + it * SM_THREADS;
    if (i < nvec) {
      float o[N];
#pragma unroll
      for (int k = 0; k < N; ++k) o[k] = v[it][k] * inv;
      xl_store16(sr + i * N, o);
    }
  }
}

// ds = p * (dp - sum(p*dp)) * scale, written over dp.
template <typename T, int ITERS>
__global__ void __launch_bounds__(SM_THREADS)
    attn_softmax_bwd_kernel(const T* __restrict__ p, T* __restrict__ dp, int Sq, int Sk, float scale, int causal) {
  constexpr int N = XlVec<T>::N;
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const int r = (int)(row % Sq);
  const int limit = causal ? min(Sk, r + (Sk - Sq) + 1) : Sk;
  const T* pr = p + row * Sk;
  T* dr = dp + row * Sk;
  const int nvec = Sk / N;
  float pv[ITERS][N], dv[ITERS][N];
  float dot = 0.f;
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int i = threadIdx.x + it * SM_THREADS;
    if (i < nvec && i * N < limit) {
      xl_load16(pr + i * N, pv[it]);
      xl_load16(dr + i * N, dv[it]);
#pragma unroll
      for (int k = 0; k < N; ++k) dot += pv[it][k] * dv[it][k];
    } else {
#pragma unroll
      for (int k = 0; k < N; ++k) { pv[it][k] = 0.f; dv[it][k] = 0.f; }
    }
  }
  dot = xl_block_sum(dot, red);
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int i = threadIdx.x + it * SM_THREADS;
    if (i < nvec) {
      float o[N];
#pragma unroll
      for (int k = 0; k < N; ++k) o[k] = pv[it][k] * (dv[it][k] - dot) * scale;
      xl_store16(dr + i * N, o);
    }
  }
}
static inline int softmax_iters(int Sk, int dtype, int max_iters) {
  const int n = dtype == XL_F32 ? 4 : 8;
  if (Sk % n != 0) return 0;
  for (int it = 1; it <= max_iters; it *= 2)
    if (Sk / n <= SM_THREADS * it) return it;
  return 0;
}
XL_API int xl_attn_softmax_fwd(void* s_, float* lse, long long rows, int Sq, int Sk, float scale, int causal, int dtype,
                               cudaStream_t s) {
  const int iters = softmax_iters(Sk, dtype, SM_MAX_ITERS);
  if (!iters) return -1;
  XL_DISPATCH_DTYPE(dtype, T, XL_DISPATCH_ITERS(iters, IT, {
    attn_softmax_fwd_kernel<T, IT><<<(unsigned)rows, SM_THREADS, 0, s>>>((T*)s_, lse, Sq, Sk, scale, causal);
  }));
  return (int)cudaGetLastError();
}
XL_API int xl_attn_softmax_bwd(const void* p, void* dp, long long rows, int Sq, int Sk, float scale, int causal,
                               int dtype, cudaStream_t s) {
  const int iters = softmax_iters(Sk, dtype, 4);
  if (!iters) return -1;
  XL_DISPATCH_DTYPE(dtype, T, XL_DISPATCH_ITERS(iters, IT, {
    attn_softmax_bwd_kernel<T, IT><<<(unsigned)rows, SM_THREADS, 0, s>>>((const T*)p, (T*)dp, Sq, Sk, scale, causal);
  }));
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------------------------
// Cross-entropy on logits with the gradient fused: one CTA per row, three sweeps over the row (max, sum-exp, write);
// the row (<= ~100 KB) stays in L2 between sweeps. loss_row[r] = -log softmax(x)[label]; dlogits = (softmax -
// onehot) * grad_scale for valid rows, 0 for ignored rows. Mean reduction and its 1/count are applied by the caller.
// ------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(512)
    ce_fwd_bwd_kernel(const T* __restrict__ logits, const int* __restrict__ labels, float* __restrict__ loss_row,
                      T* __restrict__ dlogits, int V, int ignore_index, const float* __restrict__ grad_scale_ptr,
                      float grad_scale) {
  constexpr int N = XlVec<T>::N;
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const T* xr = logits + row * V;
  const int label = labels[row];
  const bool valid = label != ignore_index && label >= 0 && label < V;
  const int nvec = V / N;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    float a[N];
    xl_load16(xr + i * N, a);
#pragma unroll
    for (int k = 0; k < N; ++k) mx = fmaxf(mx, a[k]);
  }
  for (int i = nvec * N + threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, xl_to_float(xr[i]));
  mx = xl_block_max(mx, red);
  float sum = 0.f;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    float a[N];
    xl_load16(xr + i * N, a);
#pragma unroll
    for (int k = 0; k < N; ++k) sum += __expf(a[k] - mx);
  }
  for (int i = nvec * N + threadIdx.x; i < V; i += blockDim.x) sum += __expf(xl_to_float(xr[i]) - mx);
  sum = xl_block_sum(sum, red);
  const float lse = mx + logf(sum);
  if (threadIdx.x == 0) loss_row[row] = valid ? lse - xl_to_float(xr[label]) : 0.f;
  if (dlogits == nullptr) return;
  const float gs = valid ? (grad_scale_ptr ? *grad_scale_ptr * grad_scale : grad_scale) : 0.f;
  T* dr = dlogits + row * V;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    float a[N];
    xl_load16(xr + i * N, a);
#pragma unroll
    for (int k = 0; k < N; ++k) {
      float p = __expf(a[k] - lse);
      if (i * N + k == label) p -= 1.f;
      a[k] = p * gs;
    }
    xl_store16(dr + i * N, a);
  }
  for (int i = nvec * N + threadIdx.x; i < V; i += blockDim.x) {
    float p = __expf(xl_to_float(xr[i]) - lse);
    if (i == label) p -= 1.f;
    dr[i] = xl_from_float<T>(p * gs);
  }
}
XL_API int xl_ce_fwd_bwd(const void* logits, const int* labels, float* loss_row, void* dlogits, long long rows, int V,
                         int ignore_index, const float* grad_scale_ptr, float grad_scale, int dtype, cudaStream_t s) {
  const int vec = dtype == XL_F32 ? 4 : 8;
  if ((V * (dtype == XL_F32 ? 4 : 2)) % 16 != 0 && rows > 1) return -1;  // rows must stay 16-byte aligned
  (void)vec;
  XL_DISPATCH_DTYPE(dtype, T, {
    ce_fwd_bwd_kernel<T><<<(unsigned)rows, 512, 0, s>>>((const T*)logits, labels, loss_row, (T*)dlogits, V, ignore_index,
                                                       grad_scale_ptr, grad_scale);
  });
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------------------------
// FP8: amax-based power-of-two scale and scaled cast
// ------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) amax_kernel(const T* __restrict__ x, unsigned int* __restrict__ out_bits, long long n) {
  __shared__ float red[32];
  float m = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    m = fmaxf(m, fabsf(xl_to_float(x[i])));
  m = xl_block_max(m, red);
  if (threadIdx.x == 0) atomicMax(out_bits, __float_as_uint(m));  // non-negative floats order like their bit patterns
}
XL_API int xl_amax(const void* x, int dtype, float* out_zeroed, long long n, cudaStream_t s) {
  const int grid = xl_grid_for(n, 256 * 16, 1024);
  XL_DISPATCH_DTYPE(dtype, T, { amax_kernel<T><<<grid, 256, 0, s>>>((const T*)x, (unsigned int*)out_zeroed, n); });
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------------------------
// Allocation-free sum of squares (see xl_noalloc.h). Same two kernels as xl_grad_sumsq, but the per-block partial sums
// live in a fixed array that is part of the library image instead of caller-provided scratch.
// ------------------------------------------------------------------------------------------------------------------
#include "xl_noalloc.h"

static __device__ __align__(256) float xl_noalloc_partials[XL_NOALLOC_SUMSQ_PARTS];

// Device address of the array above, per device. The array's name is only a stand-in in host code, so the address
// is looked up once per device (with that device current) and cached.
static float* xl_noalloc_partials_addr[XL_NOALLOC_MAX_DEVICES] = {nullptr};

XL_API int xl_grad_sumsq_noalloc(const void* x, int dtype, const float* scale, float* out, long long n, cudaStream_t s) {
  if (x == nullptr || out == nullptr || n <= 0) return XL_NOALLOC_BAD_ARGUMENT;
  if (n > XL_NOALLOC_SUMSQ_MAX_ELEMS) return XL_NOALLOC_TOO_LARGE;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= XL_NOALLOC_MAX_DEVICES) return XL_NOALLOC_BAD_ARGUMENT;
  if (xl_noalloc_partials_addr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, xl_noalloc_partials);
    if (e != cudaSuccess) return (int)e;
    xl_noalloc_partials_addr[dev] = p;
  }
  float* partials = xl_noalloc_partials_addr[dev];
  const int parts = xl_grid_for(n, 256 * 16, XL_NOALLOC_SUMSQ_PARTS);
  // every one of the `parts` slots is overwritten by its block before the finish kernel reads it: nothing left over
  // from an earlier call is ever consumed, so the array needs no clearing
  XL_DISPATCH_DTYPE(dtype, T, { sumsq_partial_kernel<T><<<parts, 256, 0, s>>>((const T*)x, partials, n); });
  sumsq_finish_kernel<<<1, 256, 0, s>>>(partials, parts, scale, out);
  return (int)cudaGetLastError();
}
