// Kernels for ops whose reduction axis is sharded over ranks (or over several tensors of one rank): the
// vocabulary-sharded cross-entropy and the backward pass of the hidden-sharded LayerNorm. Each op is a pair of passes
// over the local shard with a tiny per-row exchange (a few floats per row) between them, which the caller all-reduces
// with the one-shot NVLink kernel (several ranks) or combines on the device (several shards on one rank).
//
//   cross-entropy   pass 1  xl_ce_shard_stats    per row: local max m, sum of exp(x - m), x[label] if the label is local
//                   (max over ranks of m)        xl_ce_shard_rescale: s * exp(m - gmax)       (sum over ranks of s', picked)
//                   pass 2  xl_ce_shard_grad_loss  dlogits = (softmax - onehot) * scale[row], loss[row]
//                        or xl_ce_shard_nls        negative log-softmax of the shard (the op that keeps it for autodiff)
//                           xl_ce_nls_grad         gradient from the kept negative log-softmax
//   LayerNorm       pass 1  xl_ln_shard_bwd_stats  per row: sum(g*w), sum(g*w*xhat) over the local columns
//                   pass 2  xl_ln_shard_bwd_apply  dx from the group sums; per-column partial sums of dw, db
//                           (reduced over the CTAs in a fixed order by a finishing kernel: deterministic)
#include "common.cuh"

namespace {

constexpr int ROW_THREADS = 256;

__device__ __forceinline__ float block_sum(float v, float* red) { return xl_block_sum(v, red); }
__device__ __forceinline__ float block_max(float v, float* red) { return xl_block_max(v, red); }

// ---- cross-entropy ---------------------------------------------------------------------------------------------------
// stats: (3, rows) fp32 = [local max | sum of exp(x - local max) | x[label - label_offset] if that column is local else 0]
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS)
    ce_shard_stats_kernel(const T* __restrict__ x, const int* __restrict__ labels, int label_offset,
                          float* __restrict__ stats, int rows, int cols) {
  constexpr int N = XlVec<T>::N;
  __shared__ float red[32];
  const int r = blockIdx.x;
  const T* xr = x + (long long)r * cols;
  const bool vec = (cols % N == 0) && ((((uintptr_t)xr) & 15) == 0);
  // one pass: running maximum and the sum rescaled whenever the maximum moves
  float m = -INFINITY, s = 0.f;
  if (vec) {
    const int nvec = cols / N;
    for (int i = threadIdx.x; i < nvec; i += ROW_THREADS) {
      float v[N];
      xl_load16(xr + i * N, v);
      float vm = v[0];
#pragma unroll
      for (int k = 1; k < N; ++k) vm = fmaxf(vm, v[k]);
      if (vm > m) {
        s *= __expf(m - vm);  // exp(-inf) = 0 on the first vector
        m = vm;
      }
#pragma unroll
      for (int k = 0; k < N; ++k) s += __expf(v[k] - m);
    }
  } else {
    for (int c = threadIdx.x; c < cols; c += ROW_THREADS) {
      const float v = xl_to_float(xr[c]);
      if (v > m) {
        s *= __expf(m - v);
        m = v;
      }
      s += __expf(v - m);
    }
  }
  const float gm = block_max(m, red);
  const float contrib = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  const float gs = block_sum(contrib, red);
  if (threadIdx.x == 0) {
    stats[r] = gm;
    stats[rows + r] = gs;
    const int l = labels[r] - label_offset;
    stats[2 * rows + r] = (l >= 0 && l < cols) ? xl_to_float(xr[l]) : 0.f;
  }
}

// out (2, rows) = [s * exp(m - gmax) | picked]: what is summed over the ranks once the group maximum is known
__global__ void ce_shard_rescale_kernel(const float* __restrict__ stats, const float* __restrict__ gmax,
                                        float* __restrict__ out, int rows) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  out[r] = stats[rows + r] * __expf(stats[r] - gmax[r]);
  out[rows + r] = stats[2 * rows + r];
}

// several shards on one device: stats_all = (n_shards, 3, rows) -> out (3, rows) = [gmax | gsum | picked]
__global__ void ce_shard_combine_kernel(const float* __restrict__ stats_all, float* __restrict__ out, int n_shards,
                                        int rows) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  float gm = -INFINITY;
  for (int i = 0; i < n_shards; ++i) gm = fmaxf(gm, stats_all[(long long)i * 3 * rows + r]);
  float gs = 0.f, gp = 0.f;
  for (int i = 0; i < n_shards; ++i) {
    const float* st = stats_all + (long long)i * 3 * rows;
    gs += st[rows + r] * __expf(st[r] - gm);
    gp += st[2 * rows + r];
  }
  out[r] = gm;
  out[rows + r] = gs;
  out[2 * rows + r] = gp;
}

// dx = (exp(x - gmax) / gsum - onehot(label)) * scale[row];  loss[row] = log(gsum) + gmax - picked  (may be null)
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS)
    ce_shard_grad_loss_kernel(const T* __restrict__ x, const float* __restrict__ gmax, const float* __restrict__ gsum,
                              const float* __restrict__ gpicked, const int* __restrict__ labels, int label_offset,
                              const float* __restrict__ row_scale, T* __restrict__ dx, float* __restrict__ loss, int cols) {
  constexpr int N = XlVec<T>::N;
  const int r = blockIdx.x;
  const float g = gmax[r], inv = 1.f / gsum[r], sc = row_scale[r];
  const int l = labels[r] - label_offset;
  const T* xr = x + (long long)r * cols;
  T* dr = dx + (long long)r * cols;
  if ((cols % N == 0) && ((((uintptr_t)xr) & 15) == 0) && ((((uintptr_t)dr) & 15) == 0)) {
    const int nvec = cols / N;
    for (int i = threadIdx.x; i < nvec; i += ROW_THREADS) {
      float v[N];
      xl_load16(xr + i * N, v);
#pragma unroll
      for (int k = 0; k < N; ++k) {
        float p = __expf(v[k] - g) * inv;
        if (i * N + k == l) p -= 1.f;
        v[k] = p * sc;
      }
      xl_store16(dr + i * N, v);
    }
  } else {
    for (int c = threadIdx.x; c < cols; c += ROW_THREADS) {
      float p = __expf(xl_to_float(xr[c]) - g) * inv;
      if (c == l) p -= 1.f;
      dr[c] = xl_from_float<T>(p * sc);
    }
  }
  if (loss != nullptr && threadIdx.x == 0) loss[r] = __logf(gsum[r]) + g - gpicked[r];
}

// nls = -(x - gmax - log(gsum));  loss[row] = log(gsum) + gmax - picked  (may be null)
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS)
    ce_shard_nls_kernel(const T* __restrict__ x, const float* __restrict__ gmax, const float* __restrict__ gsum,
                        const float* __restrict__ gpicked, T* __restrict__ nls, T* __restrict__ loss, int cols) {
  const int r = blockIdx.x;
  const float shift = gmax[r] + __logf(gsum[r]);
  const T* xr = x + (long long)r * cols;
  T* nr = nls + (long long)r * cols;
  for (int c = threadIdx.x; c < cols; c += ROW_THREADS) nr[c] = xl_from_float<T>(shift - xl_to_float(xr[c]));
  if (loss != nullptr && threadIdx.x == 0) loss[r] = xl_from_float<T>(shift - gpicked[r]);
}

// dx = exp(-nls) * dloss[row] - onehot(label) * dloss[row]
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS)
    ce_nls_grad_kernel(const T* __restrict__ nls, const int* __restrict__ labels, int label_offset,
                       const T* __restrict__ dloss, T* __restrict__ dx, int cols) {
  const int r = blockIdx.x;
  const float dl = xl_to_float(dloss[r]);
  const int l = labels[r] - label_offset;
  const T* nr = nls + (long long)r * cols;
  T* dr = dx + (long long)r * cols;
  for (int c = threadIdx.x; c < cols; c += ROW_THREADS) {
    float p = __expf(-xl_to_float(nr[c])) * dl;
    if (c == l) p -= dl;
    dr[c] = xl_from_float<T>(p);
  }
}

// ---- hidden-sharded LayerNorm, backward ------------------------------------------------------------------------------
// stats (2, rows) = [sum over local columns of g*w | of g*w*xhat],  xhat = (x - mean) * rstd
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS)
    ln_shard_bwd_stats_kernel(const T* __restrict__ x, const T* __restrict__ w, const float* __restrict__ mean,
                              const float* __restrict__ rstd, const T* __restrict__ g, float* __restrict__ stats,
                              int rows, int cols) {
  __shared__ float red[32];
  const int r = blockIdx.x;
  const float mu = mean[r], rs = rstd[r];
  float s1 = 0.f, s2 = 0.f;
  for (int c = threadIdx.x; c < cols; c += ROW_THREADS) {
    const long long i = (long long)r * cols + c;
    const float gw = xl_to_float(g[i]) * xl_to_float(w[c]);
    s1 += gw;
    s2 += gw * (xl_to_float(x[i]) - mu) * rs;
  }
  s1 = block_sum(s1, red);
  s2 = block_sum(s2, red);
  if (threadIdx.x == 0) {
    stats[r] = s1;
    stats[rows + r] = s2;
  }
}

// dx = (g*w - c1 - xhat * c2) * rstd with c = group sums / hidden; partial (gridDim.x, 2, cols) = per-CTA sums of
// g*xhat (dw) and g (db) over the rows the CTA walked. Columns per thread: cols <= ROW_THREADS * MAX_COLS_PER_THREAD.
constexpr int MAX_COLS_PER_THREAD = 32;
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS)
    ln_shard_bwd_apply_kernel(const T* __restrict__ x, const T* __restrict__ w, const float* __restrict__ mean,
                              const float* __restrict__ rstd, const T* __restrict__ g, const float* __restrict__ gstats,
                              T* __restrict__ dx, float* __restrict__ partial, int rows, int cols, float hidden) {
  float dw[MAX_COLS_PER_THREAD], db[MAX_COLS_PER_THREAD];
#pragma unroll
  for (int j = 0; j < MAX_COLS_PER_THREAD; ++j) { dw[j] = 0.f; db[j] = 0.f; }
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const float mu = mean[r], rs = rstd[r];
    const float c1 = gstats[r] / hidden, c2 = gstats[rows + r] / hidden;
#pragma unroll
    for (int j = 0; j < MAX_COLS_PER_THREAD; ++j) {
      const int c = threadIdx.x + j * ROW_THREADS;
      if (c < cols) {
        const long long i = (long long)r * cols + c;
        const float gv = xl_to_float(g[i]);
        const float xh = (xl_to_float(x[i]) - mu) * rs;
        const float gw = gv * xl_to_float(w[c]);
        dx[i] = xl_from_float<T>((gw - c1 - xh * c2) * rs);
        dw[j] += gv * xh;
        db[j] += gv;
      }
    }
  }
  float* pw = partial + (long long)blockIdx.x * 2 * cols;
#pragma unroll
  for (int j = 0; j < MAX_COLS_PER_THREAD; ++j) {
    const int c = threadIdx.x + j * ROW_THREADS;
    if (c < cols) {
      pw[c] = dw[j];
      pw[cols + c] = db[j];
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
    ln_shard_bwd_finish_kernel(const float* __restrict__ partial, T* __restrict__ dw, T* __restrict__ db, int nparts,
                               int cols) {
  // one CTA per 32 columns; 8 groups of 32 threads walk the partial rows with stride 8, group sums added in a fixed order
  __shared__ float sw[8][33], sb[8][33];
  const int lane = threadIdx.x & 31, grp = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  float aw = 0.f, ab = 0.f;
  if (c < cols) {
    for (int p = grp; p < nparts; p += 8) {
      aw += partial[(long long)p * 2 * cols + c];
      ab += partial[(long long)p * 2 * cols + cols + c];
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
    db[c] = xl_from_float<T>(tb);
  }
}

}  // namespace

XL_API int xl_ce_shard_stats(const void* x, int dtype, const int* labels, int label_offset, float* stats, int rows,
                             int cols, cudaStream_t s) {
  if (rows <= 0 || cols <= 0) return -1;
  XL_DISPATCH_DTYPE(dtype, T, {
    ce_shard_stats_kernel<T><<<rows, ROW_THREADS, 0, s>>>((const T*)x, labels, label_offset, stats, rows, cols);
  });
  return (int)cudaGetLastError();
}

XL_API int xl_ce_shard_rescale(const float* stats, const float* gmax, float* out, int rows, cudaStream_t s) {
  if (rows <= 0) return -1;
  ce_shard_rescale_kernel<<<(rows + 255) / 256, 256, 0, s>>>(stats, gmax, out, rows);
  return (int)cudaGetLastError();
}

XL_API int xl_ce_shard_combine(const float* stats_all, float* out, int n_shards, int rows, cudaStream_t s) {
  if (rows <= 0 || n_shards <= 0) return -1;
  ce_shard_combine_kernel<<<(rows + 255) / 256, 256, 0, s>>>(stats_all, out, n_shards, rows);
  return (int)cudaGetLastError();
}

XL_API int xl_ce_shard_grad_loss(const void* x, int dtype, const float* gmax, const float* gsum, const float* gpicked,
                                 const int* labels, int label_offset, const float* row_scale, void* dx, float* loss,
                                 int rows, int cols, cudaStream_t s) {
  if (rows <= 0 || cols <= 0) return -1;
  XL_DISPATCH_DTYPE(dtype, T, {
    ce_shard_grad_loss_kernel<T><<<rows, ROW_THREADS, 0, s>>>((const T*)x, gmax, gsum, gpicked, labels, label_offset,
                                                              row_scale, (T*)dx, loss, cols);
  });
  return (int)cudaGetLastError();
}

// nls and loss have the dtype of x
XL_API int xl_ce_shard_nls(const void* x, int dtype, const float* gmax, const float* gsum, const float* gpicked, void* nls,
                           void* loss, int rows, int cols, cudaStream_t s) {
  if (rows <= 0 || cols <= 0) return -1;
  XL_DISPATCH_DTYPE(dtype, T, {
    ce_shard_nls_kernel<T><<<rows, ROW_THREADS, 0, s>>>((const T*)x, gmax, gsum, gpicked, (T*)nls, (T*)loss, cols);
  });
  return (int)cudaGetLastError();
}

XL_API int xl_ce_nls_grad(const void* nls, int dtype, const int* labels, int label_offset, const void* dloss, void* dx,
                          int rows, int cols, cudaStream_t s) {
  if (rows <= 0 || cols <= 0) return -1;
  XL_DISPATCH_DTYPE(dtype, T, {
    ce_nls_grad_kernel<T><<<rows, ROW_THREADS, 0, s>>>((const T*)nls, labels, label_offset, (const T*)dloss, (T*)dx, cols);
  });
  return (int)cudaGetLastError();
}

XL_API int xl_ln_shard_bwd_stats(const void* x, const void* w, const float* mean, const float* rstd, const void* g,
                                 float* stats, int rows, int cols, int dtype, cudaStream_t s) {
  if (rows <= 0 || cols <= 0) return -1;
  XL_DISPATCH_DTYPE(dtype, T, {
    ln_shard_bwd_stats_kernel<T><<<rows, ROW_THREADS, 0, s>>>((const T*)x, (const T*)w, mean, rstd, (const T*)g, stats,
                                                              rows, cols);
  });
  return (int)cudaGetLastError();
}

// CTAs (= rows of the scratch buffer) of the apply kernel for `rows` rows
XL_API int xl_ln_shard_bwd_parts(int rows) { return rows < 296 ? rows : 296; }

// scratch: xl_ln_shard_bwd_parts(rows) * 2 * cols floats. cols <= 8192. Returns -1 for wider shards.
XL_API int xl_ln_shard_bwd_apply(const void* x, const void* w, const float* mean, const float* rstd, const void* g,
                                 const float* gstats, void* dx, void* dw, void* db, float* scratch, int rows, int cols,
                                 float hidden, int dtype, cudaStream_t s) {
  if (rows <= 0 || cols <= 0 || cols > ROW_THREADS * MAX_COLS_PER_THREAD) return -1;
  const int parts = xl_ln_shard_bwd_parts(rows);
  XL_DISPATCH_DTYPE(dtype, T, {
    ln_shard_bwd_apply_kernel<T><<<parts, ROW_THREADS, 0, s>>>((const T*)x, (const T*)w, mean, rstd, (const T*)g, gstats,
                                                              (T*)dx, scratch, rows, cols, hidden);
    ln_shard_bwd_finish_kernel<T><<<(cols + 31) / 32, 256, 0, s>>>(scratch, (T*)dw, (T*)db, parts, cols);
  });
  return (int)cudaGetLastError();
}
