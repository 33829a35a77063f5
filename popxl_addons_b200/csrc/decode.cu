// Kernels of the token-by-token decoding path (batch of a few sequences, one new token each):
//   xl_gq_gemm_small_m   y[M<=16, N] = x[M, K] * dequant(Wq)[K, N] (+ bias): 4-bit group-quantised weights are streamed
//                        once, de-quantised in registers and fed to the tensor cores; no 16-bit copy of W ever exists
//   xl_rotary_at         rotary embedding of the new tokens at a position read from device memory
//   xl_kv_append         write the new keys / values into the KV cache at that position
//   xl_attn_decode       attention of the new query against the cache (split over the sequence + combine)
//   xl_argmax_rows       greedy sampling: per-row (max, index) of the local logits slice
// Everything that depends on the current position reads it from a device word, so one decoding step has no
// launch-time argument that changes between steps and can be replayed as a CUDA graph.
//
// The de-quantising GEMM is bandwidth-bound by construction (M <= 16: two FLOPs per weight nibble and row), so it uses
// the register-operand `mma.sync.m16n8k16` form: its operands come straight from the registers that hold the freshly
// de-quantised values, which is exactly what a streaming kernel wants. (tcgen05 needs its B operand in shared memory;
// for prefill-sized M the weights are de-quantised once and the tcgen05 GEMM is used.)
#include "common.cuh"

#include <math.h>
#include <type_traits>

// ------------------------------------------------------------------------------------------------------------------
// int4 group-quantised GEMM, M <= 16
// ------------------------------------------------------------------------------------------------------------------
constexpr int GQ_NT = 4;         // n-tiles of 8 columns per warp -> a CTA covers 32 output columns
constexpr int GQ_WARPS = 8;      // warps of a CTA split K between them
constexpr int GQ_KCHUNK = 128;   // k values per warp iteration (32 per lane quad member)

__device__ __forceinline__ void mma_m16n8k16(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2], bool bf16) {
  if (bf16) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
  } else {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
  }
}

template <typename T> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// packed: (N, K/gs, gs/4) u16, first element of a word in its top nibble; scale / zero: (N, K/gs).
// Any assignment of actual k indices to the 16 k-slots of an MMA is valid as long as A and B agree, so each lane
// keeps the 32 consecutive k values of its 16-byte weight load and feeds them to 8 MMAs, 4 values at a time.
template <typename T, typename S>
__global__ void __launch_bounds__(GQ_WARPS * 32)
    gq_gemm_small_m_kernel(const T* __restrict__ x, const uint16_t* __restrict__ packed, const S* __restrict__ scale,
                           const S* __restrict__ zero, const T* __restrict__ bias, T* __restrict__ y, int M, int N, int K,
                           int group_size) {
  __shared__ float red[GQ_WARPS][16][8 * GQ_NT + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int quad = lane >> 2, j = lane & 3;  // quad: row of A / column of B inside a tile; j: k sub-slot
  const int n_base = blockIdx.x * (8 * GQ_NT);
  const int groups = K / group_size;
  constexpr bool BF = std::is_same<T, __nv_bfloat16>::value;
  float c[GQ_NT][4];
#pragma unroll
  for (int t = 0; t < GQ_NT; ++t)
#pragma unroll
    for (int e = 0; e < 4; ++e) c[t][e] = 0.f;
  const int k_per_warp = (K / GQ_KCHUNK + GQ_WARPS - 1) / GQ_WARPS * GQ_KCHUNK;
  const int k_begin = warp * k_per_warp;
  const int k_end = min(K, k_begin + k_per_warp);
  const bool row_lo = quad < M, row_hi = quad + 8 < M;
  for (int k0 = k_begin; k0 < k_end; k0 += GQ_KCHUNK) {
    const int k_lane = k0 + j * 32;  // this lane's 32 consecutive k values
    // activations: rows quad and quad+8, 32 values each
    uint4 xa[4], xb[4];
    const uint4 zero4 = make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      xa[v] = row_lo ? *reinterpret_cast<const uint4*>(x + (long long)quad * K + k_lane + v * 8) : zero4;
      xb[v] = row_hi ? *reinterpret_cast<const uint4*>(x + (long long)(quad + 8) * K + k_lane + v * 8) : zero4;
    }
    const uint32_t* xa32 = reinterpret_cast<const uint32_t*>(xa);
    const uint32_t* xb32 = reinterpret_cast<const uint32_t*>(xb);
    const int g = k_lane / group_size;
#pragma unroll
    for (int t = 0; t < GQ_NT; ++t) {
      const int n = n_base + t * 8 + quad;
      uint4 wq = make_uint4(0, 0, 0, 0);
      float sc = 0.f, zp = 0.f;
      if (n < N) {
        wq = *reinterpret_cast<const uint4*>(packed + (long long)n * (K / 4) + k_lane / 4);
        sc = xl_to_float(scale[(long long)n * groups + g]);
        zp = xl_to_float(zero[(long long)n * groups + g]);
      }
      const uint16_t* w16 = reinterpret_cast<const uint16_t*>(&wq);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        // word i holds k_lane + 4i .. 4i+3
        const uint32_t w = w16[i];
        const float v0 = (float)((w >> 12) & 0xF) * sc + zp, v1 = (float)((w >> 8) & 0xF) * sc + zp;
        const float v2 = (float)((w >> 4) & 0xF) * sc + zp, v3 = (float)(w & 0xF) * sc + zp;
        const uint32_t b[2] = {pack2<T>(v0, v1), pack2<T>(v2, v3)};
        const uint32_t a[4] = {xa32[2 * i], xb32[2 * i], xa32[2 * i + 1], xb32[2 * i + 1]};
        mma_m16n8k16(c[t], a, b, BF);
      }
    }
  }
  // reduce the K slices of the warps through shared memory
#pragma unroll
  for (int t = 0; t < GQ_NT; ++t) {
    red[warp][quad][t * 8 + 2 * j] = c[t][0];
    red[warp][quad][t * 8 + 2 * j + 1] = c[t][1];
    red[warp][quad + 8][t * 8 + 2 * j] = c[t][2];
    red[warp][quad + 8][t * 8 + 2 * j + 1] = c[t][3];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < 16 * 8 * GQ_NT; idx += blockDim.x) {
    const int r = idx / (8 * GQ_NT), col = idx % (8 * GQ_NT);
    const int n = n_base + col;
    if (r < M && n < N) {
      float acc = 0.f;
#pragma unroll
      for (int w = 0; w < GQ_WARPS; ++w) acc += red[w][r][col];
      if (bias) acc += xl_to_float(bias[n]);
      y[(long long)r * N + n] = xl_from_float<T>(acc);
    }
  }
}

// Requirements: M <= 16, K % 128 == 0, group_size % 32 == 0, 16-byte aligned pointers. Returns -1 otherwise.
template <typename T>
static void gq_small_launch(const void* x, const void* packed, const void* scale, const void* zero, const void* bias, void* y,
                            int M, int N, int K, int group_size, int scale_dtype, int grid, cudaStream_t s) {
  if (scale_dtype == XL_F16)
    gq_gemm_small_m_kernel<T, __half><<<grid, GQ_WARPS * 32, 0, s>>>((const T*)x, (const uint16_t*)packed,
                                                                     (const __half*)scale, (const __half*)zero,
                                                                     (const T*)bias, (T*)y, M, N, K, group_size);
  else
    gq_gemm_small_m_kernel<T, __nv_bfloat16><<<grid, GQ_WARPS * 32, 0, s>>>(
        (const T*)x, (const uint16_t*)packed, (const __nv_bfloat16*)scale, (const __nv_bfloat16*)zero, (const T*)bias,
        (T*)y, M, N, K, group_size);
}
// `dtype`: type of x, bias and y (fp16 or bf16); `scale_dtype`: type of the per-group scale and zero point (fp16 / bf16).
XL_API int xl_gq_gemm_small_m(const void* x, const void* packed, const void* scale, const void* zero, const void* bias,
                              void* y, int M, int N, int K, int group_size, int dtype, int scale_dtype, cudaStream_t s) {
  if (M < 1 || M > 16 || K % GQ_KCHUNK || group_size % 32 || K % group_size || dtype == XL_F32 || scale_dtype == XL_F32)
    return -1;
  const int grid = (N + 8 * GQ_NT - 1) / (8 * GQ_NT);
  if (dtype == XL_BF16)
    gq_small_launch<__nv_bfloat16>(x, packed, scale, zero, bias, y, M, N, K, group_size, scale_dtype, grid, s);
  else
    gq_small_launch<__half>(x, packed, scale, zero, bias, y, M, N, K, group_size, scale_dtype, grid, s);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------------------------
// Rotary at a device-side position + KV-cache append.
// qkv: (B, 3*H*D) new-token projections [q | k | v]; rotates q and k in place (first R features of each head) for
// position pos = *pos_ptr and copies k, v into the caches (B, H, Smax, D) at that position.
// sin / cos tables: (Smax, R/2).
// ------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
    rotary_append_kernel(T* __restrict__ qkv, const T* __restrict__ sin_t, const T* __restrict__ cos_t,
                         T* __restrict__ k_cache, T* __restrict__ v_cache, const int* __restrict__ pos_ptr, int B, int H,
                         int D, int R, int Smax) {
  const int pos = *pos_ptr;
  const int hd = H * D;
  const long long total = (long long)B * hd;  // one thread per (b, h, d) feature of k / v, pairs handled by even d
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int d = (int)(i % D);
    const int h = (int)((i / D) % H);
    const int b = (int)(i / hd);
    T* q = qkv + (long long)b * 3 * hd + h * D;
    T* k = q + hd;
    const T* v = q + 2 * hd;
    if (d < R && (d & 1) == 0) {
      const float sn = xl_to_float(sin_t[(long long)pos * (R / 2) + d / 2]);
      const float cs = xl_to_float(cos_t[(long long)pos * (R / 2) + d / 2]);
      const float q0 = xl_to_float(q[d]), q1 = xl_to_float(q[d + 1]);
      q[d] = xl_from_float<T>(q0 * cs - q1 * sn);
      q[d + 1] = xl_from_float<T>(q1 * cs + q0 * sn);
      const float k0 = xl_to_float(k[d]), k1 = xl_to_float(k[d + 1]);
      const T r0 = xl_from_float<T>(k0 * cs - k1 * sn), r1 = xl_from_float<T>(k1 * cs + k0 * sn);
      k[d] = r0;
      k[d + 1] = r1;
    }
  }
  // second pass (after the rotation of this thread's own pairs is visible to itself only): copy is done by a separate
  // kernel launch below to avoid intra-kernel ordering between threads
}

template <typename T>
__global__ void __launch_bounds__(256)
    kv_append_kernel(const T* __restrict__ qkv, T* __restrict__ k_cache, T* __restrict__ v_cache,
                     const int* __restrict__ pos_ptr, int B, int H, int D, int Smax) {
  const int pos = *pos_ptr;
  const int hd = H * D;
  const long long total = (long long)B * hd;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int d = (int)(i % D);
    const int h = (int)((i / D) % H);
    const int b = (int)(i / hd);
    const long long src = (long long)b * 3 * hd + h * D + d;
    const long long dst = (((long long)b * H + h) * Smax + pos) * D + d;
    k_cache[dst] = qkv[src + hd];
    v_cache[dst] = qkv[src + 2 * hd];
  }
}

XL_API int xl_rotary_append(void* qkv, const void* sin_t, const void* cos_t, void* k_cache, void* v_cache,
                            const int* pos_ptr, int B, int H, int D, int R, int Smax, int dtype, cudaStream_t s) {
  const long long total = (long long)B * H * D;
  const int grid = xl_grid_for(total, 256);
  XL_DISPATCH_DTYPE(dtype, T, {
    if (R > 0)
      rotary_append_kernel<T><<<grid, 256, 0, s>>>((T*)qkv, (const T*)sin_t, (const T*)cos_t, (T*)k_cache, (T*)v_cache,
                                                   pos_ptr, B, H, D, R, Smax);
    kv_append_kernel<T><<<grid, 256, 0, s>>>((const T*)qkv, (T*)k_cache, (T*)v_cache, pos_ptr, B, H, D, Smax);
  });
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------------------------
// Decode attention: one query per (b, h) against cache positions [0, len), len = *pos_ptr + 1.
// Grid (B*H, splits): each CTA covers a slice of the positions with an online softmax (one warp per position at a
// time, lanes over the head dimension) and writes (max, sum, unnormalised output); the combine kernel merges the splits.
// ------------------------------------------------------------------------------------------------------------------
constexpr int AD_WARPS = 4;
constexpr int AD_MAX_D = 256;  // head_dim <= 256 (8 values per lane)

template <typename T>
__global__ void __launch_bounds__(AD_WARPS * 32)
    attn_decode_split_kernel(const T* __restrict__ qkv, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                             float* __restrict__ part, const int* __restrict__ pos_ptr, int H, int D, int Smax,
                             float scale, int splits) {
  const int bh = blockIdx.x, split = blockIdx.y;
  const int b = bh / H, h = bh % H;
  const int len = *pos_ptr + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per = (len + splits - 1) / splits;
  const int s_begin = split * per, s_end = min(len, s_begin + per);
  const int VPL = D / 32;  // values per lane (D multiple of 32, <= 8)
  float q[8], o[8];
  const T* qp = qkv + (long long)b * 3 * H * D + h * D;
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    q[e] = (e < VPL) ? xl_to_float(qp[lane * VPL + e]) * scale : 0.f;
    o[e] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  const T* kb = k_cache + ((long long)bh * Smax) * D;
  const T* vb = v_cache + ((long long)bh * Smax) * D;
  for (int sidx = s_begin + warp; sidx < s_end; sidx += AD_WARPS) {
    float dot = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e)
      if (e < VPL) dot += q[e] * xl_to_float(kb[(long long)sidx * D + lane * VPL + e]);
    dot = xl_warp_sum(dot);
    const float m_new = fmaxf(m, dot);
    const float corr = __expf(m - m_new), p = __expf(dot - m_new);
    l = l * corr + p;
#pragma unroll
    for (int e = 0; e < 8; ++e)
      if (e < VPL) o[e] = o[e] * corr + p * xl_to_float(vb[(long long)sidx * D + lane * VPL + e]);
    m = m_new;
  }
  // merge the warps of this CTA
  __shared__ float sm[AD_WARPS], sl[AD_WARPS], so[AD_WARPS][AD_MAX_D];
  if (lane == 0) { sm[warp] = m; sl[warp] = l; }
#pragma unroll
  for (int e = 0; e < 8; ++e)
    if (e < VPL) so[warp][lane * VPL + e] = o[e];
  __syncthreads();
  if (warp == 0) {
    float mm = -INFINITY;
    for (int w = 0; w < AD_WARPS; ++w) mm = fmaxf(mm, sm[w]);
    float ll = 0.f;
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    for (int w = 0; w < AD_WARPS; ++w) {
      const float f = (sm[w] == -INFINITY) ? 0.f : __expf(sm[w] - mm);
      ll += sl[w] * f;
#pragma unroll
      for (int e = 0; e < 8; ++e)
        if (e < VPL) acc[e] += so[w][lane * VPL + e] * f;
    }
    float* dst = part + ((long long)bh * splits + split) * (D + 2);
    if (lane == 0) { dst[0] = mm; dst[1] = ll; }
#pragma unroll
    for (int e = 0; e < 8; ++e)
      if (e < VPL) dst[2 + lane * VPL + e] = acc[e];
  }
}

template <typename T>
__global__ void attn_decode_combine_kernel(const float* __restrict__ part, T* __restrict__ out, int D, int splits) {
  const int bh = blockIdx.x;
  const float* p = part + (long long)bh * splits * (D + 2);
  float mm = -INFINITY;
  for (int s = 0; s < splits; ++s) mm = fmaxf(mm, p[s * (D + 2)]);
  float ll = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = p[s * (D + 2)];
    ll += (ms == -INFINITY) ? 0.f : p[s * (D + 2) + 1] * __expf(ms - mm);
  }
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float ms = p[s * (D + 2)];
      if (ms != -INFINITY) acc += p[s * (D + 2) + 2 + d] * __expf(ms - mm);
    }
    out[(long long)bh * D + d] = xl_from_float<T>(acc / ll);
  }
}

// out: (B, H*D). scratch: B*H*splits*(D+2) floats.
XL_API int xl_attn_decode(const void* qkv, const void* k_cache, const void* v_cache, void* out, float* scratch,
                          const int* pos_ptr, int B, int H, int D, int Smax, float scale, int splits, int dtype,
                          cudaStream_t s) {
  if (D % 32 || D > AD_MAX_D || splits < 1) return -1;
  dim3 grid(B * H, splits);
  XL_DISPATCH_DTYPE(dtype, T, {
    attn_decode_split_kernel<T><<<grid, AD_WARPS * 32, 0, s>>>((const T*)qkv, (const T*)k_cache, (const T*)v_cache,
                                                               scratch, pos_ptr, H, D, Smax, scale, splits);
    attn_decode_combine_kernel<T><<<B * H, 128, 0, s>>>(scratch, (T*)out, D, splits);
  });
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------------------------
// Greedy sampling support: per row of logits (rows, V) the maximum and its index (+ index_offset of this vocabulary
// shard); pos_ptr, if given, is incremented by one afterwards (advances the decoding position on the device).
// ------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
    argmax_rows_kernel(const T* __restrict__ logits, float* __restrict__ max_out, int* __restrict__ idx_out, int V,
                       int valid, int index_offset) {
  __shared__ float sv[256];
  __shared__ int si[256];
  const long long row = blockIdx.x;
  float best = -INFINITY;
  int bi = 0;
  for (int i = threadIdx.x; i < valid; i += blockDim.x) {
    const float v = xl_to_float(logits[row * V + i]);
    if (v > best) { best = v; bi = i; }
  }
  sv[threadIdx.x] = best;
  si[threadIdx.x] = bi;
  __syncthreads();
  for (int off = 128; off > 0; off >>= 1) {
    if (threadIdx.x < off) {
      const float o = sv[threadIdx.x + off];
      const int oi = si[threadIdx.x + off];
      if (o > sv[threadIdx.x] || (o == sv[threadIdx.x] && oi < si[threadIdx.x])) { sv[threadIdx.x] = o; si[threadIdx.x] = oi; }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) { max_out[row] = sv[0]; idx_out[row] = si[0] + index_offset; }
}
__global__ void advance_position_kernel(int* pos) { *pos += 1; }

XL_API int xl_argmax_rows(const void* logits, float* max_out, int* idx_out, long long rows, int V, int valid,
                          int index_offset, int dtype, cudaStream_t s) {
  XL_DISPATCH_DTYPE(dtype, T, {
    argmax_rows_kernel<T><<<(unsigned)rows, 256, 0, s>>>((const T*)logits, max_out, idx_out, V, valid, index_offset);
  });
  return (int)cudaGetLastError();
}
XL_API int xl_advance_position(int* pos, cudaStream_t s) {
  advance_position_kernel<<<1, 1, 0, s>>>(pos);
  return (int)cudaGetLastError();
}

// buf: (rows, B) int32; writes vals (B) into row (*pos_ptr - base).
__global__ void store_row_kernel(int* __restrict__ buf, const int* __restrict__ pos_ptr, int base, const int* __restrict__ vals,
                                 int B, int rows) {
  const int r = *pos_ptr - base;
  if (r < 0 || r >= rows) return;
  for (int i = threadIdx.x; i < B; i += blockDim.x) buf[(long long)r * B + i] = vals[i];
}
XL_API int xl_store_row(int* buf, const int* pos_ptr, int base, const int* vals, int B, int rows, cudaStream_t s) {
  store_row_kernel<<<1, 128, 0, s>>>(buf, pos_ptr, base, vals, B, rows);
  return (int)cudaGetLastError();
}
