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
constexpr int GQ_NT = 8;         // n-tiles of 8 columns per warp -> a CTA covers 64 output columns
constexpr int GQ_WARPS = 8;      // warps of a CTA split K between them
constexpr int GQ_KCHUNK = 128;   // k values per warp iteration (32 per lane quad member)

__device__ __forceinline__ void mma_m16n8k16(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2], bool bf16) {
  if (bf16) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
  } else {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
  }
}

// ---- de-quantisation without integer->float conversions ------------------------------------------------------------
// A nibble n placed in the mantissa of a 16-bit float with a suitable exponent IS the number base + n
// (bf16: 0x4180 | n << 3 = 16 + n; fp16: 0x5400 | n << 4 = 64 + n). A packed subtraction of the base (exact) and one
// packed FMA per two weights give n * s + z, rounded once like the reference. The byte shuffles below turn one 32-bit
// load (two packed words = 8 nibbles, first element of a word in its top nibble) into four registers of two
// consecutive weights each, low half first.
template <typename T> struct GqFmt;
template <> struct GqFmt<__nv_bfloat16> {
  using T2 = __nv_bfloat162;
  static constexpr uint32_t MASK = 0x78787878u, MAGIC = 0x41804180u;
  static constexpr float BASE = 16.f;
  static __device__ __forceinline__ uint32_t lo(uint32_t w) { return (w << 3) & MASK; }
  static __device__ __forceinline__ uint32_t hi(uint32_t w) { return (w >> 1) & MASK; }
  static __device__ __forceinline__ T2 pair(float a) { return __float2bfloat162_rn(a); }
};
template <> struct GqFmt<__half> {
  using T2 = __half2;
  static constexpr uint32_t MASK = 0xF0F0F0F0u, MAGIC = 0x54005400u;
  static constexpr float BASE = 64.f;
  static __device__ __forceinline__ uint32_t lo(uint32_t w) { return (w << 4) & MASK; }
  static __device__ __forceinline__ uint32_t hi(uint32_t w) { return w & MASK; }
  static __device__ __forceinline__ T2 pair(float a) { return __float2half2_rn(a); }
};

// w: two packed words (word 0 in the low half). out[0..1]: weights 0-1, 2-3 of word 0; out[2..3]: the same of word 1.
template <typename T>
__device__ __forceinline__ void gq_dequant8(uint32_t w, typename GqFmt<T>::T2 s2, typename GqFmt<T>::T2 z2, uint32_t (&out)[4]) {
  using F = GqFmt<T>;
  using T2 = typename F::T2;
  const uint32_t lo = F::lo(w), hi = F::hi(w);  // low / high nibble of every byte, moved into the mantissa position
  const uint32_t sel[4] = {0x0501u, 0x0400u, 0x0703u, 0x0602u};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t v = (__byte_perm(hi, lo, sel[i]) & 0x00FF00FFu) | F::MAGIC;
    T2 r = __hfma2(__hsub2(*reinterpret_cast<T2*>(&v), F::pair(F::BASE)), s2, z2);
    out[i] = *reinterpret_cast<uint32_t*>(&r);
  }
}

// packed: (N, K/gs, gs/4) u16, first element of a word in its top nibble; scale / zero: (N, K/gs).
// Any assignment of actual k indices to the 16 k-slots of an MMA is valid as long as A and B agree, so each lane
// keeps the 32 consecutive k values of its 16-byte weight load and feeds them to 8 MMAs, 4 values at a time.
//
// Work = (column tiles of 64) x (K chunks of 128), tile-major, cut into equal contiguous ranges, one per CTA
// ("stream-K": the grid is sized to the machine, not to the problem, so there is no partial last wave). A CTA walks
// its range tile by tile; its warps split the chunks of the current tile segment and reduce through shared memory.
// A segment that covers a whole tile is finished by its CTA; otherwise the CTAs sharing the tile add their partial
// sums into an fp32 workspace tile and the one that completes the tile's chunk count applies the epilogue and leaves
// workspace and counter zeroed for the next launch. Epilogue: + bias, GELU on the columns >= act_from_col. x and y are
// windows of wider matrices (ldx, ldy).
template <typename T, typename S>
__global__ void __launch_bounds__(GQ_WARPS * 32, 2)
    gq_gemm_small_m_kernel(const T* __restrict__ x, const uint16_t* __restrict__ packed, const S* __restrict__ scale,
                           const S* __restrict__ zero, const T* __restrict__ bias, T* __restrict__ y, int M, int N, int K,
                           int group_size, long long ldx, long long ldy, int act_from_col, float* __restrict__ ws,
                           unsigned int* __restrict__ counters, int sz_transposed) {
  using F = GqFmt<T>;
  using T2 = typename F::T2;
  __shared__ float red[GQ_WARPS][16][8 * GQ_NT + 1];
  __shared__ unsigned int finish;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int quad = lane >> 2, j = lane & 3;  // quad: row of A / column of B inside a tile; j: k sub-slot
  const int groups = K / group_size;
  constexpr bool BF = std::is_same<T, __nv_bfloat16>::value;
  constexpr int TILE = 16 * 8 * GQ_NT;
  const int chunks = K / GQ_KCHUNK;
  const int n_tiles = (N + 8 * GQ_NT - 1) / (8 * GQ_NT);
  const long long total = (long long)n_tiles * chunks;
  long long item = total * blockIdx.x / gridDim.x;
  const long long item_end = total * (blockIdx.x + 1) / gridDim.x;
  const bool row_lo = quad < M, row_hi = quad + 8 < M;
  // Weights reach the MMAs through a per-warp double buffer in shared memory filled with cp.async: while a warp works on
  // one chunk (8 tiles x 512 B) the next one, possibly of the next tile segment, is already in flight, so DRAM latency
  // is hidden without spending registers. Every lane reads back exactly the 16-byte pieces it copied itself.
  extern __shared__ uint4 wbuf_all[];
  uint4* wbuf = wbuf_all + warp * (2 * GQ_NT * 32);
  auto prefetch = [&](int tile_, int ch_, int buf_) {
    const int k_lane_ = ch_ * GQ_KCHUNK + j * 32;
#pragma unroll
    for (int t = 0; t < GQ_NT; ++t) {
      const int n = tile_ * (8 * GQ_NT) + t * 8 + quad;
      uint4* dst = wbuf + (buf_ * GQ_NT + t) * 32 + lane;
      if (n < N) {
        const uint16_t* src = packed + (long long)n * (K / 4) + k_lane_ / 4;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src)
                     : "memory");
      } else {
        *dst = make_uint4(0, 0, 0, 0);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  int buf = 0;
  bool have = false;  // wbuf[buf] already holds (or is receiving) this warp's first chunk of the current segment
  while (item < item_end) {
    const int tile = (int)(item / chunks);
    const int c0 = (int)(item - (long long)tile * chunks);
    const int c1 = (int)min((long long)chunks, c0 + (item_end - item));
    const int n_base = tile * (8 * GQ_NT);
    float c[GQ_NT][4];
#pragma unroll
    for (int t = 0; t < GQ_NT; ++t)
#pragma unroll
      for (int e = 0; e < 4; ++e) c[t][e] = 0.f;
    if (!have && c0 + warp < c1) prefetch(tile, c0 + warp, buf);
    have = false;
    for (int ch = c0 + warp; ch < c1; ch += GQ_WARPS) {
      // start the copy of the chunk after this one: the next of this segment, or this warp's first of the next segment
      bool next_issued = false;
      if (ch + GQ_WARPS < c1) {
        prefetch(tile, ch + GQ_WARPS, buf ^ 1);
        next_issued = true;
      } else {
        const long long nit = item + (c1 - c0);
        if (nit < item_end) {
          const int ntile = (int)(nit / chunks);
          const int nc0 = (int)(nit - (long long)ntile * chunks);
          const int nc1 = (int)min((long long)chunks, nc0 + (item_end - nit));
          if (nc0 + warp < nc1) {
            prefetch(ntile, nc0 + warp, buf ^ 1);
            next_issued = have = true;
          }
        }
      }
      const int k_lane = ch * GQ_KCHUNK + j * 32;  // this lane's 32 consecutive k values
      uint32_t sz[GQ_NT];  // (scale, zero) of this lane's group, two S values
      const int g = k_lane / group_size;
#pragma unroll
      for (int t = 0; t < GQ_NT; ++t) {
        const int n = n_base + t * 8 + quad;
        sz[t] = 0;
        if (n < N) {
          if (sz_transposed) {
            // scale holds (groups, N, 2): 8 consecutive columns of one group are one 32-byte segment
            sz[t] = reinterpret_cast<const uint32_t*>(scale)[(long long)g * N + n];
          } else {
            const S sv = scale[(long long)n * groups + g], zv = zero[(long long)n * groups + g];
            sz[t] = (uint32_t)(*reinterpret_cast<const uint16_t*>(&sv)) |
                    ((uint32_t)(*reinterpret_cast<const uint16_t*>(&zv)) << 16);
          }
        }
      }
      if (next_issued) asm volatile("cp.async.wait_group 1;" ::: "memory");
      else asm volatile("cp.async.wait_group 0;" ::: "memory");
      uint4 wq[GQ_NT];
#pragma unroll
      for (int t = 0; t < GQ_NT; ++t) wq[t] = wbuf[(buf * GQ_NT + t) * 32 + lane];
      buf ^= 1;
      T2 s2[GQ_NT], z2[GQ_NT];
#pragma unroll
      for (int t = 0; t < GQ_NT; ++t) {
        const uint16_t s16 = (uint16_t)(sz[t] & 0xFFFFu), z16 = (uint16_t)(sz[t] >> 16);
        s2[t] = F::pair(xl_to_float(*reinterpret_cast<const S*>(&s16)));
        z2[t] = F::pair(xl_to_float(*reinterpret_cast<const S*>(&z16)));
      }
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint4 xa[2], xb[2];
        const uint4 zero4 = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int v = 0; v < 2; ++v) {
          const long long off = k_lane + (2 * half + v) * 8;
          xa[v] = row_lo ? *reinterpret_cast<const uint4*>(x + (long long)quad * ldx + off) : zero4;
          xb[v] = row_hi ? *reinterpret_cast<const uint4*>(x + (long long)(quad + 8) * ldx + off) : zero4;
        }
        const uint32_t* xa32 = reinterpret_cast<const uint32_t*>(xa);
        const uint32_t* xb32 = reinterpret_cast<const uint32_t*>(xb);
        // k-step outermost: consecutive MMAs go to different accumulators, so none waits for its predecessor
#pragma unroll
        for (int mm = 0; mm < 2; ++mm) {
          const uint32_t a0[4] = {xa32[4 * mm], xb32[4 * mm], xa32[4 * mm + 1], xb32[4 * mm + 1]};
          const uint32_t a1[4] = {xa32[4 * mm + 2], xb32[4 * mm + 2], xa32[4 * mm + 3], xb32[4 * mm + 3]};
#pragma unroll
          for (int t = 0; t < GQ_NT; ++t) {
            // 32-bit word m of a lane's 16 bytes holds packed words 2m and 2m+1, i.e. k_lane + 8m .. 8m+7
            const uint32_t w = reinterpret_cast<const uint32_t*>(&wq[t])[2 * half + mm];
            uint32_t b[4];
            gq_dequant8<T>(w, s2[t], z2[t], b);
            const uint32_t b0[2] = {b[0], b[1]}, b1[2] = {b[2], b[3]};
            mma_m16n8k16(c[t], a0, b0, BF);
            mma_m16n8k16(c[t], a1, b1, BF);
          }
        }
      }
    }
    // reduce the K slices of the warps through shared memory
    __syncthreads();  // the previous segment's readers are done with `red`
#pragma unroll
    for (int t = 0; t < GQ_NT; ++t) {
      red[warp][quad][t * 8 + 2 * j] = c[t][0];
      red[warp][quad][t * 8 + 2 * j + 1] = c[t][1];
      red[warp][quad + 8][t * 8 + 2 * j] = c[t][2];
      red[warp][quad + 8][t * 8 + 2 * j + 1] = c[t][3];
    }
    __syncthreads();
    const bool whole = (c1 - c0) == chunks;
    float* wtile = ws + (long long)tile * TILE;
    bool finishing = whole;
    if (!whole) {
      for (int idx = threadIdx.x; idx < TILE; idx += blockDim.x) {
        const int r = idx / (8 * GQ_NT), col = idx % (8 * GQ_NT);
        if (r < M && n_base + col < N) {
          float acc = 0.f;
#pragma unroll
          for (int w = 0; w < GQ_WARPS; ++w) acc += red[w][r][col];
          atomicAdd(wtile + idx, acc);
        }
      }
      __threadfence();
      __syncthreads();
      if (threadIdx.x == 0)
        finish = atomicAdd(counters + tile, (unsigned int)(c1 - c0)) + (unsigned int)(c1 - c0) == (unsigned int)chunks;
      __syncthreads();
      finishing = finish != 0;
      if (finishing) __threadfence();
    }
    if (finishing) {
      for (int idx = threadIdx.x; idx < TILE; idx += blockDim.x) {
        const int r = idx / (8 * GQ_NT), col = idx % (8 * GQ_NT);
        const int n = n_base + col;
        if (r < M && n < N) {
          float acc = 0.f;
          if (!whole) {
            acc = __ldcg(wtile + idx);
            wtile[idx] = 0.f;
          } else {
#pragma unroll
            for (int w = 0; w < GQ_WARPS; ++w) acc += red[w][r][col];
          }
          if (bias) acc += xl_to_float(bias[n]);
          if (n >= act_from_col) acc = 0.5f * acc * (1.f + erff(acc * 0.70710678118654752f));
          y[(long long)r * ldy + n] = xl_from_float<T>(acc);
        }
      }
      if (!whole && threadIdx.x == 0) counters[tile] = 0;
    }
    item += c1 - c0;
  }
}

// Requirements: M <= 16, K % 128 == 0, group_size % 32 == 0, 16-byte aligned x rows and weight rows. `ws` / `counters`:
// zero-initialised scratch of ceil(N/64)*1024 floats / ceil(N/64) words (the kernel leaves them zeroed). `ctas`: size of
// the grid (0: two per SM of a 148-SM part). sz_transposed: `scale` holds (scale, zero) pairs laid out (K/gs, N, 2)
// and `zero` is unused: the layout in which the eight columns of an MMA tile are one contiguous 32-byte read. act_from_col: first column that gets GELU (>= N: none). Returns -1 for
// unsupported arguments.
template <typename T>
static void gq_small_launch(const void* x, const void* packed, const void* scale, const void* zero, const void* bias, void* y,
                            int M, int N, int K, int group_size, long long ldx, long long ldy, int act_from_col,
                            float* ws, unsigned int* counters, int scale_dtype, int sz_transposed, int grid,
                            cudaStream_t s) {
  constexpr int WBUF_BYTES = GQ_WARPS * 2 * GQ_NT * 32 * 16;  // per-warp double buffer of weight chunks
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(gq_gemm_small_m_kernel<T, __half>, cudaFuncAttributeMaxDynamicSharedMemorySize, WBUF_BYTES);
    cudaFuncSetAttribute(gq_gemm_small_m_kernel<T, __nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, WBUF_BYTES);
    configured = true;
  }
  if (scale_dtype == XL_F16)
    gq_gemm_small_m_kernel<T, __half><<<grid, GQ_WARPS * 32, WBUF_BYTES, s>>>(
        (const T*)x, (const uint16_t*)packed, (const __half*)scale, (const __half*)zero, (const T*)bias, (T*)y, M, N, K,
        group_size, ldx, ldy, act_from_col, ws, counters, sz_transposed);
  else
    gq_gemm_small_m_kernel<T, __nv_bfloat16><<<grid, GQ_WARPS * 32, WBUF_BYTES, s>>>(
        (const T*)x, (const uint16_t*)packed, (const __nv_bfloat16*)scale, (const __nv_bfloat16*)zero, (const T*)bias,
        (T*)y, M, N, K, group_size, ldx, ldy, act_from_col, ws, counters, sz_transposed);
}
// `dtype`: type of x, bias and y (fp16 or bf16); `scale_dtype`: type of the per-group scale and zero point (fp16 / bf16).
XL_API int xl_gq_gemm_small_m(const void* x, const void* packed, const void* scale, const void* zero, const void* bias,
                              void* y, int M, int N, int K, int group_size, long long ldx, long long ldy, int act_from_col,
                              int ctas, float* ws, unsigned int* counters, int dtype, int scale_dtype, int sz_transposed,
                              cudaStream_t s) {
  if (M < 1 || M > 16 || K % GQ_KCHUNK || group_size % 32 || K % group_size || dtype == XL_F32 || scale_dtype == XL_F32)
    return -1;
  if ((ldx % 8) || ws == nullptr || counters == nullptr) return -1;
  const long long total = (long long)((N + 8 * GQ_NT - 1) / (8 * GQ_NT)) * (K / GQ_KCHUNK);
  long long grid = ctas > 0 ? ctas : 2 * 148;
  if (grid > total) grid = total;
  if (dtype == XL_BF16)
    gq_small_launch<__nv_bfloat16>(x, packed, scale, zero, bias, y, M, N, K, group_size, ldx, ldy, act_from_col, ws,
                                   counters, scale_dtype, sz_transposed, (int)grid, s);
  else
    gq_small_launch<__half>(x, packed, scale, zero, bias, y, M, N, K, group_size, ldx, ldy, act_from_col, ws, counters,
                            scale_dtype, sz_transposed, (int)grid, s);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------------------------
// Rotary at a device-side position + KV-cache append, one launch.
// qkv: rows of `ld` elements whose first 3*H*D hold the new-token projections [q | k | v]; rotates q and k in place
// (first R features of each head, interleaved pairs) for position pos = *pos_ptr and writes k, v into the caches
// (B, H, Smax, D) at that position. sin / cos tables: (Smax, R/2). One thread per (b, h, feature pair).
// ------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
    rotary_append_kernel(T* __restrict__ qkv, long long ld, const T* __restrict__ sin_t, const T* __restrict__ cos_t,
                         T* __restrict__ k_cache, T* __restrict__ v_cache, const int* __restrict__ pos_ptr, int B, int H,
                         int D, int R, int Smax) {
  const int pos = *pos_ptr;
  if (pos < 0 || pos >= Smax) return;
  const int hd = H * D, half = D / 2;
  const long long total = (long long)B * H * half;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int d = 2 * (int)(i % half);
    const int h = (int)((i / half) % H);
    const int b = (int)(i / ((long long)half * H));
    T* q = qkv + (long long)b * ld + h * D + d;
    T* k = q + hd;
    const T* v = q + 2 * hd;
    float k0 = xl_to_float(k[0]), k1 = xl_to_float(k[1]);
    if (d < R) {
      const float sn = xl_to_float(sin_t[(long long)pos * (R / 2) + d / 2]);
      const float cs = xl_to_float(cos_t[(long long)pos * (R / 2) + d / 2]);
      const float q0 = xl_to_float(q[0]), q1 = xl_to_float(q[1]);
      q[0] = xl_from_float<T>(q0 * cs - q1 * sn);
      q[1] = xl_from_float<T>(q1 * cs + q0 * sn);
      const float r0 = k0 * cs - k1 * sn, r1 = k1 * cs + k0 * sn;
      k0 = r0;
      k1 = r1;
      k[0] = xl_from_float<T>(k0);
      k[1] = xl_from_float<T>(k1);
    }
    const long long dst = (((long long)b * H + h) * Smax + pos) * D + d;
    k_cache[dst] = xl_from_float<T>(k0);
    k_cache[dst + 1] = xl_from_float<T>(k1);
    v_cache[dst] = v[0];
    v_cache[dst + 1] = v[1];
  }
}

XL_API int xl_rotary_append(void* qkv, long long ld, const void* sin_t, const void* cos_t, void* k_cache, void* v_cache,
                            const int* pos_ptr, int B, int H, int D, int R, int Smax, int dtype, cudaStream_t s) {
  if ((D & 1) || (R & 1) || R > D) return -1;
  const long long total = (long long)B * H * (D / 2);
  const int grid = xl_grid_for(total, 256);
  XL_DISPATCH_DTYPE(dtype, T, {
    rotary_append_kernel<T><<<grid, 256, 0, s>>>((T*)qkv, ld, (const T*)sin_t, (const T*)cos_t, (T*)k_cache, (T*)v_cache,
                                                 pos_ptr, B, H, D, R, Smax);
  });
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------------------------
// Decode attention: one query per (b, h) against cache positions [0, len), len = *pos_ptr + 1, one launch.
// Grid (B*H, splits): each CTA covers a slice of the positions with an online softmax. A warp takes four positions per
// iteration (lanes over the head dimension, one vector load of D/32 values per lane, position and tensor), so eight
// independent loads are in flight per lane. Each CTA writes (max, sum, unnormalised output) of its slice; the last CTA
// of a (b, h) to finish (a counter per (b, h), left at zero again) merges the slices and writes the output row.
// ------------------------------------------------------------------------------------------------------------------
constexpr int AD_WARPS = 4;
constexpr int AD_MAX_D = 256;  // head_dim <= 256 (8 values per lane)
constexpr int AD_UNROLL = 4;

template <typename T, int VPL>
struct alignas(VPL * 2 >= 16 ? 16 : (VPL == 4 ? 8 : (VPL == 2 ? 4 : 2))) AdVec {
  T v[VPL];
};

template <typename T, int VPL>
__global__ void __launch_bounds__(AD_WARPS * 32)
    attn_decode_kernel(const T* __restrict__ qkv, long long ldq, const T* __restrict__ k_cache,
                       const T* __restrict__ v_cache, T* __restrict__ out, long long ldo, float* __restrict__ part,
                       unsigned int* __restrict__ counters, const int* __restrict__ pos_ptr, int H, int Smax, float scale) {
  constexpr int D = VPL * 32;
  using Vec = AdVec<T, VPL>;
  const int bh = blockIdx.x, split = blockIdx.y, splits = gridDim.y;
  const int b = bh / H, h = bh % H;
  const int len = min(*pos_ptr + 1, Smax);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per = (len + splits - 1) / splits;
  const int s_begin = split * per, s_end = min(len, s_begin + per);
  float q[VPL], o[VPL];
  {
    const Vec qv = *reinterpret_cast<const Vec*>(qkv + (long long)b * ldq + h * D + lane * VPL);
#pragma unroll
    for (int e = 0; e < VPL; ++e) {
      q[e] = xl_to_float(qv.v[e]) * scale;
      o[e] = 0.f;
    }
  }
  float m = -INFINITY, l = 0.f;
  const T* kb = k_cache + ((long long)bh * Smax) * D + lane * VPL;
  const T* vb = v_cache + ((long long)bh * Smax) * D + lane * VPL;
  for (int s0 = s_begin + warp * AD_UNROLL; s0 < s_end; s0 += AD_WARPS * AD_UNROLL) {
    Vec kk[AD_UNROLL], vv[AD_UNROLL];
#pragma unroll
    for (int u = 0; u < AD_UNROLL; ++u) {
      const int sidx = min(s0 + u, s_end - 1);  // clamped: the duplicates are masked out below
      kk[u] = *reinterpret_cast<const Vec*>(kb + (long long)sidx * D);
      vv[u] = *reinterpret_cast<const Vec*>(vb + (long long)sidx * D);
    }
    float dot[AD_UNROLL];
#pragma unroll
    for (int u = 0; u < AD_UNROLL; ++u) {
      float d = 0.f;
#pragma unroll
      for (int e = 0; e < VPL; ++e) d += q[e] * xl_to_float(kk[u].v[e]);
      dot[u] = d;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
      for (int u = 0; u < AD_UNROLL; ++u) dot[u] += __shfl_xor_sync(0xffffffffu, dot[u], off);
    }
    float m_new = m;
#pragma unroll
    for (int u = 0; u < AD_UNROLL; ++u) {
      if (s0 + u >= s_end) dot[u] = -INFINITY;
      m_new = fmaxf(m_new, dot[u]);
    }
    const float corr = __expf(m - m_new);  // m_new is finite here: position s0 is valid
    l *= corr;
#pragma unroll
    for (int e = 0; e < VPL; ++e) o[e] *= corr;
#pragma unroll
    for (int u = 0; u < AD_UNROLL; ++u) {
      const float p = __expf(dot[u] - m_new);  // exp(-inf) = 0 for the masked duplicates
      l += p;
#pragma unroll
      for (int e = 0; e < VPL; ++e) o[e] += p * xl_to_float(vv[u].v[e]);
    }
    m = m_new;
  }
  // merge the warps of this CTA
  __shared__ float sm[AD_WARPS], sl[AD_WARPS], so[AD_WARPS][AD_MAX_D];
  __shared__ unsigned int is_last;
  if (lane == 0) { sm[warp] = m; sl[warp] = l; }
#pragma unroll
  for (int e = 0; e < VPL; ++e) so[warp][lane * VPL + e] = o[e];
  __syncthreads();
  float* mine = part + ((long long)bh * splits + split) * (D + 2);
  if (warp == 0) {
    float mm = -INFINITY;
    for (int w = 0; w < AD_WARPS; ++w) mm = fmaxf(mm, sm[w]);
    float ll = 0.f;
    float acc[VPL];
#pragma unroll
    for (int e = 0; e < VPL; ++e) acc[e] = 0.f;
    for (int w = 0; w < AD_WARPS; ++w) {
      const float f = (sm[w] == -INFINITY) ? 0.f : __expf(sm[w] - mm);
      ll += sl[w] * f;
#pragma unroll
      for (int e = 0; e < VPL; ++e) acc[e] += so[w][lane * VPL + e] * f;
    }
    if (splits == 1) {
      const float inv = 1.f / ll;
      Vec r;
#pragma unroll
      for (int e = 0; e < VPL; ++e) r.v[e] = xl_from_float<T>(acc[e] * inv);
      *reinterpret_cast<Vec*>(out + (long long)b * ldo + h * D + lane * VPL) = r;
    } else {
      if (lane == 0) { mine[0] = mm; mine[1] = ll; }
#pragma unroll
      for (int e = 0; e < VPL; ++e) mine[2 + lane * VPL + e] = acc[e];
    }
  }
  if (splits == 1) return;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) is_last = atomicAdd(counters + bh, 1u) == (unsigned int)splits - 1;
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  const float* p = part + (long long)bh * splits * (D + 2);
  float mm = -INFINITY;
  for (int sp = 0; sp < splits; ++sp) mm = fmaxf(mm, __ldcg(p + sp * (D + 2)));
  float ll = 0.f;
  for (int sp = 0; sp < splits; ++sp) {
    const float ms = __ldcg(p + sp * (D + 2));
    ll += (ms == -INFINITY) ? 0.f : __ldcg(p + sp * (D + 2) + 1) * __expf(ms - mm);
  }
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float acc = 0.f;
    for (int sp = 0; sp < splits; ++sp) {
      const float ms = __ldcg(p + sp * (D + 2));
      if (ms != -INFINITY) acc += __ldcg(p + sp * (D + 2) + 2 + d) * __expf(ms - mm);
    }
    out[(long long)b * ldo + h * D + d] = xl_from_float<T>(acc / ll);
  }
  if (threadIdx.x == 0) counters[bh] = 0;
}

// q: rows of ldq elements (the first H*D are used); out: rows of ldo elements (H*D written). scratch: at least
// B*H*splits*(D+2) floats; counters: B*H zero-initialised words (left zeroed). D in {64, 128, 256}; ldq, ldo and the
// window offsets must keep every head 16-byte aligned.
XL_API int xl_attn_decode(const void* qkv, long long ldq, const void* k_cache, const void* v_cache, void* out, long long ldo,
                          float* scratch, unsigned int* counters, const int* pos_ptr, int B, int H, int D, int Smax,
                          float scale, int splits, int dtype, cudaStream_t s) {
  if ((D != 64 && D != 128 && D != 256) || splits < 1 || dtype == XL_F32 || (ldq % 8) || (ldo % 8)) return -1;
  if (splits > 1 && (scratch == nullptr || counters == nullptr)) return -1;
  dim3 grid(B * H, splits);
#define XL_AD_LAUNCH(T, VPL)                                                                                          \
  attn_decode_kernel<T, VPL><<<grid, AD_WARPS * 32, 0, s>>>((const T*)qkv, ldq, (const T*)k_cache, (const T*)v_cache, \
                                                            (T*)out, ldo, scratch, counters, pos_ptr, H, Smax, scale)
  if (dtype == XL_BF16) {
    if (D == 256) XL_AD_LAUNCH(__nv_bfloat16, 8);
    else if (D == 128) XL_AD_LAUNCH(__nv_bfloat16, 4);
    else XL_AD_LAUNCH(__nv_bfloat16, 2);
  } else {
    if (D == 256) XL_AD_LAUNCH(__half, 8);
    else if (D == 128) XL_AD_LAUNCH(__half, 4);
    else XL_AD_LAUNCH(__half, 2);
  }
#undef XL_AD_LAUNCH
  return (int)cudaGetLastError();
}

// N consecutive elements (N * sizeof(T) a multiple of 16, p 16-byte aligned) through 128-bit accesses
template <typename T, int N> __device__ __forceinline__ void xl_load_vec(const T* __restrict__ p, float (&out)[N]) {
  constexpr int PER = 16 / sizeof(T);
#pragma unroll
  for (int q = 0; q < N / PER; ++q) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p + q * PER);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < PER; ++i) out[q * PER + i] = xl_to_float(e[i]);
  }
}
template <typename T, int N> __device__ __forceinline__ void xl_store_vec(T* __restrict__ p, const float (&in)[N]) {
  constexpr int PER = 16 / sizeof(T);
#pragma unroll
  for (int q = 0; q < N / PER; ++q) {
    uint4 raw;
    T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int i = 0; i < PER; ++i) e[i] = xl_from_float<T>(in[q * PER + i]);
    *reinterpret_cast<uint4*>(p + q * PER) = raw;
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Residual update + LayerNorm for a few rows: x += delta (+ bias); h = LayerNorm(x) * w + b. One CTA per row.
// ------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
    add_layer_norm_kernel(T* __restrict__ x, const T* __restrict__ delta, const T* __restrict__ bias,
                          const T* __restrict__ w, const T* __restrict__ b, T* __restrict__ h, int cols, float eps) {
  constexpr int MAX_VEC = 4;  // vectors of 8 elements per thread: cols <= 256 * 8 * 4
  const int row = blockIdx.x;
  T* xr = x + (long long)row * cols;
  float v[MAX_VEC][8];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < MAX_VEC; ++i) {
    const int c = (threadIdx.x + i * 256) * 8;
    if (c < cols) {
      xl_load_vec<T, 8>(xr + c, v[i]);
      if (delta) {
        float d[8];
        xl_load_vec<T, 8>(delta + (long long)row * cols + c, d);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[i][e] += d[e];
      }
      if (bias) {
        float d[8];
        xl_load_vec<T, 8>(bias + c, d);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[i][e] += d[e];
      }
      if (delta || bias) {
        xl_store_vec<T, 8>(xr + c, v[i]);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[i][e] = xl_to_float(xl_from_float<T>(v[i][e]));  // what later readers of x see
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) sum += v[i][e];
    }
  }
  __shared__ float red[8];
  __shared__ float stat[2];
  sum = xl_warp_sum(sum);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < 8; ++i) t += red[i];
    stat[0] = t / cols;
  }
  __syncthreads();
  const float mean = stat[0];
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < MAX_VEC; ++i) {
    const int c = (threadIdx.x + i * 256) * 8;
    if (c < cols) {
#pragma unroll
      for (int e = 0; e < 8; ++e) sq += (v[i][e] - mean) * (v[i][e] - mean);
    }
  }
  sq = xl_warp_sum(sq);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sq;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < 8; ++i) t += red[i];
    stat[1] = rsqrtf(t / cols + eps);
  }
  __syncthreads();
  const float rstd = stat[1];
#pragma unroll
  for (int i = 0; i < MAX_VEC; ++i) {
    const int c = (threadIdx.x + i * 256) * 8;
    if (c < cols) {
      float wv[8], bv[8], o[8];
      xl_load_vec<T, 8>(w + c, wv);
      xl_load_vec<T, 8>(b + c, bv);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = (v[i][e] - mean) * rstd * wv[e] + bv[e];
      xl_store_vec<T, 8>(h + (long long)row * cols + c, o);
    }
  }
}

// x (rows, cols) is updated in place when delta or bias is given; h (rows, cols) receives the normalised rows.
XL_API int xl_add_layer_norm(void* x, const void* delta, const void* bias, const void* w, const void* b, void* h,
                             int rows, int cols, float eps, int dtype, cudaStream_t s) {
  if (cols > 256 * 32 || (cols % 8) || rows < 1 || w == nullptr || b == nullptr) return -1;
  XL_DISPATCH_DTYPE(dtype, T, {
    add_layer_norm_kernel<T><<<rows, 256, 0, s>>>((T*)x, (const T*)delta, (const T*)bias, (const T*)w, (const T*)b, (T*)h,
                                                 cols, eps);
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
