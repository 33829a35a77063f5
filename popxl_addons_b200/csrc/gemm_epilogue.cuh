// The plain (non-collective) epilogue of a tcgen05 GEMM: accumulator columns as read from TMEM -> C in global memory.
#pragma once
#include "common.cuh"

#include <math.h>

namespace {  // internal linkage: every kernel file that includes this gets its own copy

struct EpilogueParams {
  int N;           // columns of C: stores and bias reads stop there
  int c_dtype;     // XL_F32 / XL_F16 / XL_BF16
  const void* bias;  // length N, may be null
  int bias_dtype;
  int act;         // 0 none, 1 gelu(erf), 2 gelu(tanh), 3 relu
  int accumulate;  // 0 overwrite, 1 C += alpha*acc, 2 running mean: C = C*mean_a + alpha*acc*mean_b
};

__device__ __forceinline__ float apply_act(float v, int act) {
  if (act == 1) return 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
  if (act == 2) return 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
  if (act == 3) return fmaxf(v, 0.f);
  return v;
}

// One thread's 32 consecutive accumulator columns (row `crow`, columns col0 .. col0 + 31) -> scale, bias, activation,
// optional accumulation into the old contents, conversion and store. The caller has checked row < M and col0 < N.
__device__ __forceinline__ void epilogue_store_32cols(const EpilogueParams& p, const uint32_t (&r)[32], uint8_t* crow,
                                                      int col0, float alpha_eff, float mean_a, float mean_b) {
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * alpha_eff;
    if (p.bias) {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (col0 + j < p.N) {
          float bv;
          if (p.bias_dtype == XL_F32) bv = ((const float*)p.bias)[col0 + j];
          else if (p.bias_dtype == XL_BF16) bv = __bfloat162float(((const __nv_bfloat16*)p.bias)[col0 + j]);
          else bv = __half2float(((const __half*)p.bias)[col0 + j]);
          v[j] += bv;
        }
      }
    }
    if (p.act) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = apply_act(v[j], p.act);
    }
    const bool full = (col0 + 32 <= p.N);
    if (p.c_dtype == XL_F32) {
      float* dst = (float*)crow + col0;
      if (full && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
          if (p.accumulate) {
            const float4 old = *(const float4*)(dst + j);
            if (p.accumulate == 1) { o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w; }
            else { o.x = old.x * mean_a + o.x * mean_b; o.y = old.y * mean_a + o.y * mean_b;
                   o.z = old.z * mean_a + o.z * mean_b; o.w = old.w * mean_a + o.w * mean_b; }
          }
          *(float4*)(dst + j) = o;
        }
      } else {
        for (int j = 0; j < 32 && col0 + j < p.N; ++j) {
          float o = v[j];
          if (p.accumulate == 1) o += dst[j];
          else if (p.accumulate == 2) o = dst[j] * mean_a + o * mean_b;
          dst[j] = o;
        }
      }
    } else {
      uint16_t* dst = (uint16_t*)crow + col0;
      const bool bf = p.c_dtype == XL_BF16;
      if (full && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          uint4 old;
          if (p.accumulate) old = *(const uint4*)(dst + j);
          uint4 o;
          uint16_t* oe = (uint16_t*)&o;
          const uint16_t* ol = (const uint16_t*)&old;
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            float val = v[j + e];
            if (p.accumulate) {
              const float prev = bf ? __bfloat162float(__ushort_as_bfloat16(ol[e])) : __half2float(__ushort_as_half(ol[e]));
              val = p.accumulate == 1 ? prev + val : prev * mean_a + val * mean_b;
            }
            oe[e] = bf ? __bfloat16_as_ushort(__float2bfloat16_rn(val)) : __half_as_ushort(__float2half_rn(val));
          }
          *(uint4*)(dst + j) = o;
        }
      } else {
        for (int j = 0; j < 32 && col0 + j < p.N; ++j) {
          float val = v[j];
          if (p.accumulate) {
            const float prev = bf ? __bfloat162float(__ushort_as_bfloat16(dst[j])) : __half2float(__ushort_as_half(dst[j]));
            val = p.accumulate == 1 ? prev + val : prev * mean_a + val * mean_b;
          }
          dst[j] = bf ? __bfloat16_as_ushort(__float2bfloat16_rn(val)) : __half_as_ushort(__float2half_rn(val));
        }
      }
    }
}

}  // namespace
