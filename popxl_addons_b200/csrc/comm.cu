// Collective kernels over symmetric memory (peer loads / stores over NVLink, bounded waits):
//   xl_symm_barrier          cross-rank barrier on a signal pad (stream-ordered fence between phases of a step)
//   xl_symm_all_reduce       one-shot all-reduce of a small fp32 vector (statistics of sharded cross-entropy / LayerNorm)
//   xl_rts_adam              replicated-tensor-sharding optimizer step in ONE kernel:
//                            gradient reduce-scatter (each rank reads its shard of every peer's accumulator), mean,
//                            AdamW on the local fp32 master / moment shards, and all-gather of the updated 16-bit
//                            weights (each rank stores its shard into every peer's weight buffer)
#include "comm.cuh"

unsigned int xl_host_comm_spin_limit = XL_COMM_SPIN_DEFAULT;

// Set the poll budget of all later waits on peers (0 restores the default).
XL_API int xl_set_comm_spin_limit(unsigned int polls) {
  xl_host_comm_spin_limit = polls ? polls : XL_COMM_SPIN_DEFAULT;
  return 0;
}

__global__ void symm_barrier_kernel(unsigned int* const* pads, int rank, int world, int channel, int* err,
                                    unsigned int limit) {
  xl_group_barrier(pads, rank, world, channel, err, limit);
}

XL_API int xl_symm_barrier(const void* pads_dev, int rank, int world, int channel, int* err, cudaStream_t s) {
  if (world > 32) return -1;
  symm_barrier_kernel<<<1, 32, 0, s>>>((unsigned int* const*)pads_dev, rank, world, channel, err,
                                       xl_host_comm_spin_limit);
  return (int)cudaGetLastError();
}

// Every rank has written its `n` floats at `offset` of its own symmetric buffer before the launch (stream order).
// op: 0 add, 1 max. One CTA: the message is a few thousand elements at most (latency-bound by design).
__global__ void __launch_bounds__(1024)
    symm_all_reduce_kernel(float* const* bufs, unsigned int* const* pads, long long offset, float* out, int n, int op,
                           int rank, int world, int channel, int* err, unsigned int limit) {
  __shared__ int ok_s;
  if (threadIdx.x < 32) {
    const bool ok = xl_group_barrier(pads, rank, world, channel, err, limit);
    if (threadIdx.x == 0) ok_s = ok;
  }
  __syncthreads();
  if (ok_s) {
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      float acc = op == 0 ? 0.f : -INFINITY;
      for (int p = 0; p < world; ++p) {
        const float v = bufs[p][offset + i];
        acc = op == 0 ? acc + v : fmaxf(acc, v);
      }
      out[i] = acc;
    }
  }
  __syncthreads();
  // peers may overwrite their buffers only after everyone has read them
  if (threadIdx.x < 32) xl_group_barrier(pads, rank, world, channel + 1, err, limit);
}

XL_API int xl_symm_all_reduce(const void* bufs_dev, const void* pads_dev, long long offset_elems, float* out, int n,
                              int op, int rank, int world, int channel, int* err, cudaStream_t s) {
  if (world > 32 || n <= 0) return -1;
  symm_all_reduce_kernel<<<1, 1024, 0, s>>>((float* const*)bufs_dev, (unsigned int* const*)pads_dev, offset_elems, out,
                                             n, op, rank, world, channel, err, xl_host_comm_spin_limit);
  return (int)cudaGetLastError();
}

struct RtsAdamArgs {
  float lr, beta1, beta2, eps, weight_decay, grad_scale;
  int bias_correction;
};

constexpr int RTS_MAX_WORLD = 8;
struct RtsPtrs {
  const float* grads[RTS_MAX_WORLD];  // every rank's full gradient accumulator (fp32)
  void* weights[RTS_MAX_WORLD];       // every rank's full 16-bit weight tensor
};

// shard = elements [shard_off, shard_off + shard_n) of the flattened tensor; shard_off and shard_n are multiples of 4.
template <typename TW, typename TM>
__global__ void __launch_bounds__(256)
    rts_adam_kernel(RtsPtrs ptrs, float* __restrict__ master, TM* __restrict__ m, float* __restrict__ v,
                    const float* __restrict__ step, long long shard_off, long long shard_n, int world, RtsAdamArgs a) {
  float c1 = 1.f, c2 = 1.f;
  if (step != nullptr && a.bias_correction) {
    const float t = *step;
    c1 = 1.f / (1.f - powf(a.beta1, t));
    c2 = 1.f / (1.f - powf(a.beta2, t));
  }
  const float inv_world = 1.f / world;
  const long long nvec = shard_n / 4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    const long long e = i * 4;
    float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int p = 0; p < world; ++p) {  // reduce-scatter: my shard of every peer's gradient
      const float4 t = *reinterpret_cast<const float4*>(ptrs.grads[p] + shard_off + e);
      g.x += t.x; g.y += t.y; g.z += t.z; g.w += t.w;
    }
    float gv[4] = {g.x, g.y, g.z, g.w};
    const float4 w4 = *reinterpret_cast<const float4*>(master + e);
    const float4 v4 = *reinterpret_cast<const float4*>(v + e);
    float wv[4] = {w4.x, w4.y, w4.z, w4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
    TW wq[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float gf = gv[k] * inv_world * a.grad_scale;
      const float mf = xl_to_float(m[e + k]) * a.beta1 + gf * (1.f - a.beta1);
      vv[k] = vv[k] * a.beta2 + gf * gf * (1.f - a.beta2);
      const TM mq = xl_from_float<TM>(mf);
      m[e + k] = mq;
      const float upd = (xl_to_float(mq) * c1) / (sqrtf(vv[k] * c2) + a.eps) + wv[k] * a.weight_decay;
      wv[k] -= a.lr * upd;
      wq[k] = xl_from_float<TW>(wv[k]);
    }
    *reinterpret_cast<float4*>(master + e) = make_float4(wv[0], wv[1], wv[2], wv[3]);
    *reinterpret_cast<float4*>(v + e) = make_float4(vv[0], vv[1], vv[2], vv[3]);
    const uint2 packed = *reinterpret_cast<const uint2*>(wq);
    for (int p = 0; p < world; ++p)  // all-gather: my shard into every peer's weights
      *reinterpret_cast<uint2*>((TW*)ptrs.weights[p] + shard_off + e) = packed;
  }
}

__global__ void rts_step_increment_kernel(float* step) { *step += 1.f; }

// grads / weights: host arrays of `world` device pointers (this rank's own pointer included at index `rank`).
// Call between two xl_symm_barrier launches: the first guarantees that every rank's accumulators are final, the second
// that every rank's weight shards have arrived before the weights are used.
XL_API int xl_rts_adam(const void* const* grads, void* const* weights, int w_dtype, float* master, void* m, int m_dtype,
                       float* v, float* step, long long shard_off, long long shard_n, int world, float lr, float beta1,
                       float beta2, float eps, float weight_decay, float grad_scale, int bias_correction,
                       cudaStream_t s) {
  if (world > RTS_MAX_WORLD || (shard_off & 3) || (shard_n & 3)) return -1;
  if (w_dtype != XL_BF16 && w_dtype != XL_F16) return -1;
  RtsPtrs ptrs;
  for (int p = 0; p < world; ++p) {
    ptrs.grads[p] = (const float*)grads[p];
    ptrs.weights[p] = weights[p];
  }
  RtsAdamArgs a{lr, beta1, beta2, eps, weight_decay, grad_scale, bias_correction};
  if (step) rts_step_increment_kernel<<<1, 1, 0, s>>>(step);
  const int grid = xl_grid_for(shard_n / 4, 256, 148 * 8);
#define XL_RTS_LAUNCH(TW, TM) \
  rts_adam_kernel<TW, TM><<<grid, 256, 0, s>>>(ptrs, master, (TM*)m, v, step, shard_off, shard_n, world, a)
  if (w_dtype == XL_BF16) {
    if (m_dtype == XL_F32) XL_RTS_LAUNCH(__nv_bfloat16, float);
    else if (m_dtype == XL_BF16) XL_RTS_LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else XL_RTS_LAUNCH(__nv_bfloat16, __half);
  } else {
    if (m_dtype == XL_F32) XL_RTS_LAUNCH(__half, float);
    else if (m_dtype == XL_BF16) XL_RTS_LAUNCH(__half, __nv_bfloat16);
    else XL_RTS_LAUNCH(__half, __half);
  }
#undef XL_RTS_LAUNCH
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------------------------------
// Replicated-tensor-sharding optimizer step over a bucket of parameters (one launch per bucket, e.g. per layer).
// Every parameter of the bucket is a segment: its 16-bit weight and its fp32 gradient accumulator live at the same offset
// of every rank's symmetric arena; this rank owns elements [shard_off, shard_off + shard_n) of it, together with the
// fp32 master weights and the moments of that range. Work is cut into chunks of RTS_CHUNK elements of the owned ranges,
// numbered across the segments; a CTA finds a chunk's segment in the (short) table.
//   mode 0  reduce-scatter (mean over the ranks, read from every rank's accumulator) + AdamW + all-gather (16-bit
//           weights written into every rank's weight), all in one pass
//   mode 1  reduce-scatter only: the mean goes into this rank's own accumulator (its owned range), and the sum of
//           squares of (mean * grad_scale) over the owned ranges is added to *sumsq (per-CTA partials, summed in a
//           fixed order by a second tiny kernel: deterministic). For global-norm clipping: the caller all-reduces the sums
//           of all buckets, derives the clip factor, then runs mode 2.
//   mode 2  AdamW + all-gather from the reduced gradient that mode 1 left in the own accumulator, scaled by
//           grad_scale * (*dyn_scale) (dyn_scale: device scalar, e.g. the clip factor; may be null)
// ---------------------------------------------------------------------------------------------------------------------
constexpr int RTS_CHUNK = 4096;  // elements per chunk: 256 threads x 4 vectors of 4

struct RtsSegment {            // one parameter of the bucket (device memory, 64 bytes)
  long long acc_off;           // byte offset of the fp32 accumulator in every rank's arena
  long long w_off;             // byte offset of the 16-bit weight in every rank's arena
  float* master;               // this rank's shard of the fp32 master weights
  void* m;                     // first moment of the shard (fp32 / fp16 / bf16)
  float* v;                    // second moment of the shard
  long long shard_off;         // first owned element
  long long shard_n;           // owned elements (multiple of 4)
  float weight_decay;
  int chunk0;                  // number of the segment's first chunk
};

template <typename TM> struct RtsVec4;
template <> struct RtsVec4<float> {
  static __device__ __forceinline__ void load(const float* p, float (&o)[4]) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    o[0] = t.x; o[1] = t.y; o[2] = t.z; o[3] = t.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&o)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(o[0], o[1], o[2], o[3]);
  }
};
template <typename T16> struct RtsVec4_16 {  // four 16-bit values as one 8-byte access
  static __device__ __forceinline__ void load(const T16* p, float (&o)[4]) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const T16* e = reinterpret_cast<const T16*>(&raw);
#pragma unroll
    for (int k = 0; k < 4; ++k) o[k] = xl_to_float(e[k]);
  }
  static __device__ __forceinline__ void store(T16* p, const float (&o)[4]) {
    uint2 raw;
    T16* e = reinterpret_cast<T16*>(&raw);
#pragma unroll
    for (int k = 0; k < 4; ++k) e[k] = xl_from_float<T16>(o[k]);
    *reinterpret_cast<uint2*>(p) = raw;
  }
};
template <> struct RtsVec4<__half> : RtsVec4_16<__half> {};
template <> struct RtsVec4<__nv_bfloat16> : RtsVec4_16<__nv_bfloat16> {};

template <typename TW, typename TM>
__global__ void __launch_bounds__(256)
    rts_adam_multi_kernel(const RtsSegment* __restrict__ segs, int n_seg, int total_chunks, uint8_t* const* bases, int rank,
                          int world, int mode, const float* __restrict__ step, const float* __restrict__ dyn_scale,
                          float* __restrict__ partials, RtsAdamArgs a) {
  __shared__ float red[32];
  float c1 = 1.f, c2 = 1.f;
  if (step != nullptr && a.bias_correction) {
    const float t = *step;
    c1 = 1.f / (1.f - powf(a.beta1, t));
    c2 = 1.f / (1.f - powf(a.beta2, t));
  }
  const float inv_world = 1.f / world;
  const float gscale = a.grad_scale * (dyn_scale != nullptr ? *dyn_scale : 1.f);
  float sq = 0.f;
  for (int chunk = blockIdx.x; chunk < total_chunks; chunk += gridDim.x) {
    int si = 0;
    while (si + 1 < n_seg && segs[si + 1].chunk0 <= chunk) ++si;
    const RtsSegment sg = segs[si];
    const long long e0 = (long long)(chunk - sg.chunk0) * RTS_CHUNK;
#pragma unroll
    for (int u = 0; u < RTS_CHUNK / (256 * 4); ++u) {
      const long long e = e0 + ((long long)u * 256 + threadIdx.x) * 4;
      if (e >= sg.shard_n) continue;
      float g[4] = {0.f, 0.f, 0.f, 0.f};
      if (mode == 2) {  // already reduced into the own accumulator
        RtsVec4<float>::load(reinterpret_cast<const float*>(bases[rank] + sg.acc_off) + sg.shard_off + e, g);
      } else {
        for (int p = 0; p < world; ++p) {  // reduce-scatter: my range of every rank's accumulator
          float t[4];
          RtsVec4<float>::load(reinterpret_cast<const float*>(bases[p] + sg.acc_off) + sg.shard_off + e, t);
#pragma unroll
          for (int k = 0; k < 4; ++k) g[k] += t[k];
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) g[k] *= inv_world;
      }
      if (mode == 1) {
        RtsVec4<float>::store(reinterpret_cast<float*>(bases[rank] + sg.acc_off) + sg.shard_off + e, g);
#pragma unroll
        for (int k = 0; k < 4; ++k) sq += (g[k] * a.grad_scale) * (g[k] * a.grad_scale);
        continue;
      }
      float wv[4], vv[4], mv[4], wq[4];
      RtsVec4<float>::load(sg.master + e, wv);
      RtsVec4<float>::load(sg.v + e, vv);
      RtsVec4<TM>::load(reinterpret_cast<const TM*>(sg.m) + e, mv);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float gf = g[k] * gscale;
        // the moment is rounded to its storage type before it is used, so the update equals one computed from the
        // stored state
        mv[k] = xl_to_float(xl_from_float<TM>(mv[k] * a.beta1 + gf * (1.f - a.beta1)));
        vv[k] = vv[k] * a.beta2 + gf * gf * (1.f - a.beta2);
        const float upd = (mv[k] * c1) / (sqrtf(vv[k] * c2) + a.eps) + wv[k] * sg.weight_decay;
        wv[k] -= a.lr * upd;
        wq[k] = wv[k];
      }
      RtsVec4<float>::store(sg.master + e, wv);
      RtsVec4<float>::store(sg.v + e, vv);
      RtsVec4<TM>::store(reinterpret_cast<TM*>(sg.m) + e, mv);
      uint2 packed;
      {
        TW* q = reinterpret_cast<TW*>(&packed);
#pragma unroll
        for (int k = 0; k < 4; ++k) q[k] = xl_from_float<TW>(wq[k]);
      }
      for (int p = 0; p < world; ++p)  // all-gather: my range into every rank's weight
        *reinterpret_cast<uint2*>(reinterpret_cast<TW*>(bases[p] + sg.w_off) + sg.shard_off + e) = packed;
    }
  }
  if (mode == 1) {
    sq = xl_block_sum(sq, red);
    if (threadIdx.x == 0) partials[blockIdx.x] = sq;
  }
}

__global__ void rts_sumsq_finish_kernel(const float* __restrict__ partials, int n, float* __restrict__ sumsq) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < n; ++i) t += partials[i];
    *sumsq += t;
  }
}

// Grid size (= number of per-CTA partial sums of mode 1) for a bucket of `total_chunks` chunks.
XL_API int xl_rts_adam_multi_grid(int total_chunks) { return xl_grid_for(total_chunks, 1, 148 * 8); }

// segs: device array of n_seg RtsSegment; bases: device array [world] with every rank's arena base; step: device scalar
// incremented by this call in modes 0 and 2 (may be null); partials: xl_rts_adam_multi_grid(total_chunks) floats of scratch
// (mode 1); sumsq: device scalar that mode 1 adds to. Call between barriers as xl_rts_adam.
XL_API int xl_rts_adam_multi(const void* segs, int n_seg, int total_chunks, const void* bases, int rank, int world, int mode,
                             int w_dtype, int m_dtype, float* step, const float* dyn_scale, float* partials, float* sumsq,
                             float lr, float beta1, float beta2, float eps, float grad_scale, int bias_correction,
                             cudaStream_t s) {
  if (n_seg <= 0 || total_chunks <= 0 || world < 1 || world > 64 || mode < 0 || mode > 2) return -1;
  if (w_dtype != XL_BF16 && w_dtype != XL_F16) return -1;
  if (mode == 1 && (partials == nullptr || sumsq == nullptr)) return -1;
  RtsAdamArgs a{lr, beta1, beta2, eps, 0.f, grad_scale, bias_correction};
  if (step && mode != 1) rts_step_increment_kernel<<<1, 1, 0, s>>>(step);
  const int grid = xl_rts_adam_multi_grid(total_chunks);
#define XL_RTS_MULTI(TW, TM)                                                                                             \
  rts_adam_multi_kernel<TW, TM><<<grid, 256, 0, s>>>((const RtsSegment*)segs, n_seg, total_chunks, (uint8_t* const*)bases, \
                                                     rank, world, mode, step, dyn_scale, partials, a)
  if (w_dtype == XL_BF16) {
    if (m_dtype == XL_F32) XL_RTS_MULTI(__nv_bfloat16, float);
    else if (m_dtype == XL_BF16) XL_RTS_MULTI(__nv_bfloat16, __nv_bfloat16);
    else XL_RTS_MULTI(__nv_bfloat16, __half);
  } else {
    if (m_dtype == XL_F32) XL_RTS_MULTI(__half, float);
    else if (m_dtype == XL_BF16) XL_RTS_MULTI(__half, __nv_bfloat16);
    else XL_RTS_MULTI(__half, __half);
  }
#undef XL_RTS_MULTI
  if (mode == 1) rts_sumsq_finish_kernel<<<1, 32, 0, s>>>(partials, grid, sumsq);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------------------------------
// All-gather by multicast: every rank stores its shard (nbytes, a multiple of 16) at byte offset rank * nbytes of a
// buffer in every rank's symmetric memory with multimem.st (one store per 16 bytes reaches all ranks through NVSwitch),
// then the ranks meet at a barrier, so that when the kernel has finished on a rank the whole buffer is valid there.
// state: one zero-initialised device word of this rank (the kernel leaves it zero); uses signal channel `channel`.
// ---------------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(512)
    symm_all_gather_mc_kernel(const uint4* __restrict__ src, char* dst_mc, long long nvec, unsigned int* state,
                              unsigned int* const* pads, int rank, int world, int channel, int* err, unsigned int limit) {
  __shared__ int last_s;
  char* dst = dst_mc + (long long)rank * nvec * 16;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x)
    xl_multimem_st_b128(dst + i * 16, src[i]);
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int ticket = atomicAdd(state, 1u);
    last_s = ticket == gridDim.x - 1;
    if (last_s) *state = 0;
  }
  __syncthreads();
  if (last_s && threadIdx.x < 32) xl_group_barrier(pads, rank, world, channel, err, limit);
}

XL_API int xl_symm_all_gather_mc(const void* src, void* dst_mc, long long nbytes, unsigned int* state, const void* pads_dev,
                                 int rank, int world, int channel, int* err, cudaStream_t s) {
  if (world > 32 || nbytes <= 0 || (nbytes & 15) || (((uintptr_t)src) & 15) || (((uintptr_t)dst_mc) & 15)) return -1;
  const long long nvec = nbytes / 16;
  const int grid = xl_grid_for(nvec, 512 * 4, 64);
  symm_all_gather_mc_kernel<<<grid, 512, 0, s>>>((const uint4*)src, (char*)dst_mc, nvec, state,
                                                 (unsigned int* const*)pads_dev, rank, world, channel, err,
                                                 xl_host_comm_spin_limit);
  return (int)cudaGetLastError();
}

// One-shot all-reduce (sum) of a small 16-bit tensor, latency-bound (the 128 KiB activations of token-by-token decoding).
// Every rank copies its input into one half of a staging buffer in symmetric memory, the ranks meet at a barrier, and
// every rank reads the sum of all replicas of that half through the multicast address (`multimem.ld_reduce`: NVSwitch
// adds the replicas, fp32 accumulation). The work is split over up to MC_MAX_CTAS CTAs; CTA b handles slice b on every
// rank and synchronises only with the peers' CTA b (signal channel `channel + b`), so no grid-wide step is needed.
// The halves alternate from call to call (a counter in device memory, advanced by the last CTA to finish): a rank can
// only reach the next use of a half after every peer has passed the barrier of the call in between, i.e. has finished
// reading it, so no closing barrier is needed and the launch has no argument that changes between calls (it can be
// replayed from a CUDA graph).
constexpr int MC_MAX_CTAS = 16;
constexpr int MC_THREADS = 512;

__global__ void __launch_bounds__(MC_THREADS)
    symm_all_reduce_mc_kernel(const uint4* __restrict__ in, uint4* stage_local, const char* stage_mc, long long half_bytes,
                              unsigned int* state, unsigned int* const* pads, uint4* __restrict__ out, int nvec, int bf16,
                              int rank, int world, int channel, int* err, unsigned int limit) {
  __shared__ int ok_s;
  const unsigned int parity = *((volatile unsigned int*)state) & 1u;
  const int per = (nvec + gridDim.x - 1) / gridDim.x;
  const int v0 = blockIdx.x * per, v1 = min(nvec, v0 + per);
  uint4* mine = stage_local + parity * (half_bytes / 16);
  for (int i = v0 + threadIdx.x; i < v1; i += blockDim.x) mine[i] = in[i];
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < 32) {
    const bool ok = xl_group_barrier(pads, rank, world, channel + blockIdx.x, err, limit);
    if (threadIdx.x == 0) ok_s = ok;
  }
  __syncthreads();
  if (ok_s) {
    const char* src = stage_mc + parity * half_bytes;
    for (int i = v0 + threadIdx.x; i < v1; i += blockDim.x) {
      uint4 v;
      const char* a = src + (size_t)i * 16;
      if (bf16)
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(a) : "memory");
      else
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(a) : "memory");
      out[i] = v;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int ticket = atomicAdd(state + 1, 1u);
    if (ticket == gridDim.x - 1) {
      state[1] = 0;
      __threadfence();
      *((volatile unsigned int*)state) = parity + 1u;  // the next call uses the other half
    }
  }
}

// in / out: this rank's input and result (nbytes, a multiple of 16, at most half_bytes); stage_local / stage_mc: local
// and multicast address of a staging buffer of 2 * half_bytes in symmetric memory; state: two zero-initialised words of
// this rank; uses signal channels channel .. channel + 15.
XL_API int xl_symm_all_reduce_mc(const void* in, void* stage_local, const void* stage_mc, long long half_bytes,
                                 unsigned int* state, const void* pads_dev, void* out, long long nbytes, int dtype,
                                 int rank, int world, int channel, int* err, cudaStream_t s) {
  if (world > 32 || nbytes <= 0 || (nbytes & 15) || nbytes > half_bytes || (half_bytes & 15) || dtype == XL_F32) return -1;
  const int nvec = (int)(nbytes / 16);
  int grid = (nvec + MC_THREADS - 1) / MC_THREADS;
  if (grid > MC_MAX_CTAS) grid = MC_MAX_CTAS;
  symm_all_reduce_mc_kernel<<<grid, MC_THREADS, 0, s>>>((const uint4*)in, (uint4*)stage_local, (const char*)stage_mc,
                                                       half_bytes, state, (unsigned int* const*)pads_dev, (uint4*)out,
                                                       nvec, dtype == XL_BF16, rank, world, channel, err,
                                                       xl_host_comm_spin_limit);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------------------------------
// Decode step: all-reduce of the layer output fused with the residual update and the next LayerNorm.
//   x += sum over ranks(delta_partial) (+ bias);  h = LayerNorm(x) * w + b          rows <= 16, one CTA per row
// Same protocol as the one-shot all-reduce above (and the same staging halves, counter and signal channels, so the two
// kernels can be mixed in one program): CTA r copies row r of this rank's partial result into the current half, meets
// the peers' CTA r at a barrier, reads the sum of all replicas of the row through the multicast address and normalises
// it. One launch replaces staging copy + all-reduce + residual add + LayerNorm.
// ---------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
    ar_add_layer_norm_kernel(T* __restrict__ x, const T* __restrict__ delta_partial, const T* __restrict__ bias,
                             const T* __restrict__ w, const T* __restrict__ b, T* __restrict__ h, int cols, float eps,
                             uint4* stage_local, const char* stage_mc, long long half_bytes, unsigned int* state,
                             unsigned int* const* pads, int rank, int world, int channel, int* err, unsigned int limit) {
  constexpr int MAX_VEC = 4;  // vectors of 8 elements per thread: cols <= 256 * 8 * 4
  __shared__ int ok_s;
  __shared__ float red[8];
  __shared__ float stat[2];
  const int row = blockIdx.x;
  const int nvec = cols / 8;
  const unsigned int parity = *((volatile unsigned int*)state) & 1u;
  uint4* mine = stage_local + parity * (half_bytes / 16) + (long long)row * nvec;
  const uint4* src = reinterpret_cast<const uint4*>(delta_partial + (long long)row * cols);
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) mine[i] = src[i];
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < 32) {
    const bool ok = xl_group_barrier(pads, rank, world, channel + row, err, limit);
    if (threadIdx.x == 0) ok_s = ok;
  }
  __syncthreads();
  const bool ok = ok_s != 0;
  const char* red_src = stage_mc + parity * half_bytes + (long long)row * nvec * 16;
  T* xr = x + (long long)row * cols;
  float v[MAX_VEC][8];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < MAX_VEC; ++i) {
    const int vi = threadIdx.x + i * 256;
    if (vi < nvec) {
      uint4 raw = make_uint4(0, 0, 0, 0);
      if (ok) {
        const char* a = red_src + (size_t)vi * 16;
        if (std::is_same<T, __nv_bfloat16>::value)
          asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                       : "=r"(raw.x), "=r"(raw.y), "=r"(raw.z), "=r"(raw.w) : "l"(a) : "memory");
        else
          asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                       : "=r"(raw.x), "=r"(raw.y), "=r"(raw.z), "=r"(raw.w) : "l"(a) : "memory");
      }
      const T* de = reinterpret_cast<const T*>(&raw);
      const uint4 xraw = *reinterpret_cast<const uint4*>(xr + vi * 8);
      const T* xe = reinterpret_cast<const T*>(&xraw);
      uint4 braw = make_uint4(0, 0, 0, 0);
      if (bias) braw = *reinterpret_cast<const uint4*>(bias + vi * 8);
      const T* be = reinterpret_cast<const T*>(&braw);
      uint4 oraw;
      T* oe = reinterpret_cast<T*>(&oraw);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float t = xl_to_float(xe[e]) + xl_to_float(de[e]);
        if (bias) t += xl_to_float(be[e]);
        oe[e] = xl_from_float<T>(t);
        v[i][e] = xl_to_float(oe[e]);
        sum += v[i][e];
      }
      *reinterpret_cast<uint4*>(xr + vi * 8) = oraw;
    }
  }
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
    const int vi = threadIdx.x + i * 256;
    if (vi < nvec) {
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
    const int vi = threadIdx.x + i * 256;
    if (vi < nvec) {
      const uint4 wraw = *reinterpret_cast<const uint4*>(w + vi * 8), bbraw = *reinterpret_cast<const uint4*>(b + vi * 8);
      const T* we = reinterpret_cast<const T*>(&wraw);
      const T* bbe = reinterpret_cast<const T*>(&bbraw);
      uint4 oraw;
      T* oe = reinterpret_cast<T*>(&oraw);
#pragma unroll
      for (int e = 0; e < 8; ++e) oe[e] = xl_from_float<T>((v[i][e] - mean) * rstd * xl_to_float(we[e]) + xl_to_float(bbe[e]));
      *reinterpret_cast<uint4*>(h + (long long)row * cols + vi * 8) = oraw;
    }
  }
  if (threadIdx.x == 0) {
    const unsigned int ticket = atomicAdd(state + 1, 1u);
    if (ticket == gridDim.x - 1) {
      state[1] = 0;
      __threadfence();
      *((volatile unsigned int*)state) = parity + 1u;
    }
  }
}

// rows <= 16, cols % 8 == 0, cols <= 8192, rows * cols * 2 <= half_bytes, 16-bit dtype. Returns -1 otherwise.
XL_API int xl_ar_add_layer_norm(void* x, const void* delta_partial, const void* bias, const void* w, const void* b, void* h,
                                int rows, int cols, float eps, int dtype, void* stage_local, const void* stage_mc,
                                long long half_bytes, unsigned int* state, const void* pads_dev, int rank, int world,
                                int channel, int* err, cudaStream_t s) {
  if (rows < 1 || rows > 16 || (cols % 8) || cols > 8192 || dtype == XL_F32 || world > 32 ||
      (long long)rows * cols * 2 > half_bytes || w == nullptr || b == nullptr)
    return -1;
  if (dtype == XL_BF16)
    ar_add_layer_norm_kernel<__nv_bfloat16><<<rows, 256, 0, s>>>(
        (__nv_bfloat16*)x, (const __nv_bfloat16*)delta_partial, (const __nv_bfloat16*)bias, (const __nv_bfloat16*)w,
        (const __nv_bfloat16*)b, (__nv_bfloat16*)h, cols, eps, (uint4*)stage_local, (const char*)stage_mc, half_bytes, state,
        (unsigned int* const*)pads_dev, rank, world, channel, err, xl_host_comm_spin_limit);
  else
    ar_add_layer_norm_kernel<__half><<<rows, 256, 0, s>>>(
        (__half*)x, (const __half*)delta_partial, (const __half*)bias, (const __half*)w, (const __half*)b, (__half*)h, cols,
        eps, (uint4*)stage_local, (const char*)stage_mc, half_bytes, state, (unsigned int* const*)pads_dev, rank, world,
        channel, err, xl_host_comm_spin_limit);
  return (int)cudaGetLastError();
}
