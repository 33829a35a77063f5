// Device-side helpers for kernels that talk to peer GPUs through symmetric memory over NVLink / NVSwitch:
// signal flags with release / acquire semantics at system scope, bounded spins, and `multimem` (NVLS) accesses.
//
// Symmetric memory: every rank of a group maps the same-sized buffer of every other rank, so a kernel can use
// `peer_base[p] + offset` as an ordinary global address. A signal pad is a small zero-initialised uint32 array in that
// memory. Slot (channel, sender) of a rank's pad is written by exactly one peer and consumed by the owner, so a
// barrier needs no atomics beyond compare-and-swap on single words.
//
// Every wait is bounded: after `limit` polls (a launch argument) the waiter records an error code and returns false; the
// caller then stops communicating and returns normally, leaving the context usable.
#pragma once
#include "common.cuh"

// Poll budget of every wait on a peer. The default tolerates ranks that are tens of seconds apart (first step, host
// hiccups); tests lower it through xl_set_comm_spin_limit to watch a wait give up quickly.
#ifndef XL_COMM_SPIN_DEFAULT
#define XL_COMM_SPIN_DEFAULT (1u << 26)
#endif
extern unsigned int xl_host_comm_spin_limit;  // host-side; handed to every kernel as an argument

enum XlCommError : int { XL_COMM_OK = 0, XL_COMM_TIMEOUT_SIGNAL = 101, XL_COMM_TIMEOUT_WAIT = 102, XL_COMM_TIMEOUT_FLAG = 103 };

__device__ __forceinline__ unsigned int xl_ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned int xl_ld_acquire_gpu(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void xl_st_release_gpu(unsigned int* p, unsigned int v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int xl_cas_release_sys(unsigned int* p, unsigned int cmp, unsigned int val) {
  unsigned int old;
  asm volatile("atom.release.sys.global.cas.b32 %0, [%1], %2, %3;" : "=r"(old) : "l"(p), "r"(cmp), "r"(val) : "memory");
  return old;
}
__device__ __forceinline__ unsigned int xl_cas_acquire_sys(unsigned int* p, unsigned int cmp, unsigned int val) {
  unsigned int old;
  asm volatile("atom.acquire.sys.global.cas.b32 %0, [%1], %2, %3;" : "=r"(old) : "l"(p), "r"(cmp), "r"(val) : "memory");
  return old;
}

// Set a peer's flag 0 -> 1 (waits, bounded, until the previous signal in that slot has been consumed).
__device__ __forceinline__ bool xl_put_signal(unsigned int* slot, int* err, unsigned int limit) {
  for (unsigned int i = 0; i < limit; ++i)
    if (xl_cas_release_sys(slot, 0u, 1u) == 0u) return true;
  if (err) atomicCAS(err, 0, (int)XL_COMM_TIMEOUT_SIGNAL);
  return false;
}
// Consume an own flag 1 -> 0 (waits, bounded, until the peer has set it).
__device__ __forceinline__ bool xl_wait_signal(unsigned int* slot, int* err, unsigned int limit) {
  for (unsigned int i = 0; i < limit; ++i)
    if (xl_cas_acquire_sys(slot, 1u, 0u) == 1u) return true;
  if (err) atomicCAS(err, 0, (int)XL_COMM_TIMEOUT_WAIT);
  return false;
}

// Barrier over `world` ranks, executed by the first `world` threads of one warp (all 32 lanes must call).
// pads[p] is rank p's signal pad; slot layout: pad[channel * world + sender].
__device__ __forceinline__ bool xl_group_barrier(unsigned int* const* pads, int rank, int world, int channel, int* err,
                                                 unsigned int limit) {
  const int lane = threadIdx.x & 31;
  bool ok = true;
  __threadfence_system();
  if (lane < world && lane != rank) {
    ok = xl_put_signal(pads[lane] + channel * world + rank, err, limit);
    if (ok) ok = xl_wait_signal(pads[rank] + channel * world + lane, err, limit);
  }
  ok = __all_sync(0xffffffffu, ok);
  __threadfence_system();
  return ok;
}

// ---- multimem (NVLS): one access reaches the same offset in every replica bound to the multicast address -----------
__device__ __forceinline__ void xl_multimem_red_add_bf16x8(void* mc_addr, uint4 v) {
  asm volatile("multimem.red.relaxed.sys.global.add.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void xl_multimem_red_add_f16x8(void* mc_addr, uint4 v) {
  asm volatile("multimem.red.relaxed.sys.global.add.v4.f16x2 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}
// vector reduction into one (possibly remote) address: used when each row has a single owner (reduce-scatter)
__device__ __forceinline__ void xl_red_add_bf16x8(void* addr, uint4 v) {
  asm volatile("red.relaxed.sys.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(addr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void xl_red_add_f16x8(void* addr, uint4 v) {
  asm volatile("red.relaxed.sys.global.add.noftz.v4.f16x2 [%0], {%1, %2, %3, %4};" ::"l"(addr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void xl_multimem_red_add_f32x4(void* mc_addr, float4 v) {
  asm volatile("multimem.red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "f"(v.x), "f"(v.y),
               "f"(v.z), "f"(v.w)
               : "memory");
}
__device__ __forceinline__ float4 xl_multimem_ld_reduce_add_f32x4(const void* mc_addr) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
__device__ __forceinline__ void xl_multimem_st_b128(void* mc_addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}
