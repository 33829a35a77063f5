// bf16 / fp16 GEMM for sm_100a on CTA pairs: tcgen05.mma.cta_group::2 multiplies a 256 x 256 tile across two SMs of a
// thread-block cluster. Each CTA stages its own 128 rows of A and only its own half (128 columns) of the B tile, so a
// k-block costs 32 KB of shared-memory traffic per SM instead of 48 KB for a 128 x 256 tile on one SM, and the ring
// holds 6 stages instead of 4. Each CTA keeps the accumulator rows of its A half in its own TMEM (two buffers of 256
// columns) and drains them with its own 8 epilogue warps.
//
// Roles per CTA (320 threads):
//   warp 0    : TMA producer of this CTA's A rows and B half. The transaction bytes of both CTAs complete on the
//               "full" barrier of the leader (cluster rank 0), which alone consumes it.
//   warp 1    : allocates / frees TMEM (both CTAs, cta_group::2); in the leader one elected thread issues every MMA
//               and commits to the "empty" and "accumulator full" barriers of both CTAs (one commit each: the peer's
//               barrier is addressed through the cluster window).
//   warps 2-9 : epilogue, identical to the single-CTA kernel; "accumulator drained" arrivals of both CTAs go to the
//               leader's barrier.
// The pair walks the same persistent tile sequence (cluster index, stride = clusters of the launch).
//
// Every wait is bounded. A role that gives up records a code in `*err` and raises the abort flag of both CTAs; all roles
// then leave their loops, meet at the closing cluster barrier (which every thread of both CTAs reaches), TMEM is freed
// and the kernel returns.
//
// Scope: plain GEMMs (any operand major-ness, batch, bias / activation / accumulate epilogue) with N > 128. Collective
// epilogues, the all-gather prologue, causal tile skipping and 8-bit operands stay on the single-CTA kernel.
#include "tcgen05.cuh"
#include "gemm_epilogue.cuh"

#include <cuda.h>

namespace {

using namespace xl_tc;

constexpr int CTA_M = 128;              // rows of C per CTA
constexpr int PAIR_M = 2 * CTA_M;       // rows of C per tile
constexpr int BLOCK_K = 64;             // 64 x 2 bytes = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_EPI_WARPS = 8;
constexpr int NUM_THREADS = 64 + 32 * NUM_EPI_WARPS;
constexpr int A_BYTES = CTA_M * BLOCK_K * 2;

// Tile width PN (columns of C per tile, 256 or 128): each CTA stages PN / 2 rows of the B tile. The narrow tile is for
// shapes whose 256 x 256 tiles would fill the last wave of CTA pairs badly.
template <int PN>
struct PairCfg {
  static constexpr int PAIR_N = PN;
  static constexpr int HALF_N = PN / 2;
  static constexpr int B_BYTES = HALF_N * BLOCK_K * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = PN == 256 ? 6 : 8;
  static constexpr int TILE_BYTES = STAGES * STAGE_BYTES;
  static constexpr int STAGING_BYTES = NUM_EPI_WARPS * 32 * 32 * 4;  // one 32 x 32 fp32 chunk per epilogue warp
  static constexpr int SMEM_TOTAL = TILE_BYTES + STAGING_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
  static constexpr uint32_t TMEM_COLS = 2 * PN;  // two accumulator buffers
};

enum { ERR2_FULL_WAIT = 21, ERR2_EMPTY_WAIT = 22, ERR2_TMEM_FULL_WAIT = 23, ERR2_TMEM_EMPTY_WAIT = 24 };

struct Gemm2Params {
  int M, N, K, batch;
  int a_mn, b_mn;  // 0: K-major operand, 1: MN-major operand
  void* C;
  long long ldc, batch_stride_c;
  EpilogueParams epi;
  const float* step;  // running-mean step counter (accumulate == 2)
  float alpha;
  int is_fp16;
  int* err;
};

// ---- cluster helpers ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_id_x() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t num_clusters_x() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r));
  return r;
}
// address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void st_cluster_u32(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}

// ---- cta_group::2 forms of the tcgen05 / TMA instructions ------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
// arrives on the barrier at `cluster_addr` (own or peer CTA) once all MMAs issued so far by this thread have completed
__device__ __forceinline__ void tcgen05_commit_pair(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tcgen05_mma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                     uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Tiled load into this CTA's shared memory whose transaction bytes complete on a barrier that may live in the peer CTA
// (`bar_cluster_addr`). Each CTA loads its own tile: one source, one destination.
__device__ __forceinline__ void tma_load_3d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int c0,
                                                 int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

// Bounded wait on a barrier of this CTA; on a timeout the abort flag of both CTAs is raised.
__device__ __forceinline__ bool mbar_wait_pair(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                               uint32_t peer_abort_addr, int* err, int code) {
  for (uint32_t i = 0; i < MBAR_SPIN_LIMIT; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = 1;
  st_cluster_u32(peer_abort_addr, 1u);
  if (err) atomicCAS(err, 0, code);
  return false;
}

// tile index -> (batch, m block, n block); m-blocks are walked in groups of 8 inside each n-column so that the tiles in
// flight share operand panels in L2
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& b, int& mb, int& nb) {
  constexpr int GROUP = 8;
  const int per_batch = tiles_m * tiles_n;
  b = tile / per_batch;
  const int t = tile - b * per_batch;
  const int group_size = GROUP * tiles_n;
  const int g = t / group_size;
  const int first_m = g * GROUP;
  const int rows = min(GROUP, tiles_m - first_m);
  const int in_group = t - g * group_size;
  mb = first_m + in_group % rows;
  nb = in_group / rows;
}

template <int PN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
    gemm2cta_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                            const Gemm2Params p) {
  using Cfg = PairCfg<PN>;
  constexpr int PAIR_N = Cfg::PAIR_N, HALF_N = Cfg::HALF_N, STAGE_BYTES = Cfg::STAGE_BYTES, STAGES = Cfg::STAGES,
                TILE_BYTES = Cfg::TILE_BYTES;
  constexpr uint32_t TMEM_COLS = Cfg::TMEM_COLS;
  extern __shared__ uint8_t smem_raw[];
  // the dynamic shared-memory window starts at the same offset in both CTAs, so the aligned base does too: the MMA
  // applies one descriptor (one offset) to the shared memory of both
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* staging = smem + TILE_BYTES;               // fp32 C: chunks are transposed here so that rows are stored whole
  uint64_t* bars = (uint64_t*)(smem + TILE_BYTES + Cfg::STAGING_BYTES);
  uint64_t* full_bar = bars;                          // [STAGES]  used in the leader only
  uint64_t* empty_bar = bars + STAGES;                // [STAGES]  one per CTA, both signalled by the leader's commits
  uint64_t* tmem_full_bar = bars + 2 * STAGES;        // [2]       one per CTA, both signalled by the leader's commits
  uint64_t* tmem_empty_bar = bars + 2 * STAGES + 2;   // [2]       used in the leader only: 2 x NUM_EPI_WARPS arrivals
  uint32_t* tmem_base_slot = (uint32_t*)(bars + 2 * STAGES + 4);
  volatile int* abort_flag = (volatile int*)(tmem_base_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0: leader (issues the MMAs), 1: peer
  const uint32_t peer = rank ^ 1u;
  const bool leader = rank == 0;
  const int pair = (int)cluster_id_x(), npairs = (int)num_clusters_x();
  const int tiles_m = (p.M + PAIR_M - 1) / PAIR_M;
  const int tiles_n = (p.N + PAIR_N - 1) / PAIR_N;
  const int num_tiles = tiles_m * tiles_n * p.batch;
  const int k_blocks = (p.K + BLOCK_K - 1) / BLOCK_K;
  const uint32_t peer_abort_addr = map_to_cta(smem_u32((const void*)abort_flag), peer);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full_bar[a], 1);
      mbar_init(&tmem_empty_bar[a], 2 * NUM_EPI_WARPS);  // one arrival per epilogue warp of both CTAs
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  cluster_sync_all();  // both CTAs run and their barriers are initialised before anything involves the pair
  if (warp == 1) {
    tmem_alloc_pair(tmem_base_slot, TMEM_COLS);  // one warp of each CTA: the allocation is collective over the pair
    tmem_relinquish_pair();
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0) {
    // ------------------------------------------------ TMA producer ------------------------------------------------
    if (elect_one()) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += npairs) {
        int b, mb, nb;
        tile_coords(tile, tiles_m, tiles_n, b, mb, nb);
        const int m0 = mb * PAIR_M + (int)rank * CTA_M;   // this CTA's rows of A and C
        const int n0 = nb * PAIR_N + (int)rank * HALF_N;  // this CTA's half of the B tile
        for (int kb = 0; kb < k_blocks; ++kb) {
          ok = mbar_wait_pair(&empty_bar[stage], phase ^ 1, abort_flag, peer_abort_addr, p.err, ERR2_EMPTY_WAIT);
          if (!ok) break;
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * STAGE_BYTES);  // the bytes of both CTAs
          const uint32_t full_addr = map_to_cta(smem_u32(&full_bar[stage]), 0);
          const int k0 = kb * BLOCK_K;
          if (!p.a_mn) {
            tma_load_3d_pair(sa, &map_a, full_addr, k0, m0, b);  // box {64 k, 128 m}
          } else {
#pragma unroll
            for (int j = 0; j < CTA_M / 64; ++j)                  // boxes {64 m, 64 k}
              tma_load_3d_pair(sa + j * (BLOCK_K * 128), &map_a, full_addr, m0 + j * 64, k0, b);
          }
          if (!p.b_mn) {
            tma_load_3d_pair(sb, &map_b, full_addr, k0, n0, b);  // box {64 k, 128 n}
          } else {
#pragma unroll
            for (int j = 0; j < HALF_N / 64; ++j)                 // boxes {64 n, 64 k}
              tma_load_3d_pair(sb + j * (BLOCK_K * 128), &map_b, full_addr, n0 + j * 64, k0, b);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer (leader CTA only) -------------------------------
    if (leader && elect_one()) {
      const uint32_t fmt = p.is_fp16 ? 0u : 1u;
      const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(p.a_mn != 0) << 15) |
                             ((uint32_t)(p.b_mn != 0) << 16) | ((uint32_t)(PAIR_N >> 3) << 17) |
                             ((uint32_t)(PAIR_M >> 4) << 24);
      const uint32_t a_lbo = p.a_mn ? BLOCK_K * 128 : 16;
      const uint32_t b_lbo = p.b_mn ? BLOCK_K * 128 : 16;
      const uint32_t a_kstep = p.a_mn ? UMMA_K * 128 : UMMA_K * 2;  // bytes to advance per UMMA_K
      const uint32_t b_kstep = p.b_mn ? UMMA_K * 128 : UMMA_K * 2;
      uint32_t stage = 0, phase = 0;
      uint32_t acc = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += npairs) {
        ok = mbar_wait_pair(&tmem_empty_bar[acc], acc_phase ^ 1, abort_flag, peer_abort_addr, p.err, ERR2_TMEM_EMPTY_WAIT);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t tmem_d = tmem_base + acc * PAIR_N;
        for (int kb = 0; kb < k_blocks; ++kb) {
          ok = mbar_wait_pair(&full_bar[stage], phase, abort_flag, peer_abort_addr, p.err, ERR2_FULL_WAIT);
          if (!ok) break;
          tcgen05_fence_after();
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
            const uint64_t da = make_smem_desc(sa + k * a_kstep, a_lbo);
            const uint64_t db = make_smem_desc(sb + k * b_kstep, b_lbo);
            tcgen05_mma_f16_pair(tmem_d, da, db, idesc, (kb != 0 || k != 0) ? 1u : 0u);
          }
          // frees the stage in both CTAs once these MMAs have read it
          tcgen05_commit_pair(smem_u32(&empty_bar[stage]));
          tcgen05_commit_pair(map_to_cta(smem_u32(&empty_bar[stage]), peer));
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tcgen05_commit_pair(smem_u32(&tmem_full_bar[acc]));  // accumulator complete, in both CTAs
        tcgen05_commit_pair(map_to_cta(smem_u32(&tmem_full_bar[acc]), peer));
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------ epilogue ----------------------------------------------------
    const int q = warp & 3;                // TMEM lane quarter this warp may access
    const int col_half = (warp - 2) >> 2;  // which half of the accumulator columns this warp drains
    constexpr int COLS_PER_WARP = PAIR_N / (NUM_EPI_WARPS / 4);
    uint32_t acc = 0, acc_phase = 0;
    bool ok = true;
    float mean_a = 0.f, mean_b = 1.f;
    if (p.epi.accumulate == 2) {
      const float t = *p.step;
      mean_a = t / (t + 1.f);
      mean_b = 1.f / (t + 1.f);
    }
    const int esz = p.epi.c_dtype == XL_F32 ? 4 : 2;
    for (int tile = pair; tile < num_tiles && ok; tile += npairs) {
      int b, mb, nb;
      tile_coords(tile, tiles_m, tiles_n, b, mb, nb);
      const int row = mb * PAIR_M + (int)rank * CTA_M + q * 32 + lane;
      const bool row_ok = row < p.M;
      uint8_t* crow = (uint8_t*)p.C + ((long long)b * p.batch_stride_c + (long long)row * p.ldc) * esz;
      ok = mbar_wait_pair(&tmem_full_bar[acc], acc_phase, abort_flag, peer_abort_addr, p.err, ERR2_TMEM_FULL_WAIT);
      if (!ok) break;
      tcgen05_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + acc * PAIR_N;
      // fp32 C whose rows are 16-byte aligned: a thread holds 32 columns of ONE row, so storing from the registers would
      // touch 32 lines per instruction (and so would reading the old contents when accumulating). The chunk goes through
      // shared memory instead and leaves as whole 128-byte row pieces, four rows per instruction.
      const bool staged = p.epi.c_dtype == XL_F32 && (p.ldc % 4) == 0 && ((((uintptr_t)p.C) | ((uintptr_t)(p.batch_stride_c * 4))) & 15) == 0;
      const bool staged16 = p.epi.c_dtype != XL_F32 && !p.epi.accumulate && (p.ldc % 8) == 0 &&
                            ((((uintptr_t)p.C) | ((uintptr_t)(p.batch_stride_c * 2))) & 15) == 0;
      float4* stage = (float4*)(staging + (warp - 2) * (32 * 32 * 4));
      const int row_base = mb * PAIR_M + (int)rank * CTA_M + q * 32;
#pragma unroll 1
      for (int c = col_half * COLS_PER_WARP; c < (col_half + 1) * COLS_PER_WARP; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c, r);
        tmem_ld_wait();
        const int col0 = nb * PAIR_N + c;
        if (col0 >= p.N) continue;  // uniform over the warp
        if (staged16 && col0 + 32 <= p.N) {
          // 16-bit C, no accumulation: the thread's 32 columns (64 bytes) go to shared memory, 16-byte pieces rotated by
          // the row pair so that neither phase has bank conflicts; then 4 lanes store one row's 64 bytes, 8 rows per
          // instruction
          uint4* stage16 = (uint4*)stage;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              float x = __uint_as_float(r[j * 8 + e]) * p.alpha;
              if (p.epi.bias) {
                const int col = col0 + j * 8 + e;
                x += p.epi.bias_dtype == XL_F32 ? ((const float*)p.epi.bias)[col]
                     : p.epi.bias_dtype == XL_BF16 ? __bfloat162float(((const __nv_bfloat16*)p.epi.bias)[col])
                                                   : __half2float(((const __half*)p.epi.bias)[col]);
              }
              v[e] = apply_act(x, p.epi.act);
            }
            stage16[lane * 4 + ((j + (lane >> 1)) & 3)] = pack8_16bit(v, p.epi.c_dtype == XL_F16);
          }
          __syncwarp();
          uint16_t* cbase16 = (uint16_t*)p.C + (long long)b * p.batch_stride_c + col0 + (lane & 3) * 8;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int lr = i * 8 + (lane >> 2), rr = row_base + lr;
            const uint4 o = stage16[lr * 4 + (((lane & 3) + (lr >> 1)) & 3)];
            if (rr < p.M) *(uint4*)(cbase16 + (long long)rr * p.ldc) = o;
          }
          __syncwarp();
          continue;
        }
        if (!(staged && col0 + 32 <= p.N)) {
          if (row_ok) epilogue_store_32cols(p.epi, r, crow, col0, p.alpha, mean_a, mean_b);
          continue;
        }
        // old contents first (their latency overlaps the staging): lane -> row (lane / 8) of each group of four, 16 bytes
        const int sub_row = lane >> 3, sub_col = (lane & 7) * 4;
        float* cbase = (float*)p.C + (long long)b * p.batch_stride_c + col0 + sub_col;
        float4 old[8];
        if (p.epi.accumulate) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int rr = row_base + i * 4 + sub_row;
            old[i] = rr < p.M ? *(const float4*)(cbase + (long long)rr * p.ldc) : make_float4(0.f, 0.f, 0.f, 0.f);
          }
        }
        // this thread's row -> shared memory, 16-byte pieces swizzled by the row so that both phases are conflict-free
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float v[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float x = __uint_as_float(r[j * 4 + e]) * p.alpha;
            if (p.epi.bias) {
              const int col = col0 + j * 4 + e;
              x += p.epi.bias_dtype == XL_F32 ? ((const float*)p.epi.bias)[col]
                   : p.epi.bias_dtype == XL_BF16 ? __bfloat162float(((const __nv_bfloat16*)p.epi.bias)[col])
                                                 : __half2float(((const __half*)p.epi.bias)[col]);
            }
            v[e] = apply_act(x, p.epi.act);
          }
          stage[lane * 8 + (j ^ (lane & 7))] = make_float4(v[0], v[1], v[2], v[3]);
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int lr = i * 4 + sub_row, rr = row_base + lr;
          float4 o = stage[lr * 8 + ((lane & 7) ^ (lr & 7))];
          if (p.epi.accumulate == 1) { o.x += old[i].x; o.y += old[i].y; o.z += old[i].z; o.w += old[i].w; }
          else if (p.epi.accumulate == 2) {
            o.x = old[i].x * mean_a + o.x * mean_b; o.y = old[i].y * mean_a + o.y * mean_b;
            o.z = old[i].z * mean_a + o.z * mean_b; o.w = old[i].w * mean_a + o.w * mean_b;
          }
          if (rr < p.M) *(float4*)(cbase + (long long)rr * p.ldc) = o;
        }
        __syncwarp();  // the buffer is rewritten by the next chunk
      }
      // all TMEM reads of this warp are complete (wait::ld above): hand the accumulator back to the leader's MMA thread
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (leader) mbar_arrive(&tmem_empty_bar[acc]);
        else mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty_bar[acc]), 0));
      }
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  // ---- teardown: every role of both CTAs arrives here, also after an abort. Neither CTA may leave earlier: the peer's
  // loads complete on the leader's barriers and the leader's MMAs read the peer's shared memory and write its TMEM.
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

// 3-D map over a row-major matrix with `rows` rows of `cols` contiguous elements (leading dimension `ld`), `batch`
// matrices `batch_stride` elements apart; boxes of {box_cols, box_rows, 1} with 128-byte swizzle.
int make_map(CUtensorMap* map, const void* ptr, int is_fp16, long long rows, long long cols, long long ld, long long batch,
             long long batch_stride, int box_cols, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -2;
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)(batch > 1 ? batch_stride : rows * ld) * 2};
  cuuint32_t box[3] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapDataType dt = is_fp16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUresult r = fn(map, dt, 3, (void*)ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

// number of CTA pairs that can be resident at once on this device (0 if the query fails); looked up once
template <int PN>
int max_resident_pairs() {
  constexpr int SMEM_TOTAL = PairCfg<PN>::SMEM_TOTAL;
  static int cached = -1;
  if (cached >= 0) return cached;
  if (cudaFuncSetAttribute(gemm2cta_tcgen05_kernel<PN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL) != cudaSuccess) {
    cached = 0;
    return 0;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2, 1, 1);
  cfg.blockDim = dim3(NUM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = SMEM_TOTAL;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, gemm2cta_tcgen05_kernel<PN>, &cfg) != cudaSuccess) {
    cudaGetLastError();
    n = 0;
  }
  cached = n;
  return n;
}

template <int PN>
int launch_pairs(const CUtensorMap& ma, const CUtensorMap& mb, const Gemm2Params& p, int max_pairs, cudaStream_t s) {
  int pairs = max_resident_pairs<PN>();
  if (pairs <= 0) return -4;
  if (max_pairs > 0 && max_pairs < pairs) pairs = max_pairs;
  const long long tiles = (long long)((p.M + PAIR_M - 1) / PAIR_M) * ((p.N + PN - 1) / PN) * p.batch;
  if (tiles < pairs) pairs = (int)tiles;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(NUM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = PairCfg<PN>::SMEM_TOTAL;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm2cta_tcgen05_kernel<PN>, ma, mb, p);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

// Tile width for a shape: the one whose tiles take less time in waves over `pairs` CTA pairs (a 256 x 128 tile takes
// about two thirds of the time of a 256 x 256 one: its MMAs are less efficient and it re-reads A twice as often).
int choose_pair_n(int M, int N, int batch, int pairs) {
  if (N <= 128 || pairs <= 0) return N <= 128 ? 128 : 256;
  const long long tm = (M + PAIR_M - 1) / PAIR_M;
  const long long t256 = tm * ((N + 255) / 256) * batch, t128 = tm * ((N + 127) / 128) * batch;
  const double cost256 = (double)((t256 + pairs - 1) / pairs) * 1.0;
  const double cost128 = (double)((t128 + pairs - 1) / pairs) * 0.66;
  return cost128 < cost256 ? 128 : 256;
}

}  // namespace

// C = epilogue(A * B) on CTA pairs; same operand conventions as xl_gemm_tcgen05 (16-bit operands, fp32 accumulation).
//   accumulate: 0 overwrite, 1 C += alpha*acc, 2 running mean with the step counter `step`.
//   max_pairs: upper limit of CTA pairs to launch (<= 0: as many as can be resident).
//   tile_n: columns of C per tile, 256 or 128 (0: whichever takes fewer waves of CTA pairs for this shape).
// Returns 0, a CUDA error code, -1 for arguments this kernel does not take (the caller then uses the single-CTA
// kernel), -4 if no CTA pair can be resident on this device.
XL_API int xl_gemm2cta_tcgen05(const void* a, const void* b, void* c, int M, int N, int K, int batch, int a_mn, int b_mn,
                               long long lda, long long ldb, long long ldc, long long stride_a, long long stride_b,
                               long long stride_c, int ab_is_fp16, int c_dtype, const void* bias, int bias_dtype, int act,
                               int accumulate, const float* step, float alpha, int* err, int max_pairs, int tile_n,
                               cudaStream_t s) {
  if (M <= 0 || N <= 64 || K <= 0 || batch <= 0) return -1;
  if ((((uintptr_t)a) & 15) || (((uintptr_t)b) & 15) || (lda % 8) || (ldb % 8)) return -1;
  if (batch > 1 && ((stride_a % 8) || (stride_b % 8))) return -1;
  if (accumulate < 0 || accumulate > 2 || (accumulate == 2 && step == nullptr)) return -1;
  if (tile_n != 0 && tile_n != 128 && tile_n != 256) return -1;
  const int pair_n = tile_n ? tile_n : choose_pair_n(M, N, batch, max_pairs > 0 ? max_pairs : max_resident_pairs<256>());
  CUtensorMap ma, mb;
  int r;
  if (!a_mn) r = make_map(&ma, a, ab_is_fp16, M, K, lda, batch, stride_a, BLOCK_K, CTA_M);
  else r = make_map(&ma, a, ab_is_fp16, K, M, lda, batch, stride_a, 64, BLOCK_K);
  if (r) return r;
  if (!b_mn) r = make_map(&mb, b, ab_is_fp16, N, K, ldb, batch, stride_b, BLOCK_K, pair_n / 2);
  else r = make_map(&mb, b, ab_is_fp16, K, N, ldb, batch, stride_b, 64, BLOCK_K);
  if (r) return r;
  Gemm2Params p;
  p.M = M; p.N = N; p.K = K; p.batch = batch;
  p.a_mn = a_mn; p.b_mn = b_mn;
  p.C = c; p.ldc = ldc; p.batch_stride_c = stride_c;
  p.epi.N = N; p.epi.c_dtype = c_dtype; p.epi.bias = bias; p.epi.bias_dtype = bias_dtype; p.epi.act = act;
  p.epi.accumulate = accumulate;
  p.step = step; p.alpha = alpha; p.is_fp16 = ab_is_fp16; p.err = err;
  if (pair_n == 128) return launch_pairs<128>(ma, mb, p, max_pairs, s);
  return launch_pairs<256>(ma, mb, p, max_pairs, s);
}
