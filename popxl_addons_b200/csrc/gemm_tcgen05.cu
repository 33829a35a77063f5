// bf16 / fp16 GEMM on the 5th-generation tensor cores (tcgen05) for sm_100a.
//
//   C[b] (M x N) = epilogue( A[b] (M x K) * B[b] (K x N) )
//
// Structure: persistent kernel, one CTA per SM, 320 threads:
//   warp 0      TMA producer   : cp.async.bulk.tensor loads of A / B tiles into a 4-stage shared-memory ring
//   warp 1      MMA issuer     : one elected thread issues tcgen05.mma (128 x BLOCK_N x 16), accumulators live in TMEM,
//                                two accumulator buffers so the epilogue of tile i overlaps the main loop of tile i+1
//   warps 2..9  epilogue       : tcgen05.ld TMEM -> registers, bias / activation / accumulate, 16-byte global stores
// Either operand may be K-major (reduction dimension contiguous) or MN-major, so `x @ w`, `g @ w^T` and `x^T @ g`
// (forward, data gradient, weight gradient) all run without materialising a transpose. Shared-memory tiles use the
// 128-byte swizzle that both TMA and the UMMA shared-memory descriptors understand.
//
// Every wait on an mbarrier is bounded: when a wait gives up the kernel records a code in `*err`, raises a CTA-wide
// abort flag, all roles leave their loops, TMEM is released and the kernel returns normally.
#include "comm.cuh"
#include "tcgen05.cuh"

#include <cuda.h>
#include <cstdlib>
#include <stdio.h>

namespace {

constexpr int BLOCK_M = 128;
constexpr int BLOCK_K = 64;  // 64 x 2 bytes = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int NUM_EPI_WARPS = 8;  // two warps per TMEM lane quarter, each draining half of the accumulator columns
constexpr int NUM_THREADS = 64 + 32 * NUM_EPI_WARPS;
constexpr uint32_t SPIN_LIMIT = 1u << 22;
constexpr int EPI_STAGE_BYTES = 4096;  // per epilogue warp, only in the modes that push tiles to peers

enum { ERR_FULL_WAIT = 1, ERR_EMPTY_WAIT = 2, ERR_TMEM_FULL_WAIT = 3, ERR_TMEM_EMPTY_WAIT = 4 };
constexpr int AR_ITEMS_PER_TILE = 8;     // a reduce work item = BLOCK_M / 8 = 16 rows of one tile
constexpr int AR_SYNC_QUEUE = 8, AR_SYNC_DONE = 9;  // words of local_sync used by the pull all-reduce
constexpr int AR_CHANNEL = 2;            // signal channel of its closing barrier

struct GemmParams {
  int M, N, K, batch;
  int a_mn, b_mn;  // 0: K-major operand, 1: MN-major operand
  void* C;
  long long ldc, batch_stride_c;
  int c_dtype;
  const void* bias;  // length N, may be null
  int bias_dtype;
  int act;         // 0 none, 1 gelu(erf), 2 gelu(tanh), 3 relu
  int accumulate;  // 0 overwrite, 1 C += alpha*acc, 2 running mean: C = C*t/(t+1) + acc/(t+1), t = *step,
                   // 3 all-reduce: C is a multicast (NVLS) address, every tile is pushed with multimem.red.add into
                   //   the output buffer of every rank of the group (buffers zeroed before the launch)
  const float* step;
  float alpha;
  int is_fp16;
  int* err;
  // all-reduce mode only
  unsigned int* const* pads;  // signal pad of every rank
  int comm_rank, comm_world;
  unsigned int* local_sync;   // [0] "peers are ready" flag (set by CTA 0, cleared by the last warp to finish),
                              // [1] count of epilogue warps that finished
  unsigned int comm_spin_limit;
  // reduce-scatter mode (accumulate == 4): row r belongs to rank r / rs_rows and is added into that rank's shard buffer
  void* const* rs_dst;  // device array [world]: output shard (rs_rows x ldc) of every rank, as mapped by this rank
  int rs_rows;
  // all-gather prologue: one operand is a row-sharded matrix whose remote row blocks are pulled from the peers by the
  // first `n_copy` CTAs of this launch while the other CTAs already multiply the local rows.
  int gather_mode;                  // 0 none, 1: A (M x K, K-major) sharded over M, 2: B (K x N, N contiguous) sharded over K
  int n_copy;                       // copy CTAs
  int gather_bps;                   // row blocks per shard (a row block = BLOCK_M rows of A or BLOCK_K rows of B)
  long long gather_block_bytes;     // bytes of one row block (rows are contiguous: leading dimension == row length)
  const uint8_t* const* gather_src; // device array [world]: the full matrix in every rank's memory
  uint8_t* gather_dst;              // the full matrix in this rank's memory (own shard already in place)
  unsigned int* gather_flags;       // one word per row block of the full matrix, zeroed before the launch; 1 = landed
  // causal structure of square attention products (rows and columns / contraction index are token positions):
  //   1: output tiles entirely above the diagonal are not computed (S = Q K^T, dP = dO V^T; the softmax kernels never
  //      read them and overwrite them with zeros)
  //   2: the left operand is zero right of the diagonal (O = P V, dQ = dS K): contraction stops at the tile's last row
  //   3: the (transposed) left operand is zero before the diagonal (dV = P^T dO, dK = dS^T Q): contraction starts at
  //      the tile's first row
  int causal;
  // 8-bit float operands (tcgen05 kind::f8f6f4; both operands K-major): -1 = 16-bit operands, else the format of A / B
  // (0 = e4m3, 1 = e5m2). A k-block is then 128 elements, still one 128-byte swizzle row.
  int fp8_a, fp8_b;
  const float* alpha_log2;  // optional device scalar: the result is also multiplied by 2^(*alpha_log2)
  // second operand pair (map_a2, map_b2; same layouts as the first) contracted into the same accumulator:
  // C = A * B + A2 * B2. 0: none.
  int K2;
  // all-reduce by pulling (accumulate == 5). Every rank writes its partial product into its own buffer C (symmetric
  // memory) with plain stores and, tile by tile, tells the rank that owns the tile's rows (rows are split evenly over
  // the ranks) that its part is there. The owner adds the `world` copies of a tile inside NVSwitch with one
  // multimem.ld_reduce per 16 bytes of the partial buffers' multicast address and writes the sums into every rank's
  // result buffer with multimem.st. Reducing is done by the first `n_copy` CTAs of the launch from the start and by the
  // epilogue warps of the other CTAs once they have run out of tiles; work items (an eighth of a tile) are handed out
  // by a counter.
  const uint8_t* ar_src_mc;         // multicast address of the partial buffers (C on every rank)
  uint8_t* ar_dst_mc;               // multicast address of the result buffers; with accumulate == 6 (reduce-scatter:
                                    //   every rank keeps only the sums of its own rows) this rank's (ar_rows x ldc) shard
  unsigned int* const* ar_flags;    // device array [world]: per rank, 2 * tiles words: [tile] parts arrived (written
                                    //   by all ranks), [tiles + tile] eighths reduced (owner only). All zero between launches.
  int ar_rows;                      // rows owned by each rank (a multiple of BLOCK_M)
  unsigned long long* dbg;          // optional: 4 timestamps (ns) per CTA (start, tiles done, reduce done, finish done),
                                    // then 3 per reduce item (taken, tile ready, reduced; 4 words apart)
};

// k-block range of a tile under the causal modes; false: the tile is skipped altogether
__device__ __forceinline__ bool tile_k_range(const GemmParams& p, int mb, int nb, int k_blocks, int block_n, int& kb0,
                                             int& kb1) {
  kb0 = 0;
  kb1 = k_blocks;
  if (p.causal == 1) return nb * block_n <= mb * BLOCK_M + BLOCK_M - 1;
  if (p.causal == 2) kb1 = min(k_blocks, (mb * BLOCK_M + BLOCK_M + BLOCK_K - 1) / BLOCK_K);
  if (p.causal == 3) kb0 = min(k_blocks - 1, (mb * BLOCK_M) / BLOCK_K);
  return true;
}

using namespace xl_tc;

// plain (untiled) bulk copies, used by the copy CTAs of the all-gather prologue; never multicast
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               ::"l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N> __device__ __forceinline__ void bulk_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }

__device__ __forceinline__ float apply_act(float v, int act) {
  if (act == 1) return 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
  if (act == 2) return 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
  if (act == 3) return fmaxf(v, 0.f);
  return v;
}

template <int BLOCK_N>
struct SmemLayout {
  static constexpr int A_BYTES = BLOCK_M * BLOCK_K * 2;
  static constexpr int B_BYTES = BLOCK_N * BLOCK_K * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int TILE_BYTES = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = TILE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

// tile index -> (batch, m block, n block). Tiles that run at the same time share A / B panels in L2: m-blocks are
// walked in groups of 8 inside each n-column.
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& b, int& mb, int& nb, int GROUP = 8) {
  const int per_batch = tiles_m * tiles_n;
  b = tile / per_batch;
  int t = tile - b * per_batch;
  const int group_size = GROUP * tiles_n;
  const int g = t / group_size;
  const int first_m = g * GROUP;
  const int rows = min(GROUP, tiles_m - first_m);
  const int in_group = t - g * group_size;
  mb = first_m + in_group % rows;
  nb = in_group / rows;
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ unsigned int ld_acquire_sys_u32(const unsigned int* ptr) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add_u32(unsigned int* ptr, unsigned int v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(ptr), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 multimem_ld_reduce_16bit(const void* mc_addr, bool bf16) {
  uint4 v;
  if (bf16)
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc_addr) : "memory");
  else
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc_addr) : "memory");
  return v;
}

// Reduce work loop of the pull all-reduce, run by whole warps. Returns when no work item is left (or after a wait ran
// out). Tiles of this rank's rows are taken in the order in which the GEMM CTAs of every rank finish them (columns
// outermost), an eighth of a tile per item.
template <int BLOCK_N>
__device__ __forceinline__ void ar_pull_reduce(const GemmParams& p, int tiles_m, int tiles_n, volatile int* abort_flag) {
  const int lane = threadIdx.x & 31;
  const int mpr = p.ar_rows / BLOCK_M;  // row blocks per rank
  const unsigned int items = (unsigned int)(mpr * tiles_n * AR_ITEMS_PER_TILE);
  const int total_tiles = tiles_m * tiles_n;
  unsigned int* flags = p.ar_flags[p.comm_rank];
  const unsigned int expect = (unsigned int)(NUM_EPI_WARPS * p.comm_world);
  const bool bf = p.c_dtype == XL_BF16;
  constexpr int CHUNKS_PER_ROW = BLOCK_N / 8;                              // 16-byte chunks
  constexpr int ROWS = BLOCK_M / AR_ITEMS_PER_TILE;                        // 16
  constexpr int ITERS = ROWS * CHUNKS_PER_ROW / 32;                        // 16 (BLOCK_N 256) or 8 (128)
  for (;;) {
    if (*abort_flag) break;  // a wait of this CTA ran out: the remaining items would each wait as long
    unsigned int item = 0;
    if (lane == 0) item = atomicAdd(p.local_sync + AR_SYNC_QUEUE, 1u);
    item = __shfl_sync(0xffffffffu, item, 0);
    if (item >= items) break;
    unsigned long long* item_dbg = (p.dbg && lane == 0) ? p.dbg + (size_t)gridDim.x * 4 + (size_t)item * 4 : nullptr;
    if (item_dbg) item_dbg[0] = global_timer_ns();
    const int q = (int)(item / AR_ITEMS_PER_TILE), sub = (int)(item % AR_ITEMS_PER_TILE);
    const int nb = q / mpr, mb = p.comm_rank * mpr + q % mpr;
    const int tile_id = mb * tiles_n + nb;
    int ready = 0;
    if (lane == 0) {
      for (unsigned int i = 0; i < p.comm_spin_limit && !ready; ++i) {
        ready = ld_acquire_sys_u32(flags + tile_id) >= expect;
        if (!ready && (i & 1023u) == 1023u && *abort_flag) break;
      }
    }
    ready = __shfl_sync(0xffffffffu, ready, 0);
    if (!ready) {
      if (lane == 0) {
        *abort_flag = 1;
        if (p.err) atomicCAS(p.err, 0, (int)XL_COMM_TIMEOUT_FLAG);
      }
      break;
    }
    if (item_dbg) item_dbg[1] = global_timer_ns();
    __syncwarp();
    // Every lane reads the flag itself with acquire semantics: its loads below then come after the producers' releases.
    // (A system-scope fence here would also wait for this warp's multicast stores of the previous item to be
    // acknowledged by every rank, several microseconds per item.)
    (void)ld_acquire_sys_u32(flags + tile_id);
    const int row0 = mb * BLOCK_M + sub * ROWS, col0 = nb * BLOCK_N;
    uint4 v[ITERS];
    long long off[ITERS];
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      const int c = it * 32 + lane;
      const int row = row0 + c / CHUNKS_PER_ROW, col = col0 + (c % CHUNKS_PER_ROW) * 8;
      off[it] = (row < p.M && col < p.N) ? ((long long)row * p.ldc + col) * 2 : -1;
      if (off[it] >= 0) v[it] = multimem_ld_reduce_16bit(p.ar_src_mc + off[it], bf);
    }
    if (p.accumulate == 6) {  // reduce-scatter: plain stores into this rank's shard (rows are relative to its first row)
      const long long shard0 = (long long)p.comm_rank * p.ar_rows * p.ldc * 2;
#pragma unroll
      for (int it = 0; it < ITERS; ++it)
        if (off[it] >= 0) *reinterpret_cast<uint4*>(p.ar_dst_mc + (off[it] - shard0)) = v[it];
    } else {
#pragma unroll
      for (int it = 0; it < ITERS; ++it)
        if (off[it] >= 0) xl_multimem_st_b128(p.ar_dst_mc + off[it], v[it]);
    }
    if (item_dbg) item_dbg[2] = global_timer_ns();
    __syncwarp();
    if (lane == 0) {
      const unsigned int prev = atomicAdd(flags + total_tiles + tile_id, 1u);
      if (prev == AR_ITEMS_PER_TILE - 1) {  // the tile is complete: both of its words go back to zero for the next launch
        flags[total_tiles + tile_id] = 0;
        *((volatile unsigned int*)(flags + tile_id)) = 0;
      }
    }
  }
}

// End of the pull all-reduce on this rank: every warp that took part fences its multicast stores and checks in; the last
// one re-arms the two control words and runs the closing barrier (no rank may reuse the partial buffers, or read its
// result buffer, before every rank has finished reducing).
__device__ __forceinline__ void ar_pull_finish(const GemmParams& p, unsigned int participants) {
  const int lane = threadIdx.x & 31;
  __threadfence_system();
  unsigned int prev = 0;
  if (lane == 0) prev = atomicAdd(p.local_sync + AR_SYNC_DONE, 1u);
  prev = __shfl_sync(0xffffffffu, prev, 0);
  if (prev == participants - 1) {
    if (lane == 0) {
      p.local_sync[AR_SYNC_DONE] = 0;
      p.local_sync[AR_SYNC_QUEUE] = 0;
      __threadfence();
    }
    xl_group_barrier(p.pads, p.comm_rank, p.comm_world, AR_CHANNEL, p.err, p.comm_spin_limit);
  }
}

template <int BLOCK_N>
__global__ void __launch_bounds__(NUM_THREADS, 1)
    gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                        const __grid_constant__ CUtensorMap map_a2, const __grid_constant__ CUtensorMap map_b2,
                        const GemmParams p) {
  using L = SmemLayout<BLOCK_N>;
  constexpr uint32_t TMEM_COLS = 2 * BLOCK_N;  // two accumulator buffers (power of two: 256 or 512)
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(smem + L::TILE_BYTES);
  uint64_t* full_bar = bars;                     // [STAGES]
  uint64_t* empty_bar = bars + STAGES;           // [STAGES]
  uint64_t* tmem_full_bar = bars + 2 * STAGES;   // [2]
  uint64_t* tmem_empty_bar = bars + 2 * STAGES + 2;  // [2]
  uint32_t* tmem_base_slot = (uint32_t*)(bars + 2 * STAGES + 4);
  volatile int* abort_flag = (volatile int*)(tmem_base_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // the first n_copy CTAs of a launch with an all-gather prologue only move data; the others are the GEMM's CTAs
  const bool ar_pull = p.accumulate == 5 || p.accumulate == 6;  // 6: the owner keeps the sums (reduce-scatter)
  const int n_copy = (p.gather_mode || ar_pull) ? p.n_copy : 0;
  const bool is_copy = p.gather_mode && (int)blockIdx.x < n_copy;
  const bool is_reducer = ar_pull && (int)blockIdx.x < n_copy;
  const int cta = (int)blockIdx.x - n_copy, ncta = (int)gridDim.x - n_copy;
  const int gather_rot = p.gather_mode ? p.comm_rank * p.gather_bps : 0;  // own shard's row blocks come first
  const int tiles_m = (p.M + BLOCK_M - 1) / BLOCK_M;
  const int tiles_n = (p.N + BLOCK_N - 1) / BLOCK_N;
  const int num_tiles = tiles_m * tiles_n * p.batch;
  // pull all-reduce: every wave of tiles covers the rows of all ranks, so that all ranks have tiles to reduce throughout
  const int raster_group = p.gather_mode == 1 ? min(8, p.gather_bps) : (ar_pull ? tiles_m : 8);
  const bool fp8 = p.fp8_a >= 0;
  const int k_elems = fp8 ? 2 * BLOCK_K : BLOCK_K;  // elements per k-block: always 128 bytes
  const int k_blocks = (p.K + k_elems - 1) / k_elems;
  const int k_blocks2 = (p.K2 + k_elems - 1) / k_elems;  // second operand pair (0 if none)

  if (threadIdx.x == 0) {
    if (is_copy) {
      for (int s = 0; s < 2 * STAGES + 4; ++s) mbar_init(&bars[s], 1);  // one barrier per slot of the copy ring
    } else if (is_reducer) {
      // no barriers: a reducer CTA only polls flags in global memory
    } else {
      for (int s = 0; s < STAGES; ++s) {
        mbar_init(&full_bar[s], 1);
        mbar_init(&empty_bar[s], 1);
      }
      for (int a = 0; a < 2; ++a) {
        mbar_init(&tmem_full_bar[a], 1);
        mbar_init(&tmem_empty_bar[a], NUM_EPI_WARPS);  // one arrival per epilogue warp
      }
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (is_reducer) {
    // ------------------------------------------------ all-reduce reducer CTA: all ten warps reduce ----------------
    if (p.dbg && threadIdx.x == 0) p.dbg[blockIdx.x * 4] = p.dbg[blockIdx.x * 4 + 1] = global_timer_ns();
    ar_pull_reduce<BLOCK_N>(p, tiles_m, tiles_n, abort_flag);
    if (p.dbg && threadIdx.x == 0) p.dbg[blockIdx.x * 4 + 2] = global_timer_ns();
    ar_pull_finish(p, (unsigned int)(n_copy * (NUM_THREADS / 32) + ncta * NUM_EPI_WARPS));
    if (p.dbg && threadIdx.x == 0) p.dbg[blockIdx.x * 4 + 3] = global_timer_ns();
  } else if (is_copy) {
    // ------------------------------------------------ all-gather copy CTA -----------------------------------------
    // Lane 0 of warp 0 streams this CTA's share of the remote row blocks peer -> shared-memory ring -> local matrix
    // with bulk async copies and raises the block's flag once its bytes have landed. Remote blocks are visited in
    // order of distance (rank+1 first), the order in which the GEMM CTAs will ask for them.
    if (warp == 0) {
      constexpr int PIECE = 16384;
      constexpr int SLOTS = (L::TILE_BYTES / PIECE) < (2 * STAGES + 4) ? (L::TILE_BYTES / PIECE) : (2 * STAGES + 4);
      constexpr int STORE_LAG = SLOTS - 2;  // loads in flight ahead of the stores (remote latency dominates)
      constexpr int FLAG_LAG = 2;           // a block is flagged once its last store is FLAG_LAG groups behind
      bool ok = true;
      // peers are ready (their shards are final) once the group barrier has completed; CTA 0 runs it for all copy CTAs
      if (blockIdx.x == 0) {
        const bool peers_ok = xl_group_barrier(p.pads, p.comm_rank, p.comm_world, 8, p.err, p.comm_spin_limit);
        if (lane == 0 && peers_ok) xl_st_release_gpu(p.local_sync + 2, 1u);
      }
      if (lane == 0) {
        bool ready = false;
        for (unsigned int i = 0; i < p.comm_spin_limit && !ready; ++i) ready = xl_ld_acquire_gpu(p.local_sync + 2) == 1u;
        if (!ready) {
          ok = false;
          if (p.err) atomicCAS(p.err, 0, (int)XL_COMM_TIMEOUT_FLAG);
        }
        fence_proxy_async_global();  // the peers' shards were written through the generic proxy
        const int remote_blocks = (p.comm_world - 1) * p.gather_bps;
        const int my_chunks = ok ? (remote_blocks - (int)blockIdx.x + n_copy - 1) / n_copy : 0;
        const int ppc = (int)((p.gather_block_bytes + PIECE - 1) / PIECE);  // pieces per row block
        const int total = my_chunks * ppc;
        int flagged = 0;  // chunks of this CTA already flagged
        auto block_of = [&](int chunk_i) {  // chunk_i-th chunk of this CTA -> row block of the full matrix
          const int c = (int)blockIdx.x + chunk_i * n_copy;
          const int peer = (p.comm_rank + 1 + c / p.gather_bps) % p.comm_world;
          return peer * p.gather_bps + c % p.gather_bps;
        };
        auto piece_span = [&](int t, int& peer, long long& off, uint32_t& bytes) {
          const int blk = block_of(t / ppc);
          peer = blk / p.gather_bps;
          const long long in_blk = (long long)(t % ppc) * PIECE;
          off = (long long)blk * p.gather_block_bytes + in_blk;
          const long long left = p.gather_block_bytes - in_blk;
          bytes = (uint32_t)(left < PIECE ? left : PIECE);
        };
        auto flag_done = [&](int upto_piece) {  // every store up to piece `upto_piece` has completed
          while (flagged < my_chunks && (flagged + 1) * ppc - 1 <= upto_piece) {
            fence_proxy_async_global();
            __threadfence();
            xl_st_release_gpu(p.gather_flags + block_of(flagged), 1u);
            ++flagged;
          }
        };
        int loads_issued = 0, stores_issued = 0;
        for (int it = 0; it < total + STORE_LAG && ok; ++it) {
          if (it < total) {
            const int slot = it % SLOTS;
            if (it >= SLOTS) bulk_wait_read<SLOTS - STORE_LAG - 1>();  // the store that last used this slot has read it
            int peer; long long off; uint32_t bytes;
            piece_span(it, peer, off, bytes);
            mbar_expect_tx(&bars[slot], bytes);
            bulk_load(smem + slot * PIECE, p.gather_src[peer] + off, bytes, &bars[slot]);
            ++loads_issued;
          }
          const int j = it - STORE_LAG;
          if (j >= 0) {
            const int slot = j % SLOTS;
            ok = mbar_wait(&bars[slot], (uint32_t)(j / SLOTS) & 1u, abort_flag, p.err, ERR_FULL_WAIT);
            if (!ok) break;
            int peer; long long off; uint32_t bytes;
            piece_span(j, peer, off, bytes);
            bulk_store(p.gather_dst + off, smem + slot * PIECE, bytes);
            bulk_commit();
            ++stores_issued;
            bulk_wait_all<FLAG_LAG>();
            flag_done(j - FLAG_LAG);
          }
        }
        bulk_wait_all<0>();
        if (ok) flag_done(total - 1);
        // after an abort: loads still in flight target this CTA's shared memory; give them a bounded time to land
        for (int t = stores_issued; t < loads_issued; ++t) {
          for (uint32_t i = 0; i < SPIN_LIMIT; ++i)
            if (mbar_try_wait(&bars[t % SLOTS], (uint32_t)(t / SLOTS) & 1u)) break;
        }
      }
      __syncwarp();
      // the peers may not change their shards before every rank has finished reading: the last copy CTA of this rank
      // to finish runs the closing barrier and re-arms the two control words for the next launch
      __threadfence_system();
      unsigned int prev = 0;
      if (lane == 0) prev = atomicAdd(p.local_sync + 3, 1u);
      prev = __shfl_sync(0xffffffffu, prev, 0);
      if (prev == (unsigned int)n_copy - 1) {
        if (lane == 0) { p.local_sync[3] = 0; xl_st_release_gpu(p.local_sync + 2, 0u); }
        xl_group_barrier(p.pads, p.comm_rank, p.comm_world, 9, p.err, p.comm_spin_limit);
      }
    }
  } else if (warp == 0) {
    // ------------------------------------------------ TMA producer ------------------------------------------------
    if (elect_one()) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      uint32_t seen[8] = {0, 0, 0, 0, 0, 0, 0, 0};  // remote row blocks already known to have landed
      auto wait_block = [&](int blk) -> bool {
        if (blk / p.gather_bps == p.comm_rank) return true;  // own shard
        if (blk < 256 && (seen[blk >> 5] >> (blk & 31) & 1u)) return true;
        bool ready = false;
        for (unsigned int i = 0; i < p.comm_spin_limit && !ready; ++i) {
          ready = xl_ld_acquire_gpu(p.gather_flags + blk) == 1u;
          if (!ready && (i & 1023u) == 1023u && *abort_flag) break;
        }
        if (!ready) {
          *abort_flag = 1;
          if (p.err) atomicCAS(p.err, 0, (int)XL_COMM_TIMEOUT_FLAG);
          return false;
        }
        fence_proxy_async_global();  // the block was written through the async proxy of another SM
        if (blk < 256) seen[blk >> 5] |= 1u << (blk & 31);
        return true;
      };
      for (int tile = cta; tile < num_tiles && ok; tile += ncta) {
        int b, mb, nb;
        tile_coords(tile, tiles_m, tiles_n, b, mb, nb, raster_group);
        if (p.gather_mode == 1) {
          mb = (mb + gather_rot) % tiles_m;
          ok = wait_block(mb);
          if (!ok) break;
        }
        const int m0 = mb * BLOCK_M, n0 = nb * BLOCK_N;
        int kb0, kb1;
        if (!tile_k_range(p, mb, nb, k_blocks, BLOCK_N, kb0, kb1)) continue;
        for (int kb_i = kb0; kb_i < kb1 + k_blocks2; ++kb_i) {
          int kb = kb_i;
          const bool second = kb_i >= kb1;  // k-blocks of the second operand pair follow those of the first
          const CUtensorMap* ma = second ? &map_a2 : &map_a;
          const CUtensorMap* mb_ = second ? &map_b2 : &map_b;
          if (second) kb = kb_i - kb1;
          if (p.gather_mode == 2) {
            kb = (kb_i + gather_rot) % k_blocks;
            ok = wait_block(kb);
            if (!ok) break;
          }
          ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.err, ERR_EMPTY_WAIT);
          if (!ok) break;
          uint8_t* sa = smem + stage * L::STAGE_BYTES;
          uint8_t* sb = sa + L::A_BYTES;
          mbar_expect_tx(&full_bar[stage], L::STAGE_BYTES);
          const int k0 = kb * k_elems;
          if (!p.a_mn) {
            tma_load_3d(sa, ma, &full_bar[stage], k0, m0, b);  // box {64 k, 128 m}
          } else {
#pragma unroll
            for (int j = 0; j < BLOCK_M / 64; ++j)              // boxes {64 m, 64 k}
              tma_load_3d(sa + j * (BLOCK_K * 128), ma, &full_bar[stage], m0 + j * 64, k0, b);
          }
          if (!p.b_mn) {
            tma_load_3d(sb, mb_, &full_bar[stage], k0, n0, b);  // box {64 k, BLOCK_N n}
          } else {
#pragma unroll
            for (int j = 0; j < BLOCK_N / 64; ++j)              // boxes {64 n, 64 k}
              tma_load_3d(sb + j * (BLOCK_K * 128), mb_, &full_bar[stage], n0 + j * 64, k0, b);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (is_copy) {
    // the other warps of a copy CTA have nothing to do
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer --------------------------------------------------
    if (elect_one()) {
      const uint32_t fmt = p.is_fp16 ? 0u : 1u;
      const uint32_t fmt_a = fp8 ? (uint32_t)p.fp8_a : fmt, fmt_b = fp8 ? (uint32_t)p.fp8_b : fmt;
      const uint32_t idesc = (1u << 4) | (fmt_a << 7) | (fmt_b << 10) | ((uint32_t)(p.a_mn != 0) << 15) |
                             ((uint32_t)(p.b_mn != 0) << 16) | ((uint32_t)(BLOCK_N >> 3) << 17) |
                             ((uint32_t)(BLOCK_M >> 4) << 24);
      const uint32_t a_lbo = p.a_mn ? BLOCK_K * 128 : 16;
      const uint32_t b_lbo = p.b_mn ? BLOCK_K * 128 : 16;
      const uint32_t a_kstep = p.a_mn ? UMMA_K * 128 : UMMA_K * 2;  // bytes to advance per UMMA_K
      const uint32_t b_kstep = p.b_mn ? UMMA_K * 128 : UMMA_K * 2;
      uint32_t stage = 0, phase = 0;
      uint32_t acc = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = cta; tile < num_tiles && ok; tile += ncta) {
        int kb0 = 0, kb1 = k_blocks;
        if (p.causal) {
          int b, mb, nb;
          tile_coords(tile, tiles_m, tiles_n, b, mb, nb, raster_group);
          if (!tile_k_range(p, mb, nb, k_blocks, BLOCK_N, kb0, kb1)) continue;
        }
        ok = mbar_wait(&tmem_empty_bar[acc], acc_phase ^ 1, abort_flag, p.err, ERR_TMEM_EMPTY_WAIT);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BLOCK_N;
        for (int kb = kb0; kb < kb1 + k_blocks2; ++kb) {
          ok = mbar_wait(&full_bar[stage], phase, abort_flag, p.err, ERR_FULL_WAIT);
          if (!ok) break;
          tcgen05_fence_after();
          const uint32_t sa = smem_u32(smem + stage * L::STAGE_BYTES);
          const uint32_t sb = sa + L::A_BYTES;
#pragma unroll
          for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
            const uint64_t da = make_smem_desc(sa + k * a_kstep, a_lbo);
            const uint64_t db = make_smem_desc(sb + k * b_kstep, b_lbo);
            if (fp8) tcgen05_mma_f8(tmem_d, da, db, idesc, (kb != kb0 || k != 0) ? 1u : 0u);
            else tcgen05_mma_f16(tmem_d, da, db, idesc, (kb != kb0 || k != 0) ? 1u : 0u);
          }
          tcgen05_commit(&empty_bar[stage]);  // frees the stage once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tcgen05_commit(&tmem_full_bar[acc]);  // accumulator complete
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------ epilogue ----------------------------------------------------
    const int q = warp & 3;                     // TMEM lane quarter this warp may access
    const int col_half = (warp - 2) >> 2;       // which half of the accumulator columns this warp drains
    constexpr int COLS_PER_WARP = BLOCK_N / (NUM_EPI_WARPS / 4);
    uint32_t acc = 0, acc_phase = 0;
    bool ok = true;
    float mean_a = 0.f, mean_b = 1.f;
    if (p.dbg && ar_pull && warp == 2 && lane == 0) p.dbg[blockIdx.x * 4] = global_timer_ns();
    const bool push = p.accumulate == 3 || p.accumulate == 4;  // tiles are pushed into the peers' buffers
    const int acc_mode = ar_pull ? 0 : p.accumulate;           // the pull all-reduce stores plain partial tiles
    const float alpha_eff = p.alpha_log2 ? p.alpha * exp2f(*p.alpha_log2) : p.alpha;
    if (p.accumulate == 2) {
      const float t = *p.step;
      mean_a = t / (t + 1.f);
      mean_b = 1.f / (t + 1.f);
    }
    if (push) {
      // Nobody may push into a peer's output before that peer has zeroed it, i.e. before it has entered this kernel:
      // the first epilogue warp of the first GEMM CTA runs the cross-rank barrier and publishes it to the other CTAs.
      if (cta == 0 && warp == 2) {
        const bool peers_ok = xl_group_barrier(p.pads, p.comm_rank, p.comm_world, 0, p.err, p.comm_spin_limit);
        if (lane == 0 && peers_ok) xl_st_release_gpu(p.local_sync, 1u);
      }
      bool ready = false;
      for (unsigned int i = 0; i < p.comm_spin_limit && !ready; ++i) {
        ready = xl_ld_acquire_gpu(p.local_sync) == 1u;
        if (!ready && (i & 1023u) == 1023u && *abort_flag) break;
      }
      if (!ready) {
        ok = false;
        *abort_flag = 1;
        if (p.err) atomicCAS(p.err, 0, (int)XL_COMM_TIMEOUT_FLAG);
      }
    }
    for (int tile = cta; tile < num_tiles && ok; tile += ncta) {
      int b, mb, nb;
      tile_coords(tile, tiles_m, tiles_n, b, mb, nb, raster_group);
      if (p.gather_mode == 1) mb = (mb + gather_rot) % tiles_m;
      if (p.causal == 1 && nb * BLOCK_N > mb * BLOCK_M + BLOCK_M - 1) continue;
      ok = mbar_wait(&tmem_full_bar[acc], acc_phase, abort_flag, p.err, ERR_TMEM_FULL_WAIT);
      if (!ok) break;
      tcgen05_fence_after();
      const int row = mb * BLOCK_M + q * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BLOCK_N;
      uint8_t* crow;
      if (p.accumulate == 4) {
        // reduce-scatter: the row lives in the output shard of its owner rank
        const int owner = row_ok ? row / p.rs_rows : 0;
        crow = (uint8_t*)p.rs_dst[owner] + (long long)(row - owner * p.rs_rows) * p.ldc * 2;
      } else {
        crow = (uint8_t*)p.C + ((long long)b * p.batch_stride_c + (long long)row * p.ldc) * (p.c_dtype == XL_F32 ? 4 : 2);
      }
      if (push) {
        // Pushes over NVLink should be whole 128-byte lines. TMEM hands every lane one row, so the tile goes through
        // a per-warp staging area in shared memory (32 rows x 64 columns, 16-byte chunks swizzled by row): written by
        // rows, read back with eight lanes covering 128 contiguous bytes of one row.
        uint8_t* stage = smem + L::TILE_BYTES + 256 + (warp - 2) * EPI_STAGE_BYTES;
        const bool bf = p.c_dtype == XL_BF16;
#pragma unroll 1
        for (int c = col_half * COLS_PER_WARP; c < (col_half + 1) * COLS_PER_WARP; c += 64) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(taddr + c + h * 32, r);
            tmem_ld_wait();
            const int col0 = nb * BLOCK_N + c + h * 32;
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
              uint4 o;
              uint16_t* oe = (uint16_t*)&o;
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                float val = __uint_as_float(r[jj * 8 + e]) * alpha_eff;
                if (p.bias && col0 + jj * 8 + e < p.N) {
                  const int bc = col0 + jj * 8 + e;
                  val += p.bias_dtype == XL_F32 ? ((const float*)p.bias)[bc]
                         : p.bias_dtype == XL_BF16 ? __bfloat162float(((const __nv_bfloat16*)p.bias)[bc])
                                                   : __half2float(((const __half*)p.bias)[bc]);
                }
                if (p.act) val = apply_act(val, p.act);
                oe[e] = bf ? __bfloat16_as_ushort(__float2bfloat16_rn(val)) : __half_as_ushort(__float2half_rn(val));
              }
              const int chunk = h * 4 + jj;
              *(uint4*)(stage + lane * 128 + ((chunk ^ (lane & 7)) << 4)) = o;
            }
          }
          __syncwarp();
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int rr = it * 4 + (lane >> 3), cc = lane & 7;
            const uint4 o = *(const uint4*)(stage + rr * 128 + ((cc ^ (rr & 7)) << 4));
            const int grow = mb * BLOCK_M + q * 32 + rr;
            const int gcol = nb * BLOCK_N + c + cc * 8;
            if (grow < p.M && gcol < p.N) {
              uint16_t* dst;
              if (p.accumulate == 4) {
                const int owner = grow / p.rs_rows;
                dst = (uint16_t*)p.rs_dst[owner] + (long long)(grow - owner * p.rs_rows) * p.ldc + gcol;
                if (bf) xl_red_add_bf16x8(dst, o);
                else xl_red_add_f16x8(dst, o);
              } else {
                dst = (uint16_t*)p.C + (long long)grow * p.ldc + gcol;
                if (bf) xl_multimem_red_add_bf16x8(dst, o);
                else xl_multimem_red_add_f16x8(dst, o);
              }
            }
          }
          __syncwarp();
        }
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty_bar[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        continue;
      }
#pragma unroll 1
      for (int c = col_half * COLS_PER_WARP; c < (col_half + 1) * COLS_PER_WARP; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c, r);
        tmem_ld_wait();
        const int col0 = nb * BLOCK_N + c;
        if (!row_ok || col0 >= p.N) continue;
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
              if (acc_mode) {
                const float4 old = *(const float4*)(dst + j);
                if (acc_mode == 1) { o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w; }
                else { o.x = old.x * mean_a + o.x * mean_b; o.y = old.y * mean_a + o.y * mean_b;
                       o.z = old.z * mean_a + o.z * mean_b; o.w = old.w * mean_a + o.w * mean_b; }
              }
              *(float4*)(dst + j) = o;
            }
          } else {
            for (int j = 0; j < 32 && col0 + j < p.N; ++j) {
              float o = v[j];
              if (acc_mode == 1) o += dst[j];
              else if (acc_mode == 2) o = dst[j] * mean_a + o * mean_b;
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
              if (acc_mode) old = *(const uint4*)(dst + j);
              uint4 o;
              uint16_t* oe = (uint16_t*)&o;
              const uint16_t* ol = (const uint16_t*)&old;
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                float val = v[j + e];
                if (acc_mode) {
                  const float prev = bf ? __bfloat162float(__ushort_as_bfloat16(ol[e])) : __half2float(__ushort_as_half(ol[e]));
                  val = acc_mode == 1 ? prev + val : prev * mean_a + val * mean_b;
                }
                oe[e] = bf ? __bfloat16_as_ushort(__float2bfloat16_rn(val)) : __half_as_ushort(__float2half_rn(val));
              }
              *(uint4*)(dst + j) = o;
            }
          } else {
            for (int j = 0; j < 32 && col0 + j < p.N; ++j) {
              float val = v[j];
              if (acc_mode) {
                const float prev = bf ? __bfloat162float(__ushort_as_bfloat16(dst[j])) : __half2float(__ushort_as_half(dst[j]));
                val = acc_mode == 1 ? prev + val : prev * mean_a + val * mean_b;
              }
              dst[j] = bf ? __bfloat16_as_ushort(__float2bfloat16_rn(val)) : __half_as_ushort(__float2half_rn(val));
            }
          }
        }
      }
      // all TMEM reads of this warp are complete (wait::ld above): hand the accumulator back to the MMA warp
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty_bar[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      if (ar_pull) {
        // this warp's part of the partial tile is in this rank's buffer: tell the rank that reduces these rows
        __threadfence_system();
        __syncwarp();
        if (lane == 0) {
          const int owner = (mb * BLOCK_M) / p.ar_rows;
          red_release_sys_add_u32(p.ar_flags[owner] + (mb * tiles_n + nb), 1u);
        }
      }
    }
    if (ar_pull) {
      // out of tiles: help with the reduction of this rank's rows until nothing is left, then check in
      const bool stamp = p.dbg && warp == 2 && lane == 0;
      if (stamp) p.dbg[blockIdx.x * 4 + 1] = global_timer_ns();
      if (ok) ar_pull_reduce<BLOCK_N>(p, tiles_m, tiles_n, abort_flag);
      if (stamp) p.dbg[blockIdx.x * 4 + 2] = global_timer_ns();
      ar_pull_finish(p, (unsigned int)(n_copy * (NUM_THREADS / 32) + ncta * NUM_EPI_WARPS));
      if (stamp) p.dbg[blockIdx.x * 4 + 3] = global_timer_ns();
    }
    if (push) {
      // The kernel may only finish once every rank's pushes have landed here: the last epilogue warp of this rank
      // to finish runs the closing cross-rank barrier (each warp fences its own pushes first).
      __threadfence_system();
      unsigned int prev = 0;
      if (lane == 0) prev = atomicAdd(p.local_sync + 1, 1u);
      prev = __shfl_sync(0xffffffffu, prev, 0);
      if (prev == (unsigned int)ncta * NUM_EPI_WARPS - 1) {
        // every epilogue warp of this rank has passed the ready check by now: re-arm both words for the next launch
        if (lane == 0) { p.local_sync[1] = 0; xl_st_release_gpu(p.local_sync, 0u); }
        xl_group_barrier(p.pads, p.comm_rank, p.comm_world, 1, p.err, p.comm_spin_limit);
      }
    }
  }

  // ---- teardown: every role arrives here, also after an abort --------------------------------------------------------
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---- host side -------------------------------------------------------------------------------------------------------
// 3-D map over a row-major matrix with `rows` rows of `cols` contiguous elements (leading dimension `ld`), `batch`
// matrices `batch_stride` elements apart; boxes of {box_cols, box_rows, 1} with 128-byte swizzle.
int make_map(CUtensorMap* map, const void* ptr, int is_fp16, long long rows, long long cols, long long ld,
             long long batch, long long batch_stride, int box_cols, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -2;
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batch};
  const cuuint64_t esz = is_fp16 == 2 ? 1 : 2;  // is_fp16: 0 bf16, 1 fp16, 2 one-byte elements (fp8)
  cuuint64_t strides[2] = {(cuuint64_t)ld * esz, (cuuint64_t)(batch > 1 ? batch_stride : rows * ld) * esz};
  cuuint32_t box[3] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapDataType dt = is_fp16 == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                 : is_fp16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUresult r = fn(map, dt, 3, (void*)ptr, dims,
                  strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

template <int BLOCK_N>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, int sm_count, cudaStream_t s,
           const CUtensorMap* ma2 = nullptr, const CUtensorMap* mb2 = nullptr) {
  using L = SmemLayout<BLOCK_N>;
  static bool configured = false;
  constexpr int TOTAL_COMM = L::TOTAL + NUM_EPI_WARPS * EPI_STAGE_BYTES;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BLOCK_N>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         TOTAL_COMM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int smem_bytes = (p.accumulate == 3 || p.accumulate == 4) ? TOTAL_COMM : L::TOTAL;
  const int tiles = ((p.M + BLOCK_M - 1) / BLOCK_M) * ((p.N + BLOCK_N - 1) / BLOCK_N) * p.batch;
  // copy / reducer CTAs and GEMM CTAs wait on one another: all must be resident
  const int n_copy = (p.gather_mode || p.accumulate >= 5) ? p.n_copy : 0;
  const int gemm_ctas = tiles < sm_count - n_copy ? tiles : sm_count - n_copy;
  const int grid = gemm_ctas + n_copy;
  // without a second operand pair the kernel never touches the second pair of maps: pass the first pair again
  gemm_tcgen05_kernel<BLOCK_N><<<grid, NUM_THREADS, smem_bytes, s>>>(ma, mb, ma2 ? *ma2 : ma, mb2 ? *mb2 : mb, p);
  return (int)cudaGetLastError();
}

}  // namespace

// C = epilogue(A * B), 16-bit operands, fp32 accumulation.
//   a: if a_mn == 0 stored (M x K) row-major with leading dimension lda; if a_mn == 1 stored (K x M) row-major.
//   b: if b_mn == 0 stored (N x K) row-major with leading dimension ldb; if b_mn == 1 stored (K x N) row-major.
//   Leading dimensions and batch strides are in elements; pointers and leading dimensions must be 16-byte aligned.
//   err: device int that receives a non-zero code if a bounded wait inside the kernel gave up (may be null).
//   accumulate == 3 (GEMM fused with an all-reduce over NVSwitch): `c` is the multicast address of an output buffer
//   that every rank of the group zeroed in stream order before this launch; comm_pads = device array with the signal
//   pad of every rank, comm_local_sync = two zero-initialised device words of this rank (the kernel leaves them zero).
//   All ranks must launch the same GEMM shape. No launch argument changes between calls, so the launch can be
//   captured in a CUDA graph and replayed.
// Returns 0, a CUDA error code, or a negative value when the arguments are not supported by this kernel.
// Full entry point. On top of xl_gemm_tcgen05:
//   causal = 1 / 2 / 3: square attention products whose masked half is not computed (see GemmParams::causal).
//   accumulate == 4 (GEMM fused with a reduce-scatter over NVLink): row r of the product is added (`red.add`, 16-byte
//   vectors) into the output shard of rank r / rs_rows; rs_dst = device array with every rank's shard buffer
//   (rs_rows x ldc, zeroed in stream order before the launch), M == rs_rows * comm_world. `c` is unused.
//   gather_mode != 0 (all-gather fused into the GEMM): the sharded operand (1: A sharded over M, 2: B stored (K x N)
//   and sharded over K) lives in a full-size matrix of which only this rank's row range is valid at launch;
//   gather_src = device array with that matrix in every rank's memory, gather_dst = this rank's copy (the pointer
//   also given as `a` / `b`), gather_flags = one zeroed word per row block (128 rows of A / 64 rows of B),
//   gather_bps = row blocks per shard, n_copy = number of CTAs that pull the remote row blocks (bulk async copies
//   through shared memory) while the remaining CTAs start on the local rows. The gathered matrix stays valid after
//   the kernel. Uses comm_local_sync[2..3] and signal channels 8 and 9.
XL_API int xl_gemm_tcgen05_fused(const void* a, const void* b, void* c, int M, int N, int K, int batch, int a_mn, int b_mn,
                                 long long lda, long long ldb, long long ldc, long long stride_a, long long stride_b,
                                 long long stride_c, int ab_is_fp16, int c_dtype, const void* bias, int bias_dtype,
                                 int act, int accumulate, const float* step, float alpha, int* err, int sm_count,
                                 const void* comm_pads, int comm_rank, int comm_world, unsigned int* comm_local_sync,
                                 const void* rs_dst, int rs_rows, int gather_mode, const void* gather_src,
                                 void* gather_dst, unsigned int* gather_flags, int gather_bps, int n_copy, int causal,
                                 cudaStream_t s) {
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return -1;
  if ((((uintptr_t)a) & 15) || (((uintptr_t)b) & 15) || (lda % 8) || (ldb % 8)) return -1;
  if (batch > 1 && ((stride_a % 8) || (stride_b % 8))) return -1;
  if (sm_count <= 0) sm_count = 148;
  int block_n = (N <= 128) ? 128 : 256;
  // too few 128 x 256 tiles to occupy half of the SMs: narrower tiles double the CTAs that work
  if (block_n == 256 && !gather_mode && accumulate < 3 &&
      2LL * ((M + BLOCK_M - 1) / BLOCK_M) * ((N + 255) / 256) * batch <= sm_count)
    block_n = 128;
  CUtensorMap ma, mb;
  int r;
  if (!a_mn) r = make_map(&ma, a, ab_is_fp16, M, K, lda, batch, stride_a, BLOCK_K, BLOCK_M);
  else r = make_map(&ma, a, ab_is_fp16, K, M, lda, batch, stride_a, 64, BLOCK_K);
  if (r) return r;
  if (!b_mn) r = make_map(&mb, b, ab_is_fp16, N, K, ldb, batch, stride_b, BLOCK_K, block_n);
  else r = make_map(&mb, b, ab_is_fp16, K, N, ldb, batch, stride_b, 64, BLOCK_K);
  if (r) return r;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.batch = batch;
  p.a_mn = a_mn; p.b_mn = b_mn;
  p.C = c; p.ldc = ldc; p.batch_stride_c = stride_c; p.c_dtype = c_dtype;
  p.bias = bias; p.bias_dtype = bias_dtype; p.act = act; p.accumulate = accumulate; p.step = step;
  p.alpha = alpha; p.is_fp16 = ab_is_fp16; p.err = err;
  p.pads = (unsigned int* const*)comm_pads; p.comm_rank = comm_rank; p.comm_world = comm_world;
  p.local_sync = comm_local_sync; p.comm_spin_limit = xl_host_comm_spin_limit;
  p.rs_dst = (void* const*)rs_dst; p.rs_rows = rs_rows;
  p.gather_mode = gather_mode; p.n_copy = n_copy; p.gather_bps = gather_bps;
  p.gather_src = (const uint8_t* const*)gather_src; p.gather_dst = (uint8_t*)gather_dst; p.gather_flags = gather_flags;
  p.gather_block_bytes = 0;
  p.fp8_a = p.fp8_b = -1;
  p.alpha_log2 = nullptr;
  p.K2 = 0; p.ar_src_mc = nullptr; p.ar_dst_mc = nullptr; p.ar_flags = nullptr; p.ar_rows = 0; p.dbg = nullptr;
  p.causal = causal;
  if (causal < 0 || causal > 3 || (causal && (gather_mode || accumulate >= 3))) return -1;
  if (causal && (M != N && causal == 1)) return -1;
  if (causal >= 2 && M != K) return -1;
  if (sm_count <= 0) sm_count = 148;
  if (accumulate >= 3 && (comm_pads == nullptr || comm_local_sync == nullptr || (N % 8) || c_dtype == XL_F32 ||
                          (ldc % 8) || comm_world > 32 || batch != 1))
    return -1;
  if (accumulate == 4 && (rs_dst == nullptr || rs_rows <= 0 || (long long)rs_rows * comm_world != M)) return -1;
  if (accumulate > 4 || accumulate < 0) return -1;
  if (gather_mode) {
    if (gather_mode != 1 && gather_mode != 2) return -1;
    if (comm_pads == nullptr || comm_local_sync == nullptr || gather_src == nullptr || gather_dst == nullptr ||
        gather_flags == nullptr || comm_world < 2 || comm_world > 32 || batch != 1 || n_copy < 1 ||
        n_copy > sm_count / 2 || gather_bps < 1)
      return -1;
    if (gather_mode == 1) {  // A: (M x K) K-major, contiguous rows, M = world * bps * BLOCK_M
      if (a_mn || lda != K || (long long)gather_bps * comm_world * BLOCK_M != M || gather_dst != a) return -1;
      p.gather_block_bytes = (long long)BLOCK_M * K * 2;
    } else {                 // B: (K x N) with N contiguous, K = world * bps * BLOCK_K
      if (!b_mn || ldb != N || (long long)gather_bps * comm_world * BLOCK_K != K || gather_dst != b) return -1;
      p.gather_block_bytes = (long long)BLOCK_K * N * 2;
    }
  }
  if (block_n == 128) return launch<128>(ma, mb, p, sm_count, s);
  return launch<256>(ma, mb, p, sm_count, s);
}

// C = 2^(*alpha_log2) * alpha * (A * B^T) for 8-bit float operands (tcgen05 kind::f8f6f4), fp32 accumulation.
//   a: (M x K) row-major, b: (N x K) row-major (both K-major), one byte per element, formats fmt_a / fmt_b
//   (0 = e4m3, 1 = e5m2); lda, ldb multiples of 16; c: (M x N) fp32 / fp16 / bf16; alpha_log2 may be null.
XL_API int xl_gemm_tcgen05_fp8(const void* a, const void* b, void* c, int M, int N, int K, long long lda, long long ldb,
                               long long ldc, int fmt_a, int fmt_b, int c_dtype, const void* bias, int bias_dtype,
                               float alpha, const float* alpha_log2, int* err, int sm_count, cudaStream_t s) {
  if (M <= 0 || N <= 0 || K <= 0 || fmt_a < 0 || fmt_a > 1 || fmt_b < 0 || fmt_b > 1) return -1;
  if ((((uintptr_t)a) & 15) || (((uintptr_t)b) & 15) || (lda % 16) || (ldb % 16)) return -1;
  const int block_n = (N <= 128) ? 128 : 256;
  CUtensorMap ma, mb;
  int r = make_map(&ma, a, 2, M, K, lda, 1, 0, 2 * BLOCK_K, BLOCK_M);
  if (r) return r;
  r = make_map(&mb, b, 2, N, K, ldb, 1, 0, 2 * BLOCK_K, block_n);
  if (r) return r;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.batch = 1;
  p.a_mn = 0; p.b_mn = 0;
  p.C = c; p.ldc = ldc; p.batch_stride_c = 0; p.c_dtype = c_dtype;
  p.bias = bias; p.bias_dtype = bias_dtype; p.act = 0; p.accumulate = 0; p.step = nullptr;
  p.alpha = alpha; p.is_fp16 = 0; p.err = err;
  p.pads = nullptr; p.comm_rank = 0; p.comm_world = 1; p.local_sync = nullptr; p.comm_spin_limit = 0;
  p.rs_dst = nullptr; p.rs_rows = 0;
  p.gather_mode = 0; p.n_copy = 0; p.gather_bps = 0; p.gather_src = nullptr; p.gather_dst = nullptr;
  p.gather_flags = nullptr; p.gather_block_bytes = 0;
  p.causal = 0;
  p.fp8_a = fmt_a; p.fp8_b = fmt_b; p.alpha_log2 = alpha_log2;
  p.K2 = 0; p.ar_src_mc = nullptr; p.ar_dst_mc = nullptr; p.ar_flags = nullptr; p.ar_rows = 0; p.dbg = nullptr;
  if (sm_count <= 0) sm_count = 148;
  if (block_n == 128) return launch<128>(ma, mb, p, sm_count, s);
  return launch<256>(ma, mb, p, sm_count, s);
}

// C = epilogue(A * B), 16-bit operands, fp32 accumulation (no reduce-scatter, no all-gather prologue).
XL_API int xl_gemm_tcgen05(const void* a, const void* b, void* c, int M, int N, int K, int batch, int a_mn, int b_mn,
                           long long lda, long long ldb, long long ldc, long long stride_a, long long stride_b,
                           long long stride_c, int ab_is_fp16, int c_dtype, const void* bias, int bias_dtype, int act,
                           int accumulate, const float* step, float alpha, int* err, int sm_count,
                           const void* comm_pads, int comm_rank, int comm_world, unsigned int* comm_local_sync,
                           cudaStream_t s) {
  if (accumulate > 3) return -1;
  return xl_gemm_tcgen05_fused(a, b, c, M, N, K, batch, a_mn, b_mn, lda, ldb, ldc, stride_a, stride_b, stride_c,
                               ab_is_fp16, c_dtype, bias, bias_dtype, act, accumulate, step, alpha, err, sm_count,
                               comm_pads, comm_rank, comm_world, comm_local_sync, nullptr, 0, 0, nullptr, nullptr,
                               nullptr, 0, 0, 0, s);
}

// all_reduce over the ranks of a group of (A * B [+ A2 * B2]), 16-bit operands and result, fp32 accumulation, in one kernel
// that pulls: see GemmParams::ar_src_mc. Operand conventions as xl_gemm_tcgen05 (a2 / b2 have the layouts of a / b;
// K2 = 0 and null pointers: a single product).
//   partial      this rank's buffer for its partial product (M x ldc, symmetric memory), partial_mc its multicast address
//   result_mc    multicast address of the (M x ldc) result buffers: after the kernel every rank's buffer holds the sum.
//                With scatter != 0 (reduce-scatter) instead this rank's own (M / world x ldc) result shard (an ordinary
//                address): after the kernel it holds the sums of this rank's rows
//   flags        device array [world] with every rank's flag words (2 * tiles words each, symmetric memory, zero before
//                the first launch; the kernel leaves them zero), tiles = (M / 128) * ceil(N / 256 or 128)
//   rows are split evenly: M must be a multiple of 128 * world. n_red: CTAs that only reduce (at least 1).
//   timestamps: optional device array of 4 x grid 64-bit words: per CTA the global timer (ns) at its start, when it ran
//   out of tiles, when it ran out of reduce work and when it had checked in (for tuning; null in production).
//   Uses comm_local_sync[8..9] and signal channel 2; no launch argument changes between calls (graph replay is fine).
// Returns 0, a CUDA error code, or a negative value when the arguments are not supported.
XL_API int xl_gemm_tcgen05_ar_pull(const void* a, const void* b, const void* a2, const void* b2, void* partial,
                                   const void* partial_mc, void* result_mc, int M, int N, int K, int K2, int a_mn, int b_mn,
                                   long long lda, long long ldb, long long lda2, long long ldb2, long long ldc,
                                   int ab_is_fp16, int c_dtype, float alpha, int* err, int sm_count, const void* comm_pads,
                                   int comm_rank, int comm_world, unsigned int* comm_local_sync, const void* flags,
                                   int n_red, int scatter, unsigned long long* timestamps, cudaStream_t s) {
  if (M <= 0 || N <= 0 || K <= 0 || K2 < 0) return -1;
  if ((((uintptr_t)a) & 15) || (((uintptr_t)b) & 15) || (lda % 8) || (ldb % 8)) return -1;
  if (K2 && ((((uintptr_t)a2) & 15) || (((uintptr_t)b2) & 15) || (lda2 % 8) || (ldb2 % 8) || !a2 || !b2)) return -1;
  if (comm_pads == nullptr || comm_local_sync == nullptr || flags == nullptr || partial == nullptr ||
      partial_mc == nullptr || result_mc == nullptr)
    return -1;
  if (comm_world < 2 || comm_world > 32 || (N % 8) || (ldc % 8) || c_dtype == XL_F32 || n_red < 1) return -1;
  if (M % (BLOCK_M * comm_world)) return -1;
  if ((((uintptr_t)partial) & 15) || (((uintptr_t)partial_mc) & 15) || (((uintptr_t)result_mc) & 15)) return -1;
  if (sm_count <= 0) sm_count = 148;
  if (n_red > sm_count / 2) return -1;
  // narrower tiles give more waves per launch (less left to reduce after the last one) at some cost in MMA efficiency
  static const int forced_block_n = [] { const char* e = getenv("XL_AR_PULL_BLOCK_N"); return e ? atoi(e) : 0; }();
  const int block_n = (N <= 128 || forced_block_n == 128) ? 128 : 256;
  CUtensorMap ma, mb, ma2, mb2;
  int r;
  if (!a_mn) r = make_map(&ma, a, ab_is_fp16, M, K, lda, 1, 0, BLOCK_K, BLOCK_M);
  else r = make_map(&ma, a, ab_is_fp16, K, M, lda, 1, 0, 64, BLOCK_K);
  if (r) return r;
  if (!b_mn) r = make_map(&mb, b, ab_is_fp16, N, K, ldb, 1, 0, BLOCK_K, block_n);
  else r = make_map(&mb, b, ab_is_fp16, K, N, ldb, 1, 0, 64, BLOCK_K);
  if (r) return r;
  if (K2) {
    if (!a_mn) r = make_map(&ma2, a2, ab_is_fp16, M, K2, lda2, 1, 0, BLOCK_K, BLOCK_M);
    else r = make_map(&ma2, a2, ab_is_fp16, K2, M, lda2, 1, 0, 64, BLOCK_K);
    if (r) return r;
    if (!b_mn) r = make_map(&mb2, b2, ab_is_fp16, N, K2, ldb2, 1, 0, BLOCK_K, block_n);
    else r = make_map(&mb2, b2, ab_is_fp16, K2, N, ldb2, 1, 0, 64, BLOCK_K);
    if (r) return r;
  }
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.batch = 1;
  p.a_mn = a_mn; p.b_mn = b_mn;
  p.C = partial; p.ldc = ldc; p.batch_stride_c = 0; p.c_dtype = c_dtype;
  p.bias = nullptr; p.bias_dtype = 0; p.act = 0; p.accumulate = scatter ? 6 : 5; p.step = nullptr;
  p.alpha = alpha; p.is_fp16 = ab_is_fp16; p.err = err;
  p.pads = (unsigned int* const*)comm_pads; p.comm_rank = comm_rank; p.comm_world = comm_world;
  p.local_sync = comm_local_sync; p.comm_spin_limit = xl_host_comm_spin_limit;
  p.rs_dst = nullptr; p.rs_rows = 0;
  p.gather_mode = 0; p.n_copy = n_red; p.gather_bps = 0; p.gather_src = nullptr; p.gather_dst = nullptr;
  p.gather_flags = nullptr; p.gather_block_bytes = 0;
  p.causal = 0;
  p.fp8_a = p.fp8_b = -1;
  p.alpha_log2 = nullptr;
  p.K2 = K2;
  p.ar_src_mc = (const uint8_t*)partial_mc; p.ar_dst_mc = (uint8_t*)result_mc;
  p.ar_flags = (unsigned int* const*)flags; p.ar_rows = M / comm_world; p.dbg = timestamps;
  if (block_n == 128) return launch<128>(ma, mb, p, sm_count, s, K2 ? &ma2 : nullptr, K2 ? &mb2 : nullptr);
  return launch<256>(ma, mb, p, sm_count, s, K2 ? &ma2 : nullptr, K2 ? &mb2 : nullptr);
}
