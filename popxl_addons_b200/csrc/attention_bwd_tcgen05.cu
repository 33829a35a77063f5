// Causal softmax attention backward, first pass, in one kernel on the 5th-generation tensor cores (tcgen05) for sm_100a.
//
//   P  = softmax(scale * Q K^T + causal mask)          (recomputed from Q, K and the forward pass's log-sum-exp)
//   dP = dO V^T
//   dS = P o (dP - delta) * scale,   delta_i = sum_d dO_id O_id
//   dQ = dS K                                           accumulated on chip over all key blocks
//
// One CTA owns 128 query rows of one (batch, head) and walks the key / value rows in blocks of BKV. The scores, dP and
// the dQ accumulator never leave the chip; P and dS are written once, as 16-bit (B*H, S, S) matrices, for the two
// remaining products of the backward pass (dV = P^T dO, dK = dS^T Q), which are plain batched GEMMs over the causal
// half. That is the minimum of five products, against eight for a backward pass that recomputes the scores in a second,
// key-stationary kernel: with head dimension 256 the dK and dV accumulators alone fill the 512 TMEM columns, so a
// single kernel cannot hold them next to the score tiles.
//
//   warp 0      TMA producer : Q and dO tiles once, then K blocks and V blocks into two 2-stage shared-memory rings
//   warp 1      MMA issuer   : S_j = Q K_j^T and dP_j = dO V_j^T into one of two TMEM buffer pairs (block j+1 is issued
//                              before dS_j is awaited, so it overlaps the element-wise work on block j), then
//                              dQ += dS_j K_j (K_j consumed MN-major: no transpose)
//   warps 2..5  element-wise : one thread per query row. tcgen05.ld of the score and dP rows, p = exp2(s*c - lse*log2e),
//                              ds = p (dp - delta) scale, P and dS rows to global memory, dS as a 16-bit tile to shared
//                              memory (two buffers) for the third product; finally dQ from TMEM to global memory.
//
// TMEM columns: [0, D) dQ accumulator, then two score buffers and two dP buffers of BKV columns each (512 allocated, one
// CTA per SM). Every wait on an mbarrier is bounded: when a wait gives up the kernel records a code in `*err`, raises a
// CTA-wide abort flag, all roles leave their loops, TMEM is released and the kernel returns normally.
#include "tcgen05.cuh"
#include "attention_split.cuh"

namespace {

constexpr int BLOCK_Q = 128;
constexpr int UMMA_K = 16;
constexpr int K_STAGES = 3;  // a K block is held until the third product of its keys: one more stage than V
constexpr int V_STAGES = 2;
constexpr int NUM_EW_WARPS = 4;
constexpr int NUM_THREADS = 64 + 32 * NUM_EW_WARPS;
constexpr uint32_t SPIN_LIMIT = xl_tc::MBAR_SPIN_LIMIT;
constexpr uint32_t TMEM_COLS = 512;

enum { ERR_QDO_WAIT = 31, ERR_KV_FULL_WAIT = 32, ERR_KV_EMPTY_WAIT = 33, ERR_SDP_FULL_WAIT = 34, ERR_SDP_EMPTY_WAIT = 35,
       ERR_DS_FULL_WAIT = 36, ERR_DS_EMPTY_WAIT = 37, ERR_DQ_DONE_WAIT = 38 };

struct AttnBwdParams {
  int B, S, H, D;
  int q_col, k_col, v_col;   // first column of head 0 of Q / K / V in the packed matrix
  const void* out;           // forward output O (B*S x ldo), head h in columns [h*D, (h+1)*D)
  long long ldo;
  const void* dout;          // dO, same layout, leading dimension ld_do (read directly for delta; also behind map_do)
  long long ld_do;
  const float* lse;          // (B, H, S) natural-log log-sum-exp of the scaled scores, from the forward pass
  void* P;                   // (B*H, S, S) 16-bit: probabilities, zero above the diagonal inside the blocks that are written
  void* dS;                  // (B*H, S, S) 16-bit
  void* dq;                  // dQ: (B*S x ld_dq) 16-bit, head h in columns [dq_col + h*D, ...)
  long long ld_dq;
  int dq_col;
  float scale;
  int causal;
  int is_fp16;
  int* err;
  // Key-range splitting (chunk > 0): a query block's key blocks are divided evenly over ceil(n / chunk) CTAs. Each writes
  // its partial dQ (fp32) to the workspace; a second kernel adds the partials of every row up and writes dQ.
  int chunk;
  int items;               // CTAs per head and batch entry (grid y)
  float* part_dq;          // [B*H*items][128][D]
  float* delta;            // (B, H, S) scratch: dO . O of every row, filled by a first kernel of the launch
  long long* trace;        // optional (tuning): clock64 stamps of CTA (0, 0, 0): [role 0 MMA thread | role 1 warp 2][block][8]
};

#define XL_ATTN_BWD_STAMP(role, j, point)                                                              \
  do {                                                                                                 \
    if (p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (j) < 64)       \
      p.trace[((role) * 64 + (j)) * 8 + (point)] = clock64();                                          \
  } while (0)

using namespace xl_tc;
using namespace xl_attn_split;

// Shared-memory matrix descriptor of a K-major operand stored without swizzle as 8-row x 16-byte core matrices:
// `lbo` = byte distance between core matrices adjacent along K, `sbo` = between 8-row groups (layout type 0).
__device__ __forceinline__ uint64_t make_smem_desc_noswizzle(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;
  return d;
}
// 128-byte-swizzled tile whose swizzle atoms (8 rows x 128 B) are `sbo` = 1024 bytes apart, column blocks `lbo` apart
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr, uint32_t lbo) { return make_smem_desc(smem_addr, lbo); }

template <int D, int BKV>
struct BwdSmem {
  static constexpr int Q_BYTES = BLOCK_Q * D * 2;       // D/64 k-blocks of (128 rows x 128 B)
  static constexpr int K_BYTES = BKV * D * 2;           // D/64 boxes of (BKV rows x 128 B): K-major for S, MN-major for dQ
  static constexpr int V_BYTES = BKV * D * 2;
  static constexpr int DS_BYTES = BLOCK_Q * BKV * 2;    // BKV/8 chunk columns of 16 row groups of (8 rows x 16 B)
  static constexpr int TILE_BYTES = 2 * Q_BYTES + K_STAGES * K_BYTES + V_STAGES * V_BYTES + 2 * DS_BYTES;
  static constexpr int NEEDED = TILE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
  // more than half of an SM's shared memory, so that two CTAs (each holding all 512 TMEM columns) never share an SM
  static constexpr int TOTAL = NEEDED > 120 * 1024 ? NEEDED : 120 * 1024;
};

template <int D, int BKV>
__global__ void __launch_bounds__(NUM_THREADS, 1)
    attn_bwd_dq_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                               const __grid_constant__ CUtensorMap map_kv, const AttnBwdParams p) {
  using L = BwdSmem<D, BKV>;
  static_assert(D % 64 == 0 && D <= 256 && BKV % 32 == 0 && BKV <= 64 && D + 4 * BKV <= (int)TMEM_COLS, "unsupported tile");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;
  uint8_t* sDO = smem + L::Q_BYTES;
  uint8_t* sK = smem + 2 * L::Q_BYTES;              // K_STAGES blocks
  uint8_t* sV = sK + K_STAGES * L::K_BYTES;          // V_STAGES blocks
  uint8_t* sDS = sV + V_STAGES * L::V_BYTES;         // two buffers
  uint64_t* bars = (uint64_t*)(smem + L::TILE_BYTES);
  uint64_t* qdo_full = bars;               // [1]
  uint64_t* k_full = bars + 1;             // [K_STAGES]  K and V blocks have rings of their own: a V block is free as
  uint64_t* k_empty = bars + 4;            // [K_STAGES]  soon as dP is computed, a K block only after the third product
  uint64_t* v_full = bars + 7;             // [V_STAGES]
  uint64_t* v_empty = bars + 9;            // [V_STAGES]
  uint64_t* sdp_full = bars + 11;          // [2]  S and dP of a block are complete
  uint64_t* sdp_empty = bars + 13;         // [2]  the element-wise warps have read them
  uint64_t* ds_full = bars + 15;           // [2]  dS tile written to shared memory
  uint64_t* ds_empty = bars + 17;          // [2]  the third product has read it
  uint64_t* dq_done = bars + 19;           // [1]  all products complete (the accumulator is final)
  uint32_t* tmem_base_slot = (uint32_t*)(bars + 20);
  volatile int* abort_flag = (volatile int*)(tmem_base_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_qblocks = (p.S + BLOCK_Q - 1) / BLOCK_Q;
  // grid: x = head, y = work item (query block and part of its keys; the blocks with the most keys come first), z = batch
  const int h = blockIdx.x, b = blockIdx.z;
  int qb = n_qblocks - 1, part = (int)blockIdx.y, first_slot = 0, n_kv_all = 0, n_parts = 1;
  for (;; --qb) {
    n_kv_all = attn_kv_blocks(qb, p.S, p.causal, BKV);
    n_parts = attn_chunks(n_kv_all, p.chunk);
    if (part < n_parts || qb == 0) break;
    part -= n_parts;
    first_slot += n_parts;
  }
  const int q0 = qb * BLOCK_Q;
  const int j0 = (int)(((long long)part * n_kv_all) / n_parts);           // this CTA's key blocks: [j0, j0 + n_kv)
  const int n_kv = (int)(((long long)(part + 1) * n_kv_all) / n_parts) - j0;
  const int row0 = b * p.S;

  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1);
    for (int s = 0; s < K_STAGES; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
    }
    for (int s = 0; s < V_STAGES; ++s) {
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sdp_full[s], 1);
      mbar_init(&sdp_empty[s], NUM_EW_WARPS);
      mbar_init(&ds_full[s], NUM_EW_WARPS);
      mbar_init(&ds_empty[s], 1);
    }
    mbar_init(dq_done, 1);
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
  const uint32_t tmem_dq = tmem_base;                 // columns [0, D)
  const uint32_t tmem_s = tmem_base + D;              // two buffers of BKV columns
  const uint32_t tmem_dp = tmem_base + D + 2 * BKV;   // two buffers of BKV columns

  if (warp == 0) {
    // ------------------------------------------------ TMA producer ------------------------------------------------
    // lane 0 loads Q and dO and streams the K blocks, lane 1 streams the V blocks: each waits only on its own ring
    if (lane < 2) {
      const bool for_k = lane == 0;
      if (for_k) {
        mbar_expect_tx(qdo_full, 2 * L::Q_BYTES);
#pragma unroll
        for (int kb = 0; kb < D / 64; ++kb) {  // boxes {64 features, 128 rows}
          tma_load_2d(sQ + kb * (BLOCK_Q * 128), &map_q, qdo_full, p.q_col + h * D + kb * 64, row0 + q0);
          tma_load_2d(sDO + kb * (BLOCK_Q * 128), &map_do, qdo_full, h * D + kb * 64, row0 + q0);
        }
      }
      uint64_t* full = for_k ? k_full : v_full;
      uint64_t* empty = for_k ? k_empty : v_empty;
      const int stages = for_k ? K_STAGES : V_STAGES;
      bool ok = true;
      int issued = 0;
      for (int j = 0; j < n_kv && ok; ++j) {
        const int stage = j % stages;
        if (j >= stages) {
          ok = mbar_wait(&empty[stage], (uint32_t)(j / stages - 1) & 1u, abort_flag, p.err, ERR_KV_EMPTY_WAIT);
          if (!ok) break;
        }
        uint8_t* dst = for_k ? sK + stage * L::K_BYTES : sV + stage * L::V_BYTES;
        mbar_expect_tx(&full[stage], L::K_BYTES);
        const int k0 = row0 + (j0 + j) * BKV;
        const int col = (for_k ? p.k_col : p.v_col) + h * D;
#pragma unroll
        for (int kb = 0; kb < D / 64; ++kb)  // boxes {64 features, BKV rows}
          tma_load_2d(dst + kb * (BKV * 128), &map_kv, &full[stage], col + kb * 64, k0);
        issued = j + 1;
      }
      if (!ok || *abort_flag) {
        // loads in flight target this CTA's shared memory: give them a bounded time to land before the CTA ends
        if (for_k)
          for (uint32_t i = 0; i < SPIN_LIMIT && !mbar_try_wait(qdo_full, 0); ++i) {}
        for (int j = max(0, issued - stages); j < issued; ++j)
          for (uint32_t i = 0; i < SPIN_LIMIT && !mbar_try_wait(&full[j % stages], (uint32_t)(j / stages) & 1u); ++i) {}
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer --------------------------------------------------
    if (elect_one()) {
      const uint32_t fmt = p.is_fp16 ? 0u : 1u;
      // S = Q K^T and dP = dO V^T: both operands K-major, N = BKV.   dQ += dS K: dS K-major, K MN-major (bit 16), N = D.
      const uint32_t idesc_s = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(BKV >> 3) << 17) |
                               ((uint32_t)(BLOCK_Q >> 4) << 24);
      const uint32_t idesc_dq = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) | ((uint32_t)(D >> 3) << 17) |
                                ((uint32_t)(BLOCK_Q >> 4) << 24);
      bool ok = mbar_wait(qdo_full, 0, abort_flag, p.err, ERR_QDO_WAIT);
      auto issue_scores = [&](int j) -> bool {
        const int ks = j % K_STAGES, vs = j % V_STAGES, sb = j & 1;
        if (!mbar_wait(&k_full[ks], (uint32_t)(j / K_STAGES) & 1u, abort_flag, p.err, ERR_KV_FULL_WAIT)) return false;
        if (!mbar_wait(&v_full[vs], (uint32_t)(j / V_STAGES) & 1u, abort_flag, p.err, ERR_KV_FULL_WAIT)) return false;
        if (j >= 2 && !mbar_wait(&sdp_empty[sb], (uint32_t)(j / 2 - 1) & 1u, abort_flag, p.err, ERR_SDP_EMPTY_WAIT))
          return false;
        tcgen05_fence_after();
        const uint32_t q_addr = smem_u32(sQ), do_addr = smem_u32(sDO);
        const uint32_t k_addr = smem_u32(sK + ks * L::K_BYTES);
        const uint32_t v_addr = smem_u32(sV + vs * L::V_BYTES);
#pragma unroll
        for (int kb = 0; kb < D / 64; ++kb)
#pragma unroll
          for (int k = 0; k < 64 / UMMA_K; ++k) {
            const uint64_t da = make_smem_desc_sw128(q_addr + kb * (BLOCK_Q * 128) + k * (UMMA_K * 2), 16);
            const uint64_t db = make_smem_desc_sw128(k_addr + kb * (BKV * 128) + k * (UMMA_K * 2), 16);
            tcgen05_mma_f16(tmem_s + sb * BKV, da, db, idesc_s, (kb | k) ? 1u : 0u);
          }
#pragma unroll
        for (int kb = 0; kb < D / 64; ++kb)
#pragma unroll
          for (int k = 0; k < 64 / UMMA_K; ++k) {
            const uint64_t da = make_smem_desc_sw128(do_addr + kb * (BLOCK_Q * 128) + k * (UMMA_K * 2), 16);
            const uint64_t db = make_smem_desc_sw128(v_addr + kb * (BKV * 128) + k * (UMMA_K * 2), 16);
            tcgen05_mma_f16(tmem_dp + sb * BKV, da, db, idesc_s, (kb | k) ? 1u : 0u);
          }
        tcgen05_commit(&v_empty[vs]);  // the V block is free once dP is computed
        tcgen05_commit(&sdp_full[sb]);
        return true;
      };
      if (ok && n_kv > 0) ok = issue_scores(0);
      for (int j = 0; j < n_kv && ok; ++j) {
        XL_ATTN_BWD_STAMP(0, j, 0);
        if (j + 1 < n_kv) {
          ok = issue_scores(j + 1);
          if (!ok) break;
        }
        XL_ATTN_BWD_STAMP(0, j, 1);
        const int db_i = j & 1;
        ok = mbar_wait(&ds_full[db_i], (uint32_t)(j / 2) & 1u, abort_flag, p.err, ERR_DS_FULL_WAIT);
        if (!ok) break;
        XL_ATTN_BWD_STAMP(0, j, 2);
        tcgen05_fence_after();
        const int ks = j % K_STAGES;
        const uint32_t ds_addr = smem_u32(sDS + db_i * L::DS_BYTES);
        const uint32_t k_addr = smem_u32(sK + ks * L::K_BYTES);
#pragma unroll
        for (int k = 0; k < BKV / UMMA_K; ++k) {
          // dS: chunk column c (8 keys) starts at c * 2048 bytes; one product step spans two of them
          const uint64_t da = make_smem_desc_noswizzle(ds_addr + k * 2 * 2048, 2048, 128);
          // K_j as the MN-major operand: feature blocks (BKV rows x 128 B) are BKV * 128 bytes apart, 16 keys = 2048 bytes
          const uint64_t dbk = make_smem_desc_sw128(k_addr + k * (UMMA_K * 128), BKV * 128);
          tcgen05_mma_f16(tmem_dq, da, dbk, idesc_dq, (j | k) ? 1u : 0u);
        }
        tcgen05_commit(&k_empty[ks]);       // the K block is free once the third product has read it
        tcgen05_commit(&ds_empty[db_i]);    // and the dS buffer
        if (j == n_kv - 1) tcgen05_commit(dq_done);
        XL_ATTN_BWD_STAMP(0, j, 3);
      }
    }
  } else {
    // ------------------------------------------------ element-wise ------------------------------------------------
    const int qtr = warp & 3;            // TMEM lane quarter this warp may access
    const int r = qtr * 32 + lane;       // query row inside the block
    const int qrow = q0 + r;             // query position inside the sequence
    const bool row_ok = qrow < p.S;
    const uint32_t lane_base = (uint32_t)(qtr * 32) << 16;
    const float c = p.scale * 1.4426950408889634f;  // scores are exponentiated in base 2
    const bool is_fp16 = p.is_fp16 != 0;
    // per-row constants: log-sum-exp (base 2) and delta = dO . O
    float lse2 = 0.f, delta = 0.f;
    if (row_ok) lse2 = p.lse[((long long)b * p.H + h) * p.S + qrow] * 1.4426950408889634f;
    if (row_ok) delta = p.delta[((long long)b * p.H + h) * p.S + qrow];
    const long long mat = ((long long)b * p.H + h) * p.S * (long long)p.S;  // start of this (batch, head)'s S x S matrices
    uint16_t* prow = (uint16_t*)p.P + mat + (long long)qrow * p.S;
    uint16_t* dsrow = (uint16_t*)p.dS + mat + (long long)qrow * p.S;
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      const int sb = j & 1;
      if (warp == 2 && lane == 0) XL_ATTN_BWD_STAMP(1, j, 0);
      ok = __all_sync(0xffffffffu, mbar_wait(&sdp_full[sb], (uint32_t)(j / 2) & 1u, abort_flag, p.err, ERR_SDP_FULL_WAIT));
      if (!ok) break;
      if (warp == 2 && lane == 0) XL_ATTN_BWD_STAMP(1, j, 1);
      tcgen05_fence_after();
      float s[BKV], dp[BKV];
#pragma unroll
      for (int ch = 0; ch < BKV / 32; ++ch) {
        uint32_t raw[32];
        tmem_ld_32x32b_x32(tmem_s + lane_base + sb * BKV + ch * 32, raw);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) s[ch * 32 + i] = __uint_as_float(raw[i]);
        tmem_ld_32x32b_x32(tmem_dp + lane_base + sb * BKV + ch * 32, raw);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) dp[ch * 32 + i] = __uint_as_float(raw[i]);
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sdp_empty[sb]);  // both buffers may be overwritten
      if (warp == 2 && lane == 0) XL_ATTN_BWD_STAMP(1, j, 2);
      const int col0 = (j0 + j) * BKV;
      const int limit = p.causal ? min(qrow, p.S - 1) : p.S - 1;  // last key this row may attend
#pragma unroll
      for (int i = 0; i < BKV; ++i) {
        const float pr = (col0 + i <= limit && row_ok) ? fast_exp2(fmaf(s[i], c, -lse2)) : 0.f;
        s[i] = pr;
        dp[i] = pr * (dp[i] - delta) * p.scale;
      }
      if (warp == 2 && lane == 0) XL_ATTN_BWD_STAMP(1, j, 3);
      // dS_j -> shared memory for the third product: 16-bit, no swizzle, [chunk column][row group][8 rows x 16 B]
      const int db_i = j & 1;
      if (j >= 2) {
        ok = __all_sync(0xffffffffu, mbar_wait(&ds_empty[db_i], (uint32_t)(j / 2 - 1) & 1u, abort_flag, p.err,
                                                ERR_DS_EMPTY_WAIT));
        if (!ok) break;
      }
      if (warp == 2 && lane == 0) XL_ATTN_BWD_STAMP(1, j, 5);
      uint8_t* ds_tile = sDS + db_i * L::DS_BYTES;
#pragma unroll
      for (int ch = 0; ch < BKV / 8; ++ch) {
        const uint4 o = pack8_16bit(dp + ch * 8, is_fp16);
        *(uint4*)(ds_tile + ch * 2048 + (r >> 3) * 128 + (r & 7) * 16) = o;
      }
      fence_proxy_async_smem();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ds_full[db_i]);
      if (warp == 2 && lane == 0) XL_ATTN_BWD_STAMP(1, j, 6);
      // P and dS rows to global memory (16-bit): 2 * BKV bytes each, contiguous per thread, 32 bytes per store where the
      // rows are 32-byte aligned
      if (row_ok) {
        const bool wide = (p.S % 16) == 0 && ((((uintptr_t)p.P) | ((uintptr_t)p.dS)) & 31) == 0;
#pragma unroll
        for (int ch = 0; ch < BKV / 8; ch += 2) {
          const uint4 p0 = pack8_16bit(s + ch * 8, is_fp16), p1 = pack8_16bit(s + ch * 8 + 8, is_fp16);
          const uint4 d0 = pack8_16bit(dp + ch * 8, is_fp16), d1 = pack8_16bit(dp + ch * 8 + 8, is_fp16);
          if (wide && col0 + ch * 8 + 16 <= p.S) {
            st_global_v8(prow + col0 + ch * 8, p0, p1);
            st_global_v8(dsrow + col0 + ch * 8, d0, d1);
          } else {
            const uint4 pv[2] = {p0, p1}, dv[2] = {d0, d1};
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              const int cc = col0 + (ch + half) * 8;
              const uint16_t* pe = (const uint16_t*)&pv[half];
              const uint16_t* de = (const uint16_t*)&dv[half];
              if (cc + 8 <= p.S) {
                *(uint4*)(prow + cc) = pv[half];
                *(uint4*)(dsrow + cc) = dv[half];
              } else {
                for (int e = 0; e < 8 && cc + e < p.S; ++e) {
                  prow[cc + e] = pe[e];
                  dsrow[cc + e] = de[e];
                }
              }
            }
          }
        }
      }
      if (warp == 2 && lane == 0) XL_ATTN_BWD_STAMP(1, j, 4);
    }
    // ---- epilogue: dQ -> global memory (or this CTA's partial sum -> workspace, merged by the last warp to finish) --------
    if (ok && n_kv > 0) ok = __all_sync(0xffffffffu, mbar_wait(dq_done, 0, abort_flag, p.err, ERR_DQ_DONE_WAIT));
    if (ok && n_kv > 0) {
      tcgen05_fence_after();
      const bool split = n_parts > 1;
      const long long slot0 = (long long)(b * p.H + h) * p.items + first_slot;  // first partial of this query block
      uint16_t* qrow_out = (uint16_t*)p.dq + (long long)(row0 + qrow) * p.ld_dq + p.dq_col + h * D;
      float* prow_out = split ? p.part_dq + ((slot0 + part) * BLOCK_Q + r) * D : nullptr;
#pragma unroll 1
      for (int ch = 0; ch < D / 32; ++ch) {
        uint32_t raw[32];
        tmem_ld_32x32b_x32(tmem_dq + lane_base + ch * 32, raw);
        tmem_ld_wait();
        if (split) {
#pragma unroll
          for (int g = 0; g < 8; ++g)
            *(uint4*)(prow_out + ch * 32 + g * 4) = make_uint4(raw[g * 4], raw[g * 4 + 1], raw[g * 4 + 2], raw[g * 4 + 3]);
        } else if (row_ok) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(raw[g * 8 + e]);
            *(uint4*)(qrow_out + ch * 32 + g * 8) = pack8_16bit(v, is_fp16);
          }
        }
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

// delta = dO . O of every (batch, head, position): one warp per row, the lanes across the features.
template <int D>
__global__ void __launch_bounds__(256) attn_bwd_delta_kernel(const AttnBwdParams p) {
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (long long)p.B * p.H * p.S) return;
  const int s_pos = (int)(w % p.S);
  const int bh = (int)(w / p.S), b = bh / p.H, h = bh % p.H;
  constexpr int LANES = D / 8;  // lanes that hold 8 features each
  const bool is_fp16 = p.is_fp16 != 0;
  float part = 0.f;
  if (lane < LANES) {
    const uint16_t* orow = (const uint16_t*)p.out + (long long)(b * p.S + s_pos) * p.ldo + h * D + lane * 8;
    const uint16_t* grow = (const uint16_t*)p.dout + (long long)(b * p.S + s_pos) * p.ld_do + h * D + lane * 8;
    const uint4 ov = *(const uint4*)orow, gv = *(const uint4*)grow;
    const uint32_t* ow = (const uint32_t*)&ov;
    const uint32_t* gw = (const uint32_t*)&gv;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float o_lo, o_hi, g_lo, g_hi;
      if (is_fp16) {
        o_lo = __half2float(__ushort_as_half((uint16_t)(ow[e] & 0xffffu)));
        o_hi = __half2float(__ushort_as_half((uint16_t)(ow[e] >> 16)));
        g_lo = __half2float(__ushort_as_half((uint16_t)(gw[e] & 0xffffu)));
        g_hi = __half2float(__ushort_as_half((uint16_t)(gw[e] >> 16)));
      } else {
        o_lo = __uint_as_float(ow[e] << 16);
        o_hi = __uint_as_float(ow[e] & 0xffff0000u);
        g_lo = __uint_as_float(gw[e] << 16);
        g_hi = __uint_as_float(gw[e] & 0xffff0000u);
      }
      part = fmaf(o_lo, g_lo, part);
      part = fmaf(o_hi, g_hi, part);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
  if (lane == 0) p.delta[w] = part;
}

// Sum of the partial dQ of split query blocks: one warp per query row. Rows of query blocks that were not split were
// written by the main kernel already.
template <int D>
__global__ void __launch_bounds__(256) attn_bwd_dq_merge_kernel(const AttnBwdParams p, int bkv) {
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (long long)p.B * p.H * p.S) return;
  const int s_pos = (int)(w % p.S);
  const int bh = (int)(w / p.S), b = bh / p.H, h = bh % p.H;
  const int n_qblocks = (p.S + BLOCK_Q - 1) / BLOCK_Q, qb = s_pos / BLOCK_Q, row = s_pos % BLOCK_Q;
  const int n_parts = attn_chunks(attn_kv_blocks(qb, p.S, p.causal, bkv), p.chunk);
  if (n_parts == 1) return;
  int first_slot = 0;
  for (int q = n_qblocks - 1; q > qb; --q) first_slot += attn_chunks(attn_kv_blocks(q, p.S, p.causal, bkv), p.chunk);
  const long long slot0 = (long long)bh * p.items + first_slot;
  constexpr int EL = D / 32;  // features per lane
  float acc[EL];
#pragma unroll
  for (int e = 0; e < EL; ++e) acc[e] = 0.f;
  constexpr int UNROLL = 4;  // parts whose loads are in flight together
  for (int c0 = 0; c0 < n_parts; c0 += UNROLL) {
    float2 raw[UNROLL][EL / 2];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const bool on = c0 + u < n_parts;
      const float* src = p.part_dq + ((slot0 + (on ? c0 + u : 0)) * BLOCK_Q + row) * D + lane * EL;
#pragma unroll
      for (int e = 0; e < EL / 2; ++e) raw[u][e] = on ? *(const float2*)(src + 2 * e) : make_float2(0.f, 0.f);
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
#pragma unroll
      for (int e = 0; e < EL / 2; ++e) {
        acc[2 * e] += raw[u][e].x;
        acc[2 * e + 1] += raw[u][e].y;
      }
  }
  const bool is_fp16 = p.is_fp16 != 0;
  uint16_t* dst = (uint16_t*)p.dq + (long long)(b * p.S + s_pos) * p.ld_dq + p.dq_col + h * D + lane * EL;
#pragma unroll
  for (int e = 0; e < EL; e += 2) {
    uint32_t two;
    if (is_fp16) asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(two) : "f"(acc[e + 1]), "f"(acc[e]));
    else asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(two) : "f"(acc[e + 1]), "f"(acc[e]));
    *(uint32_t*)(dst + e) = two;
  }
}

// 2-D map over a row-major matrix (rows x cols, leading dimension ld elements), boxes of {64, box_rows}, 128-byte swizzle
int make_map(CUtensorMap* map, const void* ptr, int is_fp16, long long rows, long long cols, long long ld, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -2;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, is_fp16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)ptr, dims,
                  strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

template <int D, int BKV>
int launch(const void* qkv, long long rows, long long cols, long long ld, const AttnBwdParams& p, cudaStream_t s) {
  using L = BwdSmem<D, BKV>;
  CUtensorMap mq, mdo, mkv;
  int r = make_map(&mq, qkv, p.is_fp16, rows, cols, ld, BLOCK_Q);
  if (r) return r;
  r = make_map(&mdo, p.dout, p.is_fp16, rows, (long long)p.H * D, p.ld_do, BLOCK_Q);
  if (r) return r;
  r = make_map(&mkv, qkv, p.is_fp16, rows, cols, ld, BKV);
  if (r) return r;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_bwd_dq_tcgen05_kernel<D, BKV>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         L::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  AttnBwdParams q = p;
  q.items = attn_items(p.S, p.causal, BKV, p.chunk);
  if (q.items > 65535) return -1;
  dim3 grid(p.H, q.items, p.B);
  const long long row_warps = (long long)p.B * p.H * p.S;
  attn_bwd_delta_kernel<D><<<(unsigned int)((row_warps + 7) / 8), 256, 0, s>>>(q);
  attn_bwd_dq_tcgen05_kernel<D, BKV><<<grid, NUM_THREADS, L::TOTAL, s>>>(mq, mdo, mkv, q);
  if (p.chunk > 0) {
    const long long warps = (long long)p.B * p.H * p.S;
    attn_bwd_dq_merge_kernel<D><<<(unsigned int)((warps + 7) / 8), 256, 0, s>>>(q, BKV);
  }
  return (int)cudaGetLastError();
}

}  // namespace

// First pass of the attention backward over a packed projection matrix (see the top of this file).
//   qkv:  (B*S x cols) row-major 16-bit with leading dimension ld: the (rotated) q | k | v of the forward pass
//   out, dout: forward output and its gradient, (B*S x ldo / ld_do), head h in columns [h*D, (h+1)*D)
//   lse:  (B, H, S) fp32 from the forward pass
//   P, dS: (B*H, S, S) 16-bit outputs. Rows of a query block are written for all key columns below the end of that block
//          (zeros above the diagonal); columns beyond are left untouched (the causal GEMMs never read them).
//   dq:   (B*S x ld_dq) 16-bit output, head h in columns [dq_col + h*D, ...)
//   All column offsets and leading dimensions must be multiples of 8, pointers 16-byte aligned, S a multiple of 8.
//   chunk, part_dq: key-range splitting as planned by xl_attn_bwd_plan (chunk 0: none, the pointer may then be null).
//         part_dq holds B*H*items*128*D floats; a second kernel on the same stream adds them up into dq.
//   delta: B*H*S floats of scratch (dO . O of every row, computed by a first kernel of the launch)
//   trace: null, or 2 * 64 * 8 64-bit words that receive clock stamps of the first CTA's roles (tuning aid).
// Returns 0, a CUDA error code, or a negative value when the arguments are not supported by this kernel.
XL_API int xl_attn_bwd_dq_tcgen05(const void* qkv, long long ld, long long cols, const void* out, long long ldo,
                                  const void* dout, long long ld_do, const float* lse, void* P, void* dS, void* dq,
                                  long long ld_dq, int dq_col, int B, int S, int H, int D, int q_col, int k_col, int v_col,
                                  float scale, int causal, int is_fp16, int* err, int chunk, float* part_dq,
                                  float* delta, long long* trace, cudaStream_t s) {
  if (B <= 0 || S <= 0 || H <= 0 || B > 65535 || H > 65535 || (S % 8)) return -1;
  if ((((uintptr_t)qkv) & 15) || (((uintptr_t)out) & 15) || (((uintptr_t)dout) & 15) || (((uintptr_t)P) & 15) ||
      (((uintptr_t)dS) & 15) || (((uintptr_t)dq) & 15))
    return -1;
  if ((ld % 8) || (ldo % 8) || (ld_do % 8) || (ld_dq % 8) || (dq_col % 8) || dq_col < 0) return -1;
  if ((q_col % 8) || (k_col % 8) || (v_col % 8) || q_col < 0 || k_col < 0 || v_col < 0) return -1;
  const long long need = (long long)H * D;
  if (q_col + need > cols || k_col + need > cols || v_col + need > cols || cols > ld || ldo < need || ld_do < need ||
      dq_col + need > ld_dq)
    return -1;
  if (!(scale > 0.f) || lse == nullptr) return -1;
  AttnBwdParams p;
  p.B = B; p.S = S; p.H = H; p.D = D;
  p.q_col = q_col; p.k_col = k_col; p.v_col = v_col;
  p.out = out; p.ldo = ldo; p.dout = dout; p.ld_do = ld_do; p.lse = lse; p.P = P; p.dS = dS; p.dq = dq; p.ld_dq = ld_dq;
  p.dq_col = dq_col; p.scale = scale; p.causal = causal ? 1 : 0; p.is_fp16 = is_fp16 ? 1 : 0; p.err = err;
  if (chunk < 0 || (chunk > 0 && !part_dq)) return -1;
  if (!delta) return -1;
  p.chunk = chunk; p.items = 0; p.part_dq = part_dq; p.delta = delta; p.trace = trace;
  const long long rows = (long long)B * S;
  if (D == 256) return launch<256, 32>(qkv, rows, cols, ld, p, s);
  if (D == 128) return launch<128, 64>(qkv, rows, cols, ld, p, s);
  if (D == 64) return launch<64, 64>(qkv, rows, cols, ld, p, s);
  return -1;
}

// Plans the key-range splitting of xl_attn_bwd_dq_tcgen05 for a shape on a device with `num_sms` SMs: returns the chunk
// (key blocks per CTA, 0 = no splitting) and stores the CTAs per head and batch entry in *items.
XL_API int xl_attn_bwd_plan(int B, int S, int H, int D, int causal, int num_sms, int* items) {
  if (D != 64 && D != 128 && D != 256) return -1;
  const int bkv = D == 256 ? 32 : 64;
  const int chunk = attn_plan_chunk(S, B * H, causal ? 1 : 0, bkv, num_sms > 0 ? num_sms : 148, 2.0, 4.0);
  if (items) *items = attn_items(S, causal ? 1 : 0, bkv, chunk);
  return chunk;
}
