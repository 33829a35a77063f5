// Causal softmax attention forward in one kernel on the 5th-generation tensor cores (tcgen05) for sm_100a.
//
//   O = softmax(scale * Q K^T + causal mask) V        per (batch, head); Q, K, V: (S x D) 16-bit, D in {64, 128, 256}
//
// Q, K and V are column windows of one packed row-major matrix (rows = batch * S tokens), as the fused qkv projection
// leaves them; O is a column window of the (tokens x heads*D) output matrix. The S x S score matrix never leaves the
// chip: one CTA owns 128 query rows and walks the key / value rows in blocks of BKV.
//
//   warp 0      TMA producer : Q tile once, then K blocks and V blocks into two 2-stage shared-memory rings (a K block is
//                              released as soon as its scores are computed, so the next K load overlaps the softmax)
//   warp 1      MMA issuer   : S_j = Q K_j^T into one of two TMEM score buffers, then O += P_j V_j into the TMEM output
//                              accumulator (S_{j+1} is issued before P_j is awaited, so it overlaps the softmax of block j)
//   warps 2..5  softmax      : one thread per query row. tcgen05.ld the score row, running max / sum (base-2 exponent),
//                              rescale the output accumulator in TMEM when the running max moved (tcgen05.ld / st),
//                              write P_j as a 128-byte-swizzled 16-bit tile to shared memory for the second MMA,
//                              finally O / l to global memory and the log-sum-exp of every row.
//
// TMEM columns: [0, D) output accumulator, [D, D + 2*BKV) two score buffers; 512 columns are allocated, one CTA per SM.
// Every wait on an mbarrier is bounded: when a wait gives up the kernel records a code in `*err`, raises a CTA-wide abort
// flag, all roles leave their loops, TMEM is released and the kernel returns normally.
#include "tcgen05.cuh"
#include "attention_split.cuh"

namespace {

constexpr int BLOCK_Q = 128;
constexpr int UMMA_K = 16;
constexpr int KV_STAGES = 2;
constexpr int NUM_SOFTMAX_WARPS = 4;
constexpr int NUM_THREADS = 64 + 32 * NUM_SOFTMAX_WARPS;
constexpr uint32_t SPIN_LIMIT = xl_tc::MBAR_SPIN_LIMIT;  // also bounds the producer's drain after an abort
constexpr uint32_t TMEM_COLS = 512;

enum { ERR_Q_WAIT = 11, ERR_KV_FULL_WAIT = 12, ERR_KV_EMPTY_WAIT = 13, ERR_S_FULL_WAIT = 14, ERR_S_EMPTY_WAIT = 15,
       ERR_P_FULL_WAIT = 16, ERR_PV_DONE_WAIT = 17 };

struct AttnParams {
  int B, S, H, D;
  int q_col, k_col, v_col;  // first column of head 0 of Q / K / V in the packed matrix
  void* out;                // (B*S x ldo) 16-bit; head h occupies columns [h*D, (h+1)*D)
  long long ldo;
  float* lse;               // (B, H, S) fp32: log-sum-exp of the scaled scores of every row (natural log)
  float scale;
  int causal;
  int is_fp16;
  int* err;
  long long* trace;  // optional (tuning): clock64 stamps of CTA (0, 0, 0): [role 0 MMA thread | role 1 softmax warp][block][8]
  // Key-range splitting (chunk > 0): a query block's key blocks are divided evenly over ceil(n / chunk) CTAs. Each writes
  // its normalised partial output and log-sum-exp to the workspace; a second kernel merges the partials of every row.
  int chunk;
  int items;               // CTAs per head and batch entry (grid y)
  uint16_t* part_o;        // [B*H*items][128][D] 16-bit
  float* part_lse;         // [B*H*items][128]
};


using namespace xl_tc;
using namespace xl_attn_split;

#define XL_ATTN_STAMP(role, j, point)                                                                  \
  do {                                                                                                 \
    if (p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (j) < 64)       \
      p.trace[((role) * 64 + (j)) * 8 + (point)] = clock64();                                          \
  } while (0)

template <int D, int BKV>
struct AttnSmem {
  static constexpr int Q_BYTES = BLOCK_Q * D * 2;       // D/64 k-blocks of (128 rows x 128 B)
  static constexpr int K_BYTES = BKV * D * 2;           // D/64 k-blocks of (BKV rows x 128 B)
  static constexpr int V_BYTES = BKV * D * 2;           // BKV/64 k-blocks of D/64 boxes of (64 rows x 128 B)
  static constexpr int P_BYTES = BLOCK_Q * BKV * 2;     // BKV/64 k-blocks of (128 rows x 128 B)
  static constexpr int STAGE_BYTES = K_BYTES + V_BYTES;
  static constexpr int TILE_BYTES = Q_BYTES + KV_STAGES * STAGE_BYTES + P_BYTES;
  static constexpr int NEEDED = TILE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
  // more than half of an SM's shared memory, so that two CTAs (each holding all 512 TMEM columns) never share an SM
  static constexpr int TOTAL = NEEDED > 120 * 1024 ? NEEDED : 120 * 1024;
};

template <int D, int BKV>
__global__ void __launch_bounds__(NUM_THREADS, 1)
    attn_fwd_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
  using L = AttnSmem<D, BKV>;
  static_assert(D % 64 == 0 && D <= 256 && BKV % 64 == 0 && D + 2 * BKV <= (int)TMEM_COLS, "unsupported tile");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;
  uint8_t* sKV = smem + L::Q_BYTES;
  uint8_t* sP = sKV + KV_STAGES * L::STAGE_BYTES;
  uint64_t* bars = (uint64_t*)(smem + L::TILE_BYTES);
  uint64_t* q_full = bars;                 // [1]
  uint64_t* k_full = bars + 1;             // [KV_STAGES]  K and V blocks have rings of their own: a K block is free as
  uint64_t* k_empty = bars + 3;            // [KV_STAGES]  soon as its scores are computed, long before the V block of
  uint64_t* v_full = bars + 5;             // [KV_STAGES]  the same keys, so the next K load overlaps the softmax
  uint64_t* v_empty = bars + 7;            // [KV_STAGES]
  uint64_t* s_full = bars + 9;             // [2]
  uint64_t* s_empty = bars + 11;           // [2]
  uint64_t* p_full = bars + 13;            // [1]
  uint64_t* pv_done = bars + 14;           // [1]
  uint32_t* tmem_base_slot = (uint32_t*)(bars + 15);
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
  const int row0 = b * p.S;  // first token row of this batch entry in the packed matrix

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&s_empty[s], NUM_SOFTMAX_WARPS);
    }
    mbar_init(p_full, NUM_SOFTMAX_WARPS);
    mbar_init(pv_done, 1);
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
  const uint32_t tmem_o = tmem_base;          // columns [0, D)
  const uint32_t tmem_s = tmem_base + D;      // two buffers of BKV columns

  if (warp == 0) {
    // ------------------------------------------------ TMA producer ------------------------------------------------
    // lane 0 loads Q and streams the K blocks, lane 1 streams the V blocks: each waits only on its own ring
    if (lane < 2) {
      const bool for_k = lane == 0;
      if (for_k) {
        mbar_expect_tx(q_full, L::Q_BYTES);
#pragma unroll
        for (int kb = 0; kb < D / 64; ++kb)  // boxes {64 features, 128 rows}
          tma_load_2d(sQ + kb * (BLOCK_Q * 128), &map_q, q_full, p.q_col + h * D + kb * 64, row0 + q0);
      }
      uint64_t* full = for_k ? k_full : v_full;
      uint64_t* empty = for_k ? k_empty : v_empty;
      bool ok = true;
      int issued = 0;
      for (int j = 0; j < n_kv && ok; ++j) {
        const int stage = j % KV_STAGES;
        if (j >= KV_STAGES) {
          ok = mbar_wait(&empty[stage], (uint32_t)(j / KV_STAGES - 1) & 1u, abort_flag, p.err, ERR_KV_EMPTY_WAIT);
          if (!ok) break;
        }
        uint8_t* sK = sKV + stage * L::STAGE_BYTES;
        uint8_t* sV = sK + L::K_BYTES;
        const int k0 = row0 + (j0 + j) * BKV;
        if (for_k) {
          mbar_expect_tx(&full[stage], L::K_BYTES);
#pragma unroll
          for (int kb = 0; kb < D / 64; ++kb)  // boxes {64 features, BKV rows}
            tma_load_2d(sK + kb * (BKV * 128), &map_k, &full[stage], p.k_col + h * D + kb * 64, k0);
        } else {
          mbar_expect_tx(&full[stage], L::V_BYTES);
#pragma unroll
          for (int kk = 0; kk < BKV / 64; ++kk)
#pragma unroll
            for (int jn = 0; jn < D / 64; ++jn)  // boxes {64 features, 64 rows}
              tma_load_2d(sV + (kk * (D / 64) + jn) * 8192, &map_v, &full[stage], p.v_col + h * D + jn * 64,
                          k0 + kk * 64);
        }
        issued = j + 1;
      }
      if (!ok || *abort_flag) {
        // loads in flight target this CTA's shared memory: give them a bounded time to land before the CTA ends
        if (for_k)
          for (uint32_t i = 0; i < SPIN_LIMIT && !mbar_try_wait(q_full, 0); ++i) {}
        for (int j = max(0, issued - KV_STAGES); j < issued; ++j)
          for (uint32_t i = 0; i < SPIN_LIMIT && !mbar_try_wait(&full[j % KV_STAGES], (uint32_t)(j / KV_STAGES) & 1u); ++i) {}
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer --------------------------------------------------
    if (elect_one()) {
      const uint32_t fmt = p.is_fp16 ? 0u : 1u;
      // S = Q K^T: both operands K-major, N = BKV.   O += P V: P K-major, V MN-major (bit 16), N = D.
      const uint32_t idesc_s = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(BKV >> 3) << 17) |
                               ((uint32_t)(BLOCK_Q >> 4) << 24);
      const uint32_t idesc_o = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) | ((uint32_t)(D >> 3) << 17) |
                               ((uint32_t)(BLOCK_Q >> 4) << 24);
      bool ok = mbar_wait(q_full, 0, abort_flag, p.err, ERR_Q_WAIT);
      auto issue_scores = [&](int j) -> bool {
        const int stage = j % KV_STAGES, sb = j & 1;
        if (!mbar_wait(&k_full[stage], (uint32_t)(j / KV_STAGES) & 1u, abort_flag, p.err, ERR_KV_FULL_WAIT)) return false;
        if (j >= 2 && !mbar_wait(&s_empty[sb], (uint32_t)(j / 2 - 1) & 1u, abort_flag, p.err, ERR_S_EMPTY_WAIT))
          return false;
        tcgen05_fence_after();
        const uint32_t q_addr = smem_u32(sQ);
        const uint32_t k_addr = smem_u32(sKV + stage * L::STAGE_BYTES);
#pragma unroll
        for (int kb = 0; kb < D / 64; ++kb)
#pragma unroll
          for (int k = 0; k < 64 / UMMA_K; ++k) {
            const uint64_t da = make_smem_desc(q_addr + kb * (BLOCK_Q * 128) + k * (UMMA_K * 2), 16);
            const uint64_t db = make_smem_desc(k_addr + kb * (BKV * 128) + k * (UMMA_K * 2), 16);
            tcgen05_mma_f16(tmem_s + sb * BKV, da, db, idesc_s, (kb | k) ? 1u : 0u);
          }
        tcgen05_commit(&k_empty[stage]);  // the K block is free once its scores are computed
        tcgen05_commit(&s_full[sb]);
        return true;
      };
      if (ok && n_kv > 0) ok = issue_scores(0);
      for (int j = 0; j < n_kv && ok; ++j) {
        XL_ATTN_STAMP(0, j, 0);
        if (j + 1 < n_kv) {
          ok = issue_scores(j + 1);
          if (!ok) break;
        }
        XL_ATTN_STAMP(0, j, 1);
        const int stage = j % KV_STAGES;
        ok = mbar_wait(&v_full[stage], (uint32_t)(j / KV_STAGES) & 1u, abort_flag, p.err, ERR_KV_FULL_WAIT);
        if (!ok) break;
        XL_ATTN_STAMP(0, j, 2);
        ok = mbar_wait(p_full, (uint32_t)j & 1u, abort_flag, p.err, ERR_P_FULL_WAIT);
        if (!ok) break;
        XL_ATTN_STAMP(0, j, 3);
        tcgen05_fence_after();
        const uint32_t p_addr = smem_u32(sP);
        const uint32_t v_addr = smem_u32(sKV + stage * L::STAGE_BYTES + L::K_BYTES);
#pragma unroll
        for (int kk = 0; kk < BKV / 64; ++kk)
#pragma unroll
          for (int k = 0; k < 64 / UMMA_K; ++k) {
            const uint64_t da = make_smem_desc(p_addr + kk * (BLOCK_Q * 128) + k * (UMMA_K * 2), 16);
            const uint64_t db = make_smem_desc(v_addr + kk * (D / 64) * 8192 + k * (UMMA_K * 128), 8192);
            tcgen05_mma_f16(tmem_o, da, db, idesc_o, (j | kk | k) ? 1u : 0u);
          }
        tcgen05_commit(&v_empty[stage]);   // the V block is free once these MMAs have read it
        tcgen05_commit(pv_done);           // output accumulator and the P tile are free again
        XL_ATTN_STAMP(0, j, 4);
      }
    }
  } else {
    // ------------------------------------------------ softmax -----------------------------------------------------
    const int qtr = warp & 3;  // TMEM lane quarter this warp may access
    const int r = qtr * 32 + lane;  // query row inside the block
    const int qrow = q0 + r;        // query position inside the sequence
    const uint32_t lane_base = (uint32_t)(qtr * 32) << 16;
    const float c = p.scale * 1.4426950408889634f;  // scores are exponentiated in base 2
    const bool is_fp16 = p.is_fp16 != 0;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      const int sb = j & 1;
      if (warp == 2 && lane == 0) XL_ATTN_STAMP(1, j, 0);
      ok = __all_sync(0xffffffffu, mbar_wait(&s_full[sb], (uint32_t)(j / 2) & 1u, abort_flag, p.err, ERR_S_FULL_WAIT));
      if (!ok) break;
      if (warp == 2 && lane == 0) XL_ATTN_STAMP(1, j, 1);
      tcgen05_fence_after();
      float s[BKV];
#pragma unroll
      for (int ch = 0; ch < BKV / 32; ++ch) {
        uint32_t raw[32];
        tmem_ld_32x32b_x32(tmem_s + lane_base + sb * BKV + ch * 32, raw);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) s[ch * 32 + i] = __uint_as_float(raw[i]);
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[sb]);  // the score buffer may be overwritten
      if (warp == 2 && lane == 0) XL_ATTN_STAMP(1, j, 2);
      const int col0 = (j0 + j) * BKV;
      const int limit = p.causal ? min(qrow, p.S - 1) : p.S - 1;  // last key this row may attend
      float m_blk = -INFINITY;
      if (col0 + BKV - 1 > limit) {
#pragma unroll
        for (int i = 0; i < BKV; ++i)
          if (col0 + i > limit) s[i] = -INFINITY;
      }
#pragma unroll
      for (int i = 0; i < BKV; ++i) m_blk = fmaxf(m_blk, s[i]);
      // Lazy rescaling: `m` is the reference maximum of the exponent, not the exact running maximum. It only moves (and
      // the sum and the output accumulator are only rescaled) when the block's maximum exceeds it by more than
      // RESCALE_LOG2 in the base-2 exponent, so probabilities stay below 2^RESCALE_LOG2 (exact in fp32 sums, and with the
      // usual relative precision as 16-bit operands of the second product) and the TMEM round trip of the accumulator,
      // which would otherwise run in almost every block (some row of a warp finds a new maximum), becomes rare.
      constexpr float RESCALE_LOG2 = 8.f;
      const bool move = m_blk > -INFINITY && (m == -INFINITY || (m_blk - m) * c > RESCALE_LOG2);
      const float m_new = move ? m_blk : m;
      const float m_use = m_new == -INFINITY ? 0.f : m_new;  // a row with no admissible key yet keeps p = 0
      const float alpha = (move && m != -INFINITY) ? fast_exp2((m - m_use) * c) : 1.f;
      float sum = 0.f;
      const float mc = m_use * c;
#pragma unroll
      for (int i = 0; i < BKV; ++i) {
        s[i] = fast_exp2(fmaf(s[i], c, -mc));
        sum += s[i];
      }
      l = l * alpha + sum;
      m = m_new;
      if (warp == 2 && lane == 0) XL_ATTN_STAMP(1, j, 3);
      if (j > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(pv_done, (uint32_t)(j - 1) & 1u, abort_flag, p.err, ERR_PV_DONE_WAIT));
        if (!ok) break;
        tcgen05_fence_after();
        if (__any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
          for (int ch = 0; ch < D / 32; ++ch) {
            uint32_t raw[32];
            tmem_ld_32x32b_x32(tmem_o + lane_base + ch * 32, raw);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) raw[i] = __float_as_uint(__uint_as_float(raw[i]) * alpha);
            tmem_st_32x32b_x32(tmem_o + lane_base + ch * 32, raw);
          }
          tmem_st_wait();
        }
      }
      if (warp == 2 && lane == 0) XL_ATTN_STAMP(1, j, 4);
      // P_j -> shared memory, 16-bit, 128-byte swizzle (16-byte chunk index xor row mod 8), one 64-key k-block per 16 KB
#pragma unroll
      for (int ch = 0; ch < BKV / 8; ++ch) {
        const uint4 o = pack8_16bit(s + ch * 8, is_fp16);
        *(uint4*)(sP + (ch >> 3) * (BLOCK_Q * 128) + r * 128 + (((ch & 7) ^ (r & 7)) << 4)) = o;
      }
      fence_proxy_async_smem();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
      if (warp == 2 && lane == 0) XL_ATTN_STAMP(1, j, 5);
    }
    // ---- epilogue: O / l -> global memory, log-sum-exp ---------------------------------------------------------------
    if (ok && n_kv > 0)
      ok = __all_sync(0xffffffffu, mbar_wait(pv_done, (uint32_t)(n_kv - 1) & 1u, abort_flag, p.err, ERR_PV_DONE_WAIT));
    if (ok && n_kv > 0) {
      tcgen05_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const bool split = n_parts > 1;
      const long long slot0 = (long long)(b * p.H + h) * p.items + first_slot;  // first partial of this query block
      const bool row_ok = split || qrow < p.S;  // partial rows past the end are written too (the workspace has room)
      uint16_t* orow = split ? p.part_o + ((slot0 + part) * BLOCK_Q + r) * D
                             : (uint16_t*)p.out + (long long)(row0 + qrow) * p.ldo + h * D;
#pragma unroll 1
      for (int ch = 0; ch < D / 32; ++ch) {
        uint32_t raw[32];
        tmem_ld_32x32b_x32(tmem_o + lane_base + ch * 32, raw);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(raw[g * 8 + e]) * inv;
            *(uint4*)(orow + ch * 32 + g * 8) = pack8_16bit(v, is_fp16);
          }
        }
      }
      const float lse_row = l > 0.f ? m * p.scale + logf(l) : -INFINITY;
      if (!split) {
        if (row_ok && p.lse) p.lse[((long long)b * p.H + h) * p.S + qrow] = lse_row;
      } else {
        p.part_lse[(slot0 + part) * BLOCK_Q + r] = lse_row;
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

// Merge of the partial results of split query blocks: one warp per query row. Rows of query blocks that were not split
// were written by the main kernel already.
template <int D>
__global__ void __launch_bounds__(256) attn_fwd_merge_kernel(const AttnParams p, int bkv) {
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
  const bool is_fp16 = p.is_fp16 != 0;
  // log-sum-exp over the parts (lane c holds part c; more than 32 parts are folded in by the loops)
  float lse_c = -INFINITY, mx = -INFINITY;
  for (int c0 = 0; c0 < n_parts; c0 += 32) {
    const float v = c0 + lane < n_parts ? p.part_lse[(slot0 + c0 + lane) * BLOCK_Q + row] : -INFINITY;
    mx = fmaxf(mx, v);
    if (c0 == 0) lse_c = v;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float den = 0.f;
  for (int c0 = 0; c0 < n_parts; c0 += 32) {
    const float v = c0 + lane < n_parts ? p.part_lse[(slot0 + c0 + lane) * BLOCK_Q + row] : -INFINITY;
    den += v > -INFINITY ? __expf(v - mx) : 0.f;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
  const float lse_all = den > 0.f ? mx + logf(den) : -INFINITY;
  constexpr int EL = D / 32;  // output features per lane
  float acc[EL];
#pragma unroll
  for (int e = 0; e < EL; ++e) acc[e] = 0.f;
  constexpr int UNROLL = 4;  // parts whose loads are in flight together
  for (int c0 = 0; c0 < n_parts; c0 += UNROLL) {
    uint32_t raw[UNROLL][EL / 2];
    float wgt[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int c = c0 + u;
      const bool on = c < n_parts;
      const uint16_t* src = p.part_o + ((slot0 + (on ? c : 0)) * BLOCK_Q + row) * D + lane * EL;
#pragma unroll
      for (int e = 0; e < EL / 2; ++e) raw[u][e] = on ? *(const uint32_t*)(src + 2 * e) : 0u;
      const float lc = c < 32 ? __shfl_sync(0xffffffffu, lse_c, c & 31) : (on ? p.part_lse[(slot0 + c) * BLOCK_Q + row] : -INFINITY);
      wgt[u] = (on && lc > -INFINITY) ? __expf(lc - lse_all) : 0.f;
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
#pragma unroll
      for (int e = 0; e < EL / 2; ++e) {
        const uint32_t two = raw[u][e];
        const float lo = is_fp16 ? __half2float(__ushort_as_half((uint16_t)(two & 0xffffu))) : __uint_as_float(two << 16);
        const float hi = is_fp16 ? __half2float(__ushort_as_half((uint16_t)(two >> 16))) : __uint_as_float(two & 0xffff0000u);
        acc[2 * e] = fmaf(wgt[u], lo, acc[2 * e]);
        acc[2 * e + 1] = fmaf(wgt[u], hi, acc[2 * e + 1]);
      }
  }
  uint16_t* dst = (uint16_t*)p.out + (long long)(b * p.S + s_pos) * p.ldo + h * D + lane * EL;
#pragma unroll
  for (int e = 0; e < EL; e += 2) {
    uint32_t two;
    if (is_fp16) asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(two) : "f"(acc[e + 1]), "f"(acc[e]));
    else asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(two) : "f"(acc[e + 1]), "f"(acc[e]));
    *(uint32_t*)(dst + e) = two;
  }
  if (lane == 0 && p.lse) p.lse[((long long)b * p.H + h) * p.S + s_pos] = lse_all;
}

// ---- host side -------------------------------------------------------------------------------------------------------
// 2-D map over the packed row-major matrix (rows x cols, leading dimension ld elements), boxes of {64, box_rows}
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
int launch(const void* qkv, long long rows, long long cols, long long ld, const AttnParams& p, cudaStream_t s) {
  using L = AttnSmem<D, BKV>;
  CUtensorMap mq, mk, mv;
  int r = make_map(&mq, qkv, p.is_fp16, rows, cols, ld, BLOCK_Q);
  if (r) return r;
  r = make_map(&mk, qkv, p.is_fp16, rows, cols, ld, BKV);
  if (r) return r;
  r = make_map(&mv, qkv, p.is_fp16, rows, cols, ld, 64);
  if (r) return r;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_tcgen05_kernel<D, BKV>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         L::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  AttnParams q = p;
  q.items = attn_items(p.S, p.causal, BKV, p.chunk);
  if (q.items > 65535) return -1;
  dim3 grid(p.H, q.items, p.B);
  attn_fwd_tcgen05_kernel<D, BKV><<<grid, NUM_THREADS, L::TOTAL, s>>>(mq, mk, mv, q);
  if (p.chunk > 0) {
    const long long warps = (long long)p.B * p.H * p.S;
    attn_fwd_merge_kernel<D><<<(unsigned int)((warps + 7) / 8), 256, 0, s>>>(q, BKV);
  }
  return (int)cudaGetLastError();
}

int bkv_of(int D) { return D == 256 ? 64 : 128; }

}  // namespace

// Causal (or full) softmax attention forward over a packed projection matrix.
//   qkv: (B*S x cols) row-major 16-bit matrix with leading dimension ld (elements); head h of Q / K / V occupies columns
//        [x_col + h*D, x_col + (h+1)*D) for x in {q, k, v}. All column offsets and ld must be multiples of 8.
//   out: (B*S x ldo) 16-bit, head h in columns [h*D, (h+1)*D); ldo a multiple of 8, out 16-byte aligned.
//   lse: (B, H, S) fp32, may be null.      D in {64, 128, 256}.
//   err: device int that receives a non-zero code if a bounded wait inside the kernel gave up (may be null).
//   trace: null, or 2 * 64 * 8 64-bit words that receive clock stamps of the first CTA's roles (tuning aid).
// Returns 0, a CUDA error code, or a negative value when the arguments are not supported by this kernel.
//   chunk, part_o, part_lse: key-range splitting as planned by xl_attn_fwd_plan (chunk 0: none, the pointers may then
//        be null). part_o holds B*H*items*128*D 16-bit values, part_lse B*H*items*128 floats; a second kernel on the
//        same stream merges them into `out` and `lse`.
XL_API int xl_attn_fwd_tcgen05(const void* qkv, long long ld, long long cols, void* out, long long ldo, float* lse, int B,
                               int S, int H, int D, int q_col, int k_col, int v_col, float scale, int causal,
                               int is_fp16, int* err, long long* trace, int chunk, void* part_o, float* part_lse,
                               cudaStream_t s) {
  if (B <= 0 || S <= 0 || H <= 0 || B > 65535 || H > 65535) return -1;
  if ((((uintptr_t)qkv) & 15) || (((uintptr_t)out) & 15) || (ld % 8) || (ldo % 8)) return -1;
  if ((q_col % 8) || (k_col % 8) || (v_col % 8) || q_col < 0 || k_col < 0 || v_col < 0) return -1;
  const long long need = (long long)H * D;
  if (q_col + need > cols || k_col + need > cols || v_col + need > cols || cols > ld || ldo < need) return -1;
  if (!(scale > 0.f)) return -1;
  AttnParams p;
  p.B = B; p.S = S; p.H = H; p.D = D;
  p.q_col = q_col; p.k_col = k_col; p.v_col = v_col;
  p.out = out; p.ldo = ldo; p.lse = lse; p.scale = scale; p.causal = causal ? 1 : 0; p.is_fp16 = is_fp16 ? 1 : 0;
  p.err = err;
  p.trace = trace;
  if (chunk < 0 || (chunk > 0 && (!part_o || !part_lse))) return -1;
  p.chunk = chunk; p.items = 0; p.part_o = (uint16_t*)part_o; p.part_lse = part_lse;
  const long long rows = (long long)B * S;
  if (D == 256) return launch<256, 64>(qkv, rows, cols, ld, p, s);
  if (D == 128) return launch<128, 128>(qkv, rows, cols, ld, p, s);
  if (D == 64) return launch<64, 128>(qkv, rows, cols, ld, p, s);
  return -1;
}

// Plans the key-range splitting of xl_attn_fwd_tcgen05 for a shape on a device with `num_sms` SMs: returns the chunk
// (key blocks per CTA, 0 = no splitting) and stores the CTAs per head and batch entry in *items.
XL_API int xl_attn_fwd_plan(int B, int S, int H, int D, int causal, int num_sms, int* items) {
  if (D != 64 && D != 128 && D != 256) return -1;
  const int bkv = bkv_of(D);
  const int chunk = attn_plan_chunk(S, B * H, causal ? 1 : 0, bkv, num_sms > 0 ? num_sms : 148, 1.5, 2.5);
  if (items) *items = attn_items(S, causal ? 1 : 0, bkv, chunk);
  return chunk;
}
