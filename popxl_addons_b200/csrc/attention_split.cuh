// Splitting the key range of a query block over several CTAs (attention forward and backward kernels): which key blocks
// a CTA gets, how many CTAs a launch has, and the planner that picks the number of key blocks per CTA for a shape.
// A query block of 128 rows attends `n` key blocks (all of them, or those up to its diagonal when causal); with
// `chunk > 0` they are divided evenly over ceil(n / chunk) CTAs, each of which produces a partial result.
#pragma once
#include <queue>
#include <vector>

namespace xl_attn_split {

constexpr int SPLIT_BLOCK_Q = 128;

// key blocks that query block qb attends, and the CTAs they are divided over
__host__ __device__ inline int attn_kv_blocks(int qb, int S, int causal, int bkv) {
  const int kv_end = causal ? (S < (qb + 1) * SPLIT_BLOCK_Q ? S : (qb + 1) * SPLIT_BLOCK_Q) : S;
  return (kv_end + bkv - 1) / bkv;
}
__host__ __device__ inline int attn_chunks(int n_kv, int chunk) { return chunk > 0 ? (n_kv + chunk - 1) / chunk : 1; }

// work items (CTAs per head and batch entry) of a launch
inline int attn_items(int S, int causal, int bkv, int chunk) {
  const int n_qblocks = (S + SPLIT_BLOCK_Q - 1) / SPLIT_BLOCK_Q;
  int items = 0;
  for (int qb = 0; qb < n_qblocks; ++qb) items += attn_chunks(attn_kv_blocks(qb, S, causal, bkv), chunk);
  return items;
}

// Time (in key-block iterations) until the last CTA ends when the launch's CTAs, in launch order, each go to the SM
// that frees up first. `fixed` / `fixed_split` is the cost of a CTA besides its key blocks (loading the query block,
// the epilogue, and for a split query block the pass over the partial results), in the same unit.
inline double attn_makespan(int S, int BH, int causal, int bkv, int chunk, int num_sms, double fixed, double fixed_split) {
  const int n_qblocks = (S + SPLIT_BLOCK_Q - 1) / SPLIT_BLOCK_Q;
  std::priority_queue<double, std::vector<double>, std::greater<double>> sms;
  for (int i = 0; i < num_sms; ++i) sms.push(0.0);
  double end = 0.0;
  for (int qb = n_qblocks - 1; qb >= 0; --qb) {
    const int n = attn_kv_blocks(qb, S, causal, bkv), parts = attn_chunks(n, chunk);
    for (int c = 0; c < parts; ++c) {
      const int len = (int)(((long long)(c + 1) * n) / parts) - (int)(((long long)c * n) / parts);
      const double cost = len + (parts > 1 ? fixed_split : fixed);
      for (int h = 0; h < BH; ++h) {
        const double t = sms.top() + cost;
        sms.pop();
        sms.push(t);
        end = t > end ? t : end;
      }
    }
  }
  return end;
}

// Key blocks per CTA that minimise the modelled time of the launch (0: every query block keeps all its keys).
inline int attn_plan_chunk(int S, int BH, int causal, int bkv, int num_sms, double fixed, double fixed_split) {
  const int n_qblocks = (S + SPLIT_BLOCK_Q - 1) / SPLIT_BLOCK_Q;
  if ((long long)BH * n_qblocks > 6LL * num_sms || n_qblocks * (SPLIT_BLOCK_Q / bkv) < 4) return 0;  // enough CTAs as it is
  const double whole = attn_makespan(S, BH, causal, bkv, 0, num_sms, fixed, fixed_split);
  double best = whole * 0.92;  // splitting has to pay for the extra pass over the partial results
  int best_chunk = 0;
  const int n_max = attn_kv_blocks(n_qblocks - 1, S, causal, bkv);
  for (int chunk = n_max - 1; chunk >= 2; --chunk) {
    if (attn_items(S, causal, bkv, chunk) > 65535) break;
    const double t = attn_makespan(S, BH, causal, bkv, chunk, num_sms, fixed, fixed_split);
    if (t < best) { best = t; best_chunk = chunk; }
  }
  return best_chunk;
}

}  // namespace xl_attn_split
