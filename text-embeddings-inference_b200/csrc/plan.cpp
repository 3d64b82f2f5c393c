// Host-side planning for a packed batch: attention work items and the split of a batch over
// several GPU replicas.  Pure integer code, no CUDA calls, so it is testable without a GPU.
#include "kernels.h"
#include "plan.h"

#include <algorithm>
#include <cstdint>
#include <numeric>
#include <vector>

namespace tei {

int plan_attention(const int* cu_seqlens, int n_seqs, int causal, int* work_out,
                   int capacity_items, int window_left, int window_right) {
  struct Item {
    int start, len, q0, kv_begin;
    long long cost;
  };
  if (causal) window_right = 0;
  std::vector<Item> items;
  for (int s = 0; s < n_seqs; ++s) {
    const int start = cu_seqlens[s];
    const int len = cu_seqlens[s + 1] - start;
    for (int q0 = 0; q0 < len; q0 += 128) {
      const int kv_end = window_right >= 0 ? std::min(len, q0 + 128 + window_right) : len;
      const int kv_begin = window_left >= 0 ? std::max(0, q0 - window_left) / 64 * 64 : 0;
      items.push_back({start, len, q0, kv_begin, static_cast<long long>((kv_end - kv_begin + 63) / 64)});
    }
  }
  // Most expensive first: the hardware hands CTAs to SMs in index order, so this is the
  // longest-processing-time-first rule.  stable_sort keeps the result deterministic.
  std::stable_sort(items.begin(), items.end(),
                   [](const Item& a, const Item& b) { return a.cost > b.cost; });
  const int n = static_cast<int>(items.size());
  if (n > capacity_items || work_out == nullptr) return n;
  for (int i = 0; i < n; ++i) {
    work_out[i * 4 + 0] = items[i].start;
    work_out[i * 4 + 1] = items[i].len;
    work_out[i * 4 + 2] = items[i].q0;
    work_out[i * 4 + 3] = items[i].kv_begin;
  }
  return n;
}

int count_attention_items(const int* cu_seqlens, int n_seqs) {
  long long n = 0;
  for (int s = 0; s < n_seqs; ++s) n += (cu_seqlens[s + 1] - cu_seqlens[s] + 127) / 128;
  return static_cast<int>(n);
}

void plan_shards(const uint32_t* cu_seqlens, int n_seqs, int n_shards, double linear_cost,
                 double quadratic_cost, int* shard_of_seq) {
  // Greedy longest-first assignment to the least loaded shard.  The cost of a sequence of
  // length L is linear_cost * L (dense layers) + quadratic_cost * L^2 (attention).
  std::vector<int> order(n_seqs);
  std::iota(order.begin(), order.end(), 0);
  std::vector<double> cost(n_seqs);
  for (int s = 0; s < n_seqs; ++s) {
    const double len = static_cast<double>(cu_seqlens[s + 1] - cu_seqlens[s]);
    cost[s] = linear_cost * len + quadratic_cost * len * len;
  }
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return cost[a] > cost[b]; });
  std::vector<double> load(std::max(n_shards, 1), 0.0);
  for (int idx : order) {
    int best = 0;
    for (int d = 1; d < n_shards; ++d) {
      if (load[d] < load[best]) best = d;
    }
    shard_of_seq[idx] = best;
    load[best] += cost[idx];
  }
}

}  // namespace tei
