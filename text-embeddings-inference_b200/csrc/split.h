// Split of one packed batch over the replicas of a handle, and the way back: which sequence goes
// to which replica, the sub-batch each replica sees (token arrays gathered, cumulative lengths
// rebased, pooled / raw index lists renumbered) and where each result row lands in the caller's
// buffers.  Host-only code without CUDA calls: the replica that runs a shard is a parameter.
//
// The reference keeps one batch in flight per backend (backends/src/lib.rs:612-647,
// core/src/infer.rs:547-625), so behind an unchanged router several GPUs can only share work
// inside one embed / predict call; sequences of a packed batch are independent
// (backends/core/src/lib.rs:9-17), which is what makes the split legal.
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

#include "model.h"

namespace tei {

// A sub-batch for one replica plus where its rows go in the caller's buffers.
struct Shard {
  // set by assign_shards (caller thread; sequences only, no token is touched)
  std::vector<size_t> seqs;             // original batch positions, in shard order
  std::vector<uint32_t> pooled_idx, raw_idx;  // shard-local positions of the pooled / raw requests
  std::vector<size_t> pooled_dst_row;   // caller's pooled row of each pooled entry of the shard
  std::vector<size_t> raw_dst_row;      // caller's first raw row of each raw entry
  std::vector<size_t> raw_len;
  // set by gather_shard_tokens (the replica's own thread)
  std::vector<uint32_t> ids, types, pos, cu;
  uint32_t max_length = 0;
  // results of the shard before they are scattered
  std::vector<float> pooled, raw, scores;
  int err_kind = 0;
  std::string err_msg;

  void clear();
  HostBatch view() const;
};

// Plans the split (plan_shards: longest-first greedy on linear_cost * L + quadratic_cost * L^2)
// and fills the sequence-level fields of `shards` (resized to n_shards; vectors keep their
// capacity from call to call).
void assign_shards(const HostBatch& b, bool predict, int n_shards, double linear_cost,
                   double quadratic_cost, std::vector<Shard>& shards);
// Copies the shard's tokens out of the caller's arrays and rebases the cumulative lengths.
void gather_shard_tokens(const HostBatch& b, Shard& sh);
// Sizes the shard's result buffers: D floats per pooled row, DR per raw row, C per score row.
void size_shard_results(Shard& sh, bool predict, size_t D, size_t DR, size_t C);
// Copies the shard's result rows to their places in the caller's buffers.  Shards own disjoint
// rows, so the replicas' threads may scatter at the same time.
void scatter_shard(const Shard& sh, bool predict, size_t D, size_t DR, size_t C, float* pooled_out,
                   float* raw_out, float* scores_out);

}  // namespace tei
