// Host-side batch planning helpers (no CUDA).
#pragma once
#include <cstdint>

namespace tei {

// Number of (sequence, 128-row query tile) attention work items of a packed batch.
int count_attention_items(const int* cu_seqlens, int n_seqs);

// Assigns every sequence of a packed batch to one of n_shards replicas, balancing
// linear_cost * L + quadratic_cost * L^2 with the longest-first greedy rule.
// shard_of_seq[s] receives the shard of sequence s.
void plan_shards(const uint32_t* cu_seqlens, int n_seqs, int n_shards, double linear_cost,
                 double quadratic_cost, int* shard_of_seq);

}  // namespace tei
