#include "split.h"

#include <algorithm>
#include <cstring>

#include "plan.h"

namespace tei {

void Shard::clear() {
  seqs.clear();
  pooled_idx.clear();
  raw_idx.clear();
  pooled_dst_row.clear();
  raw_dst_row.clear();
  raw_len.clear();
  ids.clear();
  types.clear();
  pos.clear();
  cu.clear();
  max_length = 0;
  err_kind = 0;
  err_msg.clear();
}

HostBatch Shard::view() const {
  HostBatch b;
  b.input_ids = ids.data();
  b.token_type_ids = types.data();
  b.position_ids = pos.data();
  b.n_tokens = ids.size();
  b.cu_seqlens = cu.data();
  b.n_seqs = seqs.size();
  b.max_length = max_length;
  b.pooled_indices = pooled_idx.data();
  b.n_pooled = pooled_idx.size();
  b.raw_indices = raw_idx.data();
  b.n_raw = raw_idx.size();
  return b;
}

void assign_shards(const HostBatch& b, bool predict, int n_shards, double linear_cost,
                   double quadratic_cost, std::vector<Shard>& shards) {
  std::vector<int> shard_of(b.n_seqs, 0);
  plan_shards(b.cu_seqlens, static_cast<int>(b.n_seqs), n_shards, linear_cost, quadratic_cost, shard_of.data());
  shards.resize(static_cast<size_t>(n_shards));
  for (Shard& sh : shards) sh.clear();
  std::vector<uint32_t> local_index(b.n_seqs, 0);
  for (size_t s = 0; s < b.n_seqs; ++s) {
    Shard& sh = shards[shard_of[s]];
    local_index[s] = static_cast<uint32_t>(sh.seqs.size());
    sh.seqs.push_back(s);
  }
  if (predict) return;
  // pooled row i <-> pooled_indices[i]; raw rows in raw_indices order (backends/candle/src/lib.rs:694-706)
  for (size_t i = 0; i < b.n_pooled; ++i) {
    const uint32_t s = b.pooled_indices[i];
    Shard& sh = shards[shard_of[s]];
    sh.pooled_idx.push_back(local_index[s]);
    sh.pooled_dst_row.push_back(i);
  }
  size_t row = 0;
  for (size_t i = 0; i < b.n_raw; ++i) {
    const uint32_t s = b.raw_indices[i];
    Shard& sh = shards[shard_of[s]];
    const size_t len = b.cu_seqlens[s + 1] - b.cu_seqlens[s];
    sh.raw_idx.push_back(local_index[s]);
    sh.raw_dst_row.push_back(row);
    sh.raw_len.push_back(len);
    row += len;
  }
}

void gather_shard_tokens(const HostBatch& b, Shard& sh) {
  size_t total = 0;
  for (size_t s : sh.seqs) total += b.cu_seqlens[s + 1] - b.cu_seqlens[s];
  sh.ids.resize(total);
  sh.types.resize(total);
  sh.pos.resize(total);
  sh.cu.resize(sh.seqs.size() + 1);
  sh.cu[0] = 0;
  sh.max_length = 0;
  size_t off = 0;
  for (size_t i = 0; i < sh.seqs.size(); ++i) {
    const uint32_t a = b.cu_seqlens[sh.seqs[i]], e = b.cu_seqlens[sh.seqs[i] + 1];
    const size_t n = e - a;
    std::memcpy(sh.ids.data() + off, b.input_ids + a, n * 4);
    if (b.token_type_ids) std::memcpy(sh.types.data() + off, b.token_type_ids + a, n * 4);
    else std::memset(sh.types.data() + off, 0, n * 4);
    std::memcpy(sh.pos.data() + off, b.position_ids + a, n * 4);
    off += n;
    sh.cu[i + 1] = static_cast<uint32_t>(off);
    sh.max_length = std::max(sh.max_length, static_cast<uint32_t>(n));
  }
}

void size_shard_results(Shard& sh, bool predict, size_t D, size_t DR, size_t C) {
  size_t raw_rows = 0;
  for (size_t l : sh.raw_len) raw_rows += l;
  sh.pooled.resize(sh.pooled_idx.size() * D);
  sh.raw.resize(raw_rows * DR);
  sh.scores.resize(predict ? sh.seqs.size() * C : 0);
}

void scatter_shard(const Shard& sh, bool predict, size_t D, size_t DR, size_t C, float* pooled_out,
                   float* raw_out, float* scores_out) {
  if (pooled_out) {
    for (size_t i = 0; i < sh.pooled_dst_row.size(); ++i) {
      std::memcpy(pooled_out + sh.pooled_dst_row[i] * D, sh.pooled.data() + i * D, D * 4);
    }
  }
  if (raw_out) {
    size_t src_row = 0;
    for (size_t i = 0; i < sh.raw_dst_row.size(); ++i) {
      std::memcpy(raw_out + sh.raw_dst_row[i] * DR, sh.raw.data() + src_row * DR, sh.raw_len[i] * DR * 4);
      src_row += sh.raw_len[i];
    }
  }
  if (predict && scores_out) {  // scores by batch position (backends/candle/src/lib.rs:718-722)
    for (size_t i = 0; i < sh.seqs.size(); ++i) {
      std::memcpy(scores_out + sh.seqs[i] * C, sh.scores.data() + i * C, C * 4);
    }
  }
}

}  // namespace tei
