// The batching queue (include/tei_b200_queue.h): FIFO of encoded requests and the NextBatch rule
// of core/src/queue.rs:118-200, written over a mutex instead of the reference's command channel
// so that several consumers (one per replica) can ask for batches.
#include "../../include/tei_b200_queue.h"

#include "../../include/tei_b200.h"

#include <algorithm>
#include <cstring>
#include <deque>
#include <mutex>
#include <new>
#include <vector>

namespace {

struct Entry {
  std::vector<uint32_t> ids, types, pos;
  bool pooling = true;
  bool dropped = false;
  uint64_t tag = 0;
};

}  // namespace

struct tei_b200_queue {
  bool padded_model = false;
  size_t max_batch_tokens = 0;
  size_t max_batch_requests = 0;  // 0: no limit
  mutable std::mutex mu;
  std::deque<Entry> entries;
};

extern "C" {

int tei_b200_queue_create(int padded_model, size_t max_batch_tokens, size_t max_batch_requests,
                          tei_b200_queue_t** out) {
  if (!out) return TEI_B200_ERR_START;
  *out = nullptr;
  if (max_batch_tokens == 0) return TEI_B200_ERR_START;
  tei_b200_queue* q = new (std::nothrow) tei_b200_queue();
  if (!q) return TEI_B200_ERR_START;
  q->padded_model = padded_model != 0;
  q->max_batch_tokens = max_batch_tokens;
  q->max_batch_requests = max_batch_requests;
  *out = q;
  return TEI_B200_OK;
}

void tei_b200_queue_destroy(tei_b200_queue_t* q) { delete q; }

int tei_b200_queue_append(tei_b200_queue_t* q, const uint32_t* input_ids, const uint32_t* token_type_ids,
                          const uint32_t* position_ids, size_t len, uint32_t position_offset,
                          int pooling, uint64_t tag) {
  if (!q || !input_ids || len == 0) return TEI_B200_ERR_INFERENCE;
  try {
    Entry e;
    e.ids.assign(input_ids, input_ids + len);
    if (token_type_ids) e.types.assign(token_type_ids, token_type_ids + len);
    else e.types.assign(len, 0u);
    if (position_ids) {
      e.pos.assign(position_ids, position_ids + len);
    } else {
      e.pos.resize(len);
      for (size_t i = 0; i < len; ++i) e.pos[i] = position_offset + static_cast<uint32_t>(i);
    }
    e.pooling = pooling != 0;
    e.tag = tag;
    std::lock_guard<std::mutex> lock(q->mu);
    q->entries.push_back(std::move(e));
  } catch (...) {
    return TEI_B200_ERR_INFERENCE;
  }
  return TEI_B200_OK;
}

int tei_b200_queue_cancel(tei_b200_queue_t* q, uint64_t tag, size_t* n_marked) {
  if (!q) return TEI_B200_ERR_INFERENCE;
  size_t n = 0;
  std::lock_guard<std::mutex> lock(q->mu);
  for (Entry& e : q->entries) {
    if (e.tag == tag && !e.dropped) {
      e.dropped = true;
      ++n;
    }
  }
  if (n_marked) *n_marked = n;
  return TEI_B200_OK;
}

size_t tei_b200_queue_len(const tei_b200_queue_t* q) {
  if (!q) return 0;
  std::lock_guard<std::mutex> lock(q->mu);
  return q->entries.size();
}

int tei_b200_queue_next_batch(tei_b200_queue_t* q, uint32_t* input_ids, uint32_t* token_type_ids,
                              uint32_t* position_ids, size_t token_cap, uint32_t* cu_seqlens,
                              uint32_t* pooled_idx, uint32_t* raw_idx, uint64_t* tags, size_t seq_cap,
                              size_t* n_tokens, size_t* n_seqs, size_t* n_pooled, size_t* n_raw,
                              uint32_t* max_length) {
  if (!q || !input_ids || !token_type_ids || !position_ids || !cu_seqlens || !pooled_idx || !raw_idx ||
      !tags || !n_tokens || !n_seqs || !n_pooled || !n_raw || !max_length) {
    return TEI_B200_ERR_INFERENCE;
  }
  size_t current_tokens = 0, taken = 0, np = 0, nr = 0;
  uint32_t max_len = 0;
  cu_seqlens[0] = 0;
  std::lock_guard<std::mutex> lock(q->mu);
  while (!q->entries.empty()) {
    Entry& e = q->entries.front();
    if (e.dropped) {  // the client went away while the request was queued
      q->entries.pop_front();
      continue;
    }
    const size_t entry_tokens = e.ids.size();
    // The reference computes the padded product in u32 (queue.rs:151); do it in 64 bits and
    // compare: a product that would have wrapped is over any budget anyway.
    const unsigned long long total_tokens =
        q->padded_model ? static_cast<unsigned long long>(std::max<size_t>(max_len, entry_tokens)) * (taken + 1)
                        : static_cast<unsigned long long>(current_tokens) + entry_tokens;
    if (total_tokens > q->max_batch_tokens) break;  // stays at the head of the queue
    if (current_tokens + entry_tokens > token_cap || taken + 1 > seq_cap) break;  // the caller's buffers
    if (e.pooling) pooled_idx[np++] = static_cast<uint32_t>(taken);
    else raw_idx[nr++] = static_cast<uint32_t>(taken);
    max_len = std::max<uint32_t>(max_len, static_cast<uint32_t>(entry_tokens));
    std::memcpy(input_ids + current_tokens, e.ids.data(), entry_tokens * sizeof(uint32_t));
    std::memcpy(token_type_ids + current_tokens, e.types.data(), entry_tokens * sizeof(uint32_t));
    std::memcpy(position_ids + current_tokens, e.pos.data(), entry_tokens * sizeof(uint32_t));
    current_tokens += entry_tokens;
    tags[taken] = e.tag;
    ++taken;
    cu_seqlens[taken] = static_cast<uint32_t>(current_tokens);
    q->entries.pop_front();
    if (q->max_batch_requests != 0 && taken == q->max_batch_requests) break;
  }
  *n_tokens = current_tokens;
  *n_seqs = taken;
  *n_pooled = np;
  *n_raw = nr;
  *max_length = max_len;
  return TEI_B200_OK;
}

}  // extern "C"
