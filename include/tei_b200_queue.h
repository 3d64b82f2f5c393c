/* C ABI of the batching queue of libtei_b200.so: the caller-side row next to the backend.
 *
 * Replaces the state machine of `queue_blocking_task` (core/src/queue.rs:98-200) for hosts that
 * drive the backend without the router (the gRPC adapter, tests, the benchmark) or that want N
 * batches in flight and therefore N consumers: requests are appended in arrival order and every
 * `next_batch` call packs the longest FIFO prefix that fits into one `Batch`
 * (backends/core/src/lib.rs:9-27).  Integer work only; results are bit-exact with the
 * reference's rules:
 *   - unpadded models: a request joins while current_tokens + len <= max_batch_tokens
 *     (queue.rs:150-155); padded models: while max(max_length, len) * (batch size + 1) fits
 *     (queue.rs:150-152);
 *   - the first request that does not fit stays at the head of the queue and ends the batch,
 *     nothing behind it is taken (queue.rs:157-160);
 *   - at most max_batch_requests requests per batch (queue.rs:179);
 *   - cumulative_seq_lengths starts at 0 (queue.rs:131-132,175); pooled_indices / raw_indices
 *     hold batch positions by the request's pooling flag (queue.rs:162-165);
 *   - requests whose client went away are skipped (queue.rs:142-146): tei_b200_queue_cancel.
 * Every function is safe to call from several threads; status codes are those of tei_b200.h.
 */
#ifndef TEI_B200_QUEUE_H_
#define TEI_B200_QUEUE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct tei_b200_queue tei_b200_queue_t;

/* Queue::new (core/src/queue.rs:40-65).  max_batch_requests = 0 means None. */
int tei_b200_queue_create(int padded_model, size_t max_batch_tokens, size_t max_batch_requests,
                          tei_b200_queue_t** out);
void tei_b200_queue_destroy(tei_b200_queue_t* q);

/* Queue::append (queue.rs:67-75) of one Entry.  The encoding (core/src/tokenization.rs:368-419)
 * is copied.  token_type_ids == NULL stands for zeros; position_ids == NULL for
 * position_offset, position_offset + 1, ... (tokenization.rs:406-411 with the offset of
 * router/src/lib.rs:185-192).  pooling: 1 pooled, 0 raw (Metadata::pooling).  `tag` is the
 * caller's name for the request (what Metadata carries in the reference); it comes back with the
 * batch.  len == 0 is refused (the tokenizer never produces an empty encoding). */
int tei_b200_queue_append(tei_b200_queue_t* q, const uint32_t* input_ids, const uint32_t* token_type_ids,
                          const uint32_t* position_ids, size_t len, uint32_t position_offset,
                          int pooling, uint64_t tag);

/* Marks every queued request with this tag as dropped by its client; next_batch skips them.
 * Returns how many were marked through *n_marked (may be NULL). */
int tei_b200_queue_cancel(tei_b200_queue_t* q, uint64_t tag, size_t* n_marked);

/* Requests waiting (the te_queue_size gauge of queue.rs:112-113,197-198). */
size_t tei_b200_queue_len(const tei_b200_queue_t* q);

/* One NextBatch command (queue.rs:118-195) into caller-allocated buffers: input_ids,
 * token_type_ids, position_ids hold token_cap entries; cu_seqlens seq_cap + 1; pooled_idx,
 * raw_idx and tags seq_cap.  The buffer sizes act as further limits of the batch: a request
 * that does not fit them stays queued like one that exceeds max_batch_tokens (size them
 * max_batch_tokens and max_batch_requests to get exactly the reference's batches).  *n_seqs == 0
 * afterwards means None (nothing fitted or the queue was empty). */
int tei_b200_queue_next_batch(tei_b200_queue_t* q, uint32_t* input_ids, uint32_t* token_type_ids,
                              uint32_t* position_ids, size_t token_cap, uint32_t* cu_seqlens,
                              uint32_t* pooled_idx, uint32_t* raw_idx, uint64_t* tags, size_t seq_cap,
                              size_t* n_tokens, size_t* n_seqs, size_t* n_pooled, size_t* n_raw,
                              uint32_t* max_length);

#ifdef __cplusplus
}
#endif
#endif  /* TEI_B200_QUEUE_H_ */
