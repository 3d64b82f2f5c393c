/* C ABI of libtei_b200.so: a B200 (sm_100a) implementation of the `Backend` trait of Text
 * Embeddings Inference (backends/core/src/lib.rs:37-48) for the model paths that backends/candle
 * serves with its flash models (flash_bert, flash_distilbert, flash_gte, flash_jina,
 * flash_jina_code, flash_mistral, flash_modernbert, flash_nomic, flash_qwen2, flash_qwen3).  A Rust shim (`text-embeddings-inference_b200/rust_shim`) binds these functions
 * and implements `text_embeddings_backend_core::Backend` on top of them.
 *
 * Conventions
 *   - Every function returns a status code: 0 ok, 1 START (-> BackendError::Start), 2 INFERENCE
 *     (-> Inference), 3 UNHEALTHY (-> Unhealthy), 4 WEIGHTS_NOT_FOUND (-> WeightsNotFound),
 *     5 TIMEOUT (a kernel's bounded wait ran out; map to Inference).  When `err` is not NULL a
 *     NUL-terminated message is copied into it (at most err_cap bytes).
 *   - All batch pointers are HOST pointers borrowed for the duration of the call
 *     (`Batch`, backends/core/src/lib.rs:9-17); output buffers are caller-allocated host memory.
 *   - A handle is used by one thread at a time, as the reference's single backend thread does
 *     (backends/src/lib.rs:612-647), except through the per-replica entry points below.
 *     Nothing throws or aborts across this boundary.
 *   - The library owns all device memory: weights, a workspace that grows only when a larger
 *     batch than ever before arrives, and pinned staging buffers.
 */
#ifndef TEI_B200_H_
#define TEI_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct tei_b200 tei_b200_t;

enum {
  TEI_B200_OK = 0,
  TEI_B200_ERR_START = 1,
  TEI_B200_ERR_INFERENCE = 2,
  TEI_B200_ERR_UNHEALTHY = 3,
  TEI_B200_ERR_WEIGHTS_NOT_FOUND = 4,
  TEI_B200_ERR_TIMEOUT = 5
};

/* model_type (ModelType, backends/core/src/lib.rs:50-54) */
enum { TEI_B200_CLASSIFIER = 0, TEI_B200_EMBEDDING = 1 };
/* pool (Pool, backends/core/src/lib.rs:56-70) */
enum { TEI_B200_POOL_CLS = 0, TEI_B200_POOL_MEAN = 1, TEI_B200_POOL_SPLADE = 2, TEI_B200_POOL_LAST_TOKEN = 3 };

/* Replaces CandleBackend::new(model_path, dtype, model_type, dense_paths)
 * (backends/candle/src/lib.rs:163-168): reads config.json and the safetensors weights under
 * model_dir, dispatches on `model_type` like lib.rs:282-577 and places one full replica on each
 * listed CUDA device (devices == NULL or n_devices <= 0: device 0 only).  dtype: "float16" or
 * "bfloat16".  With more than one device a packed batch is split at sequence boundaries
 * across the replicas inside each call; no data crosses GPUs. */
int tei_b200_create(const char* model_dir, const char* dtype, int model_type, int pool,
                    const int* devices, int n_devices, tei_b200_t** out, char* err,
                    size_t err_cap);

/* The `dense_paths` argument of CandleBackend::new (backends/candle/src/lib.rs:579-629): appends
 * the Sentence-Transformers Dense module stored under `<model_dir>/<dense_path>/`
 * (`config.json` with in_features / out_features / bias / activation_function, and
 * `model.safetensors` with `linear.weight` [out, in] and `linear.bias`;
 * backends/candle/src/models/dense.rs:26-75).  Modules are applied to the pooled rows, in the
 * order of the calls, before the rows leave the device (lib.rs:672-680); raw rows are not
 * affected and tei_b200_output_dim() reports the last module's out_features.  A path without a
 * weight file is skipped like the reference does (returns OK, `err` holds the warning);
 * everything else that is wrong is TEI_B200_ERR_START.  Call between create and the first
 * batch. */
int tei_b200_add_dense(tei_b200_t* h, const char* dense_path, char* err, size_t err_cap);

void tei_b200_destroy(tei_b200_t* h);

/* Backend::health (backends/core/src/lib.rs:38).  Cheap when the last call succeeded; after a
 * failed call it runs a one-token forward, like the probe of backends/src/lib.rs:393-409. */
int tei_b200_health(tei_b200_t* h);

/* Backend::is_padded: always 0, the path is unpadded (flash_bert.rs:530-532). */
int tei_b200_is_padded(const tei_b200_t* h);
/* Backend::max_batch_size: -1 means None (backends/core/src/lib.rs:39-41). */
int tei_b200_max_batch_size(const tei_b200_t* h);
/* Width of a pooled embedding row (hidden size; vocabulary size for SPLADE). */
int tei_b200_output_dim(const tei_b200_t* h);
/* Width of a raw (per-token) embedding row. */
int tei_b200_hidden_size(const tei_b200_t* h);
/* Number of classes of a classifier (0 for embedding models). */
int tei_b200_num_classes(const tei_b200_t* h);
/* First position id of every sequence: what the router adds when it builds position_ids
 * (router/src/lib.rs:184-192 -> core/src/tokenization.rs:406-411): pad_token_id + 1 for the
 * RoBERTa family, else 0.  For hosts that build batches themselves (tei_b200_queue_append). */
int tei_b200_position_offset(const tei_b200_t* h);

/* Backend::embed (backends/candle/src/lib.rs:656-709).
 *   pooled_out [n_pooled, output_dim]: row i is the embedding of batch position pooled_idx[i]
 *                                      (lib.rs:696-698);
 *   raw_out    [sum of len(raw_idx[j]), hidden]: token rows of the raw_idx sequences, in
 *                                      raw_idx order (lib.rs:700-706).
 * normalize != 0 L2-normalises the pooled rows on the device (the router does it on the host,
 * core/src/infer.rs:288-303; doing it twice is harmless). */
int tei_b200_embed(tei_b200_t* h, const uint32_t* input_ids, const uint32_t* token_type_ids,
                   const uint32_t* position_ids, size_t n_tokens,
                   const uint32_t* cumulative_seq_lengths, size_t n_seqs, uint32_t max_length,
                   const uint32_t* pooled_idx, size_t n_pooled, const uint32_t* raw_idx,
                   size_t n_raw, int normalize, float* pooled_out, float* raw_out, char* err,
                   size_t err_cap);

/* Backend::predict (backends/candle/src/lib.rs:711-725): scores_out [n_seqs, num_classes],
 * row i = raw logits of batch position i (sigmoid / softmax stay with the caller,
 * core/src/infer.rs:458-480). */
int tei_b200_predict(tei_b200_t* h, const uint32_t* input_ids, const uint32_t* token_type_ids,
                     const uint32_t* position_ids, size_t n_tokens,
                     const uint32_t* cumulative_seq_lengths, size_t n_seqs, uint32_t max_length,
                     float* scores_out, char* err, size_t err_cap);

/* Several batches in flight, one per replica.  The reference runs exactly one backend thread
 * that takes one command at a time from a channel (backends/src/lib.rs:612-647), so a second
 * batch waits in core/src/infer.rs:547-625 while the first one computes.  A host that wants N
 * batches in flight starts N such threads over one handle created with N devices (the same
 * index may be listed twice: two replicas on one GPU overlap one batch's copies and host work
 * with the other's kernels) and gives thread i the replica index i:
 *   tei_b200_num_replicas : how many replicas the handle owns;
 *   tei_b200_embed_on / tei_b200_predict_on : embed / predict with the WHOLE batch on that one
 *       replica; same arguments, results and error codes as tei_b200_embed / tei_b200_predict.
 * Calls with different replica indices may run concurrently; calls with the same index are
 * serialised inside the library.  They do not touch the staged-batch state of the handle.  The
 * whole-handle calls (embed, predict, stage, run, sync, fetch) use every replica and wait for
 * per-replica calls in flight; tei_b200_health runs its probe on replica 0 under that
 * replica's lock, so it is safe next to per-replica callers. */
int tei_b200_num_replicas(const tei_b200_t* h);
int tei_b200_embed_on(tei_b200_t* h, int replica, const uint32_t* input_ids,
                      const uint32_t* token_type_ids, const uint32_t* position_ids, size_t n_tokens,
                      const uint32_t* cumulative_seq_lengths, size_t n_seqs, uint32_t max_length,
                      const uint32_t* pooled_idx, size_t n_pooled, const uint32_t* raw_idx,
                      size_t n_raw, int normalize, float* pooled_out, float* raw_out, char* err,
                      size_t err_cap);
int tei_b200_predict_on(tei_b200_t* h, int replica, const uint32_t* input_ids,
                        const uint32_t* token_type_ids, const uint32_t* position_ids, size_t n_tokens,
                        const uint32_t* cumulative_seq_lengths, size_t n_seqs, uint32_t max_length,
                        float* scores_out, char* err, size_t err_cap);

/* The three phases of embed / predict, exposed separately so that a caller can keep a batch
 * resident in HBM and time the forward alone.  No counterpart in the reference, whose forward
 * always uploads its inputs (flash_bert.rs:376-383).
 *   stage : validate, split across replicas, copy the batch to the device(s);
 *   run   : enqueue one forward of the staged batch on every replica (asynchronous);
 *   sync  : wait for all replicas and check their status words;
 *   fetch : copy the results of the last run back (same layout as embed / predict). */
int tei_b200_stage(tei_b200_t* h, const uint32_t* input_ids, const uint32_t* token_type_ids,
                   const uint32_t* position_ids, size_t n_tokens,
                   const uint32_t* cumulative_seq_lengths, size_t n_seqs, uint32_t max_length,
                   const uint32_t* pooled_idx, size_t n_pooled, const uint32_t* raw_idx,
                   size_t n_raw, int normalize, int predict, char* err, size_t err_cap);
int tei_b200_run_staged(tei_b200_t* h, char* err, size_t err_cap);
int tei_b200_sync(tei_b200_t* h, char* err, size_t err_cap);
int tei_b200_fetch(tei_b200_t* h, float* pooled_out, float* raw_out, float* scores_out, char* err,
                   size_t err_cap);

/* Runs the staged forward `steps` times back to back on every replica and returns the device
 * time of the whole sequence in milliseconds (CUDA events on the launching stream, max over
 * replicas).  Synchronises before returning. */
int tei_b200_run_staged_timed(tei_b200_t* h, int steps, double* device_ms, char* err,
                              size_t err_cap);

/* Per-kernel-class device timing.  While on, every kernel launch is bracketed by a pair of
 * CUDA events on its stream; tei_b200_kernel_times returns, per class, the milliseconds and
 * the launches accumulated since profiling was switched on (classes: 0 embedding, 1 dense
 * layer GEMM, 2 attention, 3 LayerNorm / RMSNorm, 4 rotary, 5 pooling and heads).  Returns the
 * number of classes written. */
int tei_b200_set_profiling(tei_b200_t* h, int on);
int tei_b200_kernel_times(const tei_b200_t* h, double* ms_out, double* launches_out, int n);

/* Counters of the last call, summed / maxed over replicas.  out[0] device ms of the forward
 * (max over replicas), [1] host-to-device bytes, [2] device-to-host bytes, [3] kernels
 * launched, [4] tokens, [5] calls so far, [6] total device ms, [7] total tokens.  Returns the
 * number of values written (at most n). */
int tei_b200_stats(const tei_b200_t* h, double* out, int n);

/* Host-only helpers, no GPU needed.  The compute capability the library is built for, in the
 * reference's notation (major * 10 + minor: 100), and the reference's rule for which device a
 * build may run on (backends/candle/src/compute_cap.rs:8-12,27-40).  `create` applies the rule
 * to every device it is given and refuses with a `Start` error worded like
 * backends/candle/src/lib.rs:240-248 ("Runtime compute cap .. is not compatible with compile time
 * compute cap ..") where the reference's CUDA build refuses too. */
int tei_b200_compile_compute_cap(void);
int tei_b200_compute_cap_matching(int runtime_cap, int compile_cap);

/* Host-only helper, no GPU needed: the replica a sequence of a packed batch is sent to when a
 * handle has n_shards devices.  Cost of a sequence of length L: linear_cost * L +
 * quadratic_cost * L * L, balanced longest-first.  shard_of_seq has n_seqs entries. */
int tei_b200_plan_shards(const uint32_t* cumulative_seq_lengths, size_t n_seqs, int n_shards,
                         double linear_cost, double quadratic_cost, int* shard_of_seq);

/* Host-only, no GPU needed: the split of one packed batch over n_shards replicas and the way
 * back, with a stand-in for the forward.  The batch is split exactly as tei_b200_embed /
 * tei_b200_predict split it on a handle with n_shards devices (same planner, same gather of
 * the tokens, same renumbering of the pooled / raw index lists, same scatter of the rows); in
 * place of a model every shard echoes its own sub-batch: a pooled row (and, with predict != 0,
 * a score row) is (sum of the sequence's input ids mod 65521) + column, a raw row is
 * id mod 4096 + 7 * type id + 13 * (position id mod 4096) + column, `width` columns each.  The
 * rows come back in the layout of Backend::embed / predict (backends/candle/src/lib.rs:694-706,
 * 718-722), so a caller can check the whole bookkeeping of the split against the unsplit batch.
 * shard_tokens_out (optional, n_shards entries) receives the tokens each shard got. */
int tei_b200_split_echo(const uint32_t* input_ids, const uint32_t* token_type_ids, const uint32_t* position_ids,
                        size_t n_tokens, const uint32_t* cumulative_seq_lengths, size_t n_seqs,
                        const uint32_t* pooled_idx, size_t n_pooled, const uint32_t* raw_idx, size_t n_raw,
                        int predict, int n_shards, double linear_cost, double quadratic_cost, int width,
                        float* pooled_out, float* raw_out, float* scores_out, int* shard_tokens_out);

/* Self-test of the TIMEOUT path; no counterpart in the reference.  The next forward on
 * `replica` ends with a kernel that writes `device_code` (> 0, e.g. 104) to the status word, which
 * is all a kernel whose bounded wait ran out leaves behind; nothing hangs or faults.  That call
 * then returns TEI_B200_ERR_TIMEOUT (-> BackendError::Inference, backends/candle/src/lib.rs:728-740),
 * the handle turns unhealthy (backends/src/lib.rs:621-642) and the next tei_b200_health runs its
 * one-token probe (backends/src/lib.rs:393-409).  One shot. */
int tei_b200_selftest_report_timeout(tei_b200_t* h, int replica, int device_code);

/* The last-layer shortcut, on by default: when only one row per sequence leaves the model (CLS
 * or last-token pooling, or a classifier head, and no raw request in the batch), everything
 * behind the last layer's attention scores runs on those rows only.  on == 0 makes every call
 * compute every row, as the reference does (flash_bert.rs:169-185); the results are the same
 * bit for bit.  No counterpart in the reference. */
int tei_b200_set_last_layer_shortcut(tei_b200_t* h, int on);

/* Rotary models (NomicBERT, GTE, Qwen3 / Qwen2 / Mistral / Llama, ModernBERT): the rotary
 * embedding and Qwen3's per-head q/k RMSNorm run in the epilogue of the q/k/v projection
 * (on == 1) or as a kernel of their own behind it, the form the reference has (on == 0;
 * flash_nomic.rs:81, flash_qwen3.rs:150-153).  on < 0, the default, picks per model whichever
 * measured faster: the epilogue for RoPE alone, the separate kernel when the q/k RMSNorm comes
 * with it.  The results are the same bit for bit in every mode. */
int tei_b200_set_fused_rope(tei_b200_t* h, int on);

/* Post-LN models (BERT family, NomicBERT): the residual of the feed-forward block is added by the
 * LayerNorm kernel behind the block (on == 0, the default: the form the reference has, bert.rs /
 * flash_bert.rs: `layer_norm.forward(&hidden_states, Some(&residual))`), or (on != 0) in the
 * epilogue of the block's output projection, where that projection's reduction is at least 2048
 * long so that the tile's main loop hides the extra reads; the LayerNorm then reads one tensor.
 * The sum is rounded to the activation dtype once either way; results agree within that
 * rounding, not bit for bit.  On the benchmark batch the two forms are equally fast. */
int tei_b200_set_fused_residual(tei_b200_t* h, int on);

#ifdef __cplusplus
}
#endif
#endif /* TEI_B200_H_ */
