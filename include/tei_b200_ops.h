/* Kernel-level C ABI of libtei_b200.so: one entry point per native kernel that the reference's
 * Candle backend reaches through a third-party crate.  All pointers named *_dev / "device" are
 * device pointers owned by the caller; `stream` is a cudaStream_t passed as void* (NULL = the
 * default stream).  Every function enqueues work and returns immediately: 0 on success, a
 * cudaError_t / CUresult value otherwise.  `status_dev` is a device int the caller zeroes; a
 * kernel whose bounded wait ran out stores a non-zero code there (101 producer, 102 MMA issuer,
 * 103 epilogue, 104 attention, 105 shared-memory alignment) instead of hanging.  Where a
 * function takes `status_dev` it is mandatory: NULL is refused with cudaErrorInvalidValue before
 * anything is launched.
 *
 * dtype: 0 = float16, 1 = bfloat16.  Nothing here allocates device memory.
 */
#ifndef TEI_B200_OPS_H_
#define TEI_B200_OPS_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Activations of tei_b200_op_linear. */
enum {
  TEI_B200_ACT_NONE = 0,
  TEI_B200_ACT_GELU = 1,       /* tanh approximation */
  TEI_B200_ACT_RELU = 2,
  TEI_B200_ACT_TANH = 3,
  TEI_B200_ACT_SWIGLU = 4,     /* weight rows interleaved: 128 gate rows, 128 up rows, ... */
  TEI_B200_ACT_RELU_LOG1P = 5
};

/* out[M, N'] = act(a[M,K] @ w[N,K]^T + bias[N]) (+ residual[M,N']), N' = N/2 for SWIGLU else N.
 * Replaces Linear::forward -> CublasLtWrapper::matmul
 * (backends/candle/src/layers/linear.rs:51-75, layers/cublaslt.rs:49-87).
 * K and lda must be multiples of 8; a and w 16-byte aligned.  bias / residual may be NULL. */
int tei_b200_op_linear(const void* a_dev, const void* w_dev, const void* bias_dev,
                       const void* residual_dev, void* out_dev, int M, int N, int K, int lda,
                       int ldo, int ldr, int act, int dtype, int* status_dev, void* stream);

/* Host helper (no GPU needed): the tiling tei_b200_op_linear uses for an M x N problem on a GPU
 * of `sms` SMs: 0 = pairs of CTAs on 256 x 256 tiles (cta_group::2), 256 / 128 / 64 = one CTA per
 * 128 x that-many-columns tile.  The narrow tiles (narrow_ok != 0: no gated activation, no
 * rotary epilogue) are taken where the wide ones would leave most SMs without a tile: batches
 * of up to about two thousand tokens (a wave of narrow tiles is hardly shorter than a wave of
 * pairs, so larger batches stay with the pairs).  -1 on bad arguments. */
int tei_b200_gemm_tiling(int M, int N, int sms, int narrow_ok);

/* Host helper: lists the (sequence, 128-row query tile) work items of a packed batch as
 * {seq_start, seq_len, q0, 0} int quadruples, most expensive first.  Returns the item count;
 * writes nothing when the count exceeds capacity_items or work_out is NULL.  cu_seqlens is a
 * HOST array of n_seqs + 1 entries (Batch::cumulative_seq_lengths,
 * backends/core/src/lib.rs:9-17). */
int tei_b200_attention_plan(const int32_t* cu_seqlens_host, int n_seqs, int causal,
                            int32_t* work_out, int capacity_items);
/* The same for sliding-window attention (window_size_left / window_size_right of
 * backends/candle/src/flash_attn.rs:23-36,72-95): key j counts for query i when
 * i - window_left <= j <= i + window_right, -1 = no limit on that side, causal forces
 * window_right = 0.  The fourth number of each quadruple is the first key the tile can see,
 * rounded down to a multiple of 64. */
int tei_b200_attention_plan_windowed(const int32_t* cu_seqlens_host, int n_seqs, int causal,
                                     int window_left, int window_right, int32_t* work_out,
                                     int capacity_items);

/* Variable-length attention over a packed batch.  Replaces flash_attn_varlen
 * (backends/candle/src/flash_attn.rs:23-120).  q/k/v are token-major strided views
 * (row stride ld_* elements, head h at column h*head_dim); work_dev holds the quadruples from
 * tei_b200_attention_plan copied to the device.  head_dim 32, 64 or 128.  alibi_slopes_dev: fp32
 * [n_heads] or NULL. */
int tei_b200_op_attention(const void* q_dev, const void* k_dev, const void* v_dev, void* out_dev,
                          const int32_t* work_dev, int n_work, int total_tokens, int n_heads,
                          int n_kv_heads, int head_dim, int ld_q, int ld_k, int ld_v, int ld_o,
                          int causal, float softmax_scale, const float* alibi_slopes_dev,
                          int dtype, int* status_dev, void* stream);
/* The same with a sliding window; work_dev must come from tei_b200_attention_plan_windowed
 * called with the same causal / window arguments. */
int tei_b200_op_attention_windowed(const void* q_dev, const void* k_dev, const void* v_dev,
                                   void* out_dev, const int32_t* work_dev, int n_work,
                                   int total_tokens, int n_heads, int n_kv_heads, int head_dim,
                                   int ld_q, int ld_k, int ld_v, int ld_o, int causal,
                                   int window_left, int window_right, float softmax_scale,
                                   const float* alibi_slopes_dev, int dtype, int* status_dev,
                                   void* stream);

/* out[t] = LayerNorm(word[ids[t]] + type[type_ids[t]] + pos[pos_ids[t]]).  Replaces
 * BertEmbeddings::forward (backends/candle/src/models/bert.rs:83-101) and
 * NomicBertEmbeddings::forward (models/nomic.rs:84-95; pos table NULL).  With gamma NULL it is
 * the plain embedding gather of flash_qwen3.rs:409. */
int tei_b200_op_embed_layernorm(const int32_t* ids_dev, const int32_t* type_ids_dev,
                                const int32_t* pos_ids_dev, const void* word_dev,
                                const void* type_dev, const void* pos_dev, const void* gamma_dev,
                                const void* beta_dev, void* out_dev, int n_tokens, int hidden,
                                float eps, int dtype, void* stream);

/* rms = 0: out = LayerNorm(x + residual) (layers/layer_norm.rs:54-72,108-132); residual has the
 * model dtype.  rms = 1: sum = x + residual kept in fp32 in sum_out_dev (residual_dev is fp32
 * too and may alias sum_out_dev), out = RMSNorm(sum) (layers/rms_norm.rs:30-83). */
int tei_b200_op_add_norm(const void* x_dev, const void* residual_dev, const void* gamma_dev,
                         const void* beta_dev, void* out_dev, float* sum_out_dev, int n_tokens,
                         int hidden, float eps, int rms, int dtype, void* stream);

/* In place on q and k: optional per-head RMSNorm (flash_qwen3.rs:150-151) then half-rotation
 * rotary embedding (candle-rotary apply_rotary_inplace at flash_nomic.rs:81, flash_qwen3.rs:153;
 * CPU formula layers/rotary.rs:118-130).  cos/sin: fp32 [max_pos, head_dim/2]. */
int tei_b200_op_qk_norm_rope(void* q_dev, void* k_dev, const int32_t* pos_ids_dev,
                             const float* cos_dev, const float* sin_dev, const void* q_gamma_dev,
                             const void* k_gamma_dev, int n_tokens, int n_heads, int n_kv_heads,
                             int head_dim, int ld_q, int ld_k, float eps, int dtype, void* stream);

/* Segmented pooling driven by cu_seqlens: out[i] = pool(rows of sequence seq_index[i]).
 * mode 0 CLS, 1 mean, 2 max (SPLADE), 3 last token (flash_bert.rs:396-490).  fp32 output,
 * optionally L2-normalised (core/src/infer.rs:288-303). */
int tei_b200_op_pool(const void* x_dev, const int32_t* cu_seqlens_dev, const int32_t* seq_index_dev,
                     float* out_dev, int n_out, int hidden, int mode, int normalize, int dtype,
                     void* stream);

/* out[i] = float(x[row_index[i]]): the raw-embedding row gather + fp32 cast
 * (flash_bert.rs:496-523, backends/candle/src/lib.rs:689-692). */
int tei_b200_op_gather_rows_f32(const void* x_dev, const int32_t* row_index_dev, float* out_dev,
                                int n_rows, int hidden, int dtype, void* stream);

/* out[r, n] = act(in[r,:] . w[n,:] + b[n]) on fp32 rows: classification heads
 * (models/bert.rs:405-465) and Dense modules (backends/candle/src/lib.rs:672-680). */
int tei_b200_op_head_linear(const float* in_dev, const void* w_dev, const void* b_dev,
                            float* out_dev, int rows, int N, int K, int act, int dtype,
                            void* stream);

/* The fused q/k/v projection with its rotary epilogue: out[M, N] = a @ w^T + bias, then on the
 * output's q heads (columns [0, q_cols)) and k heads (columns [q_cols, q_cols + k_cols)), heads of
 * head_dim (32, 64 or 128) columns: per-head RMSNorm with q_gamma / k_gamma when they are not
 * NULL (flash_qwen3.rs:150-151), then the rotary embedding with the cos / sin row of
 * pos_ids[row] (flash_nomic.rs:81, flash_qwen3.rs:153; tables [max_pos, head_dim / 2] fp32, as
 * for tei_b200_op_qk_norm_rope).  The remaining columns (v) are the plain projection.  Same
 * result, bit for bit, as tei_b200_op_linear followed by tei_b200_op_qk_norm_rope on its
 * output, without the second pass over q and k.  ldo must be a multiple of 8 and out 16-byte
 * aligned. */
int tei_b200_op_linear_rope(const void* a_dev, const void* w_dev, const void* bias_dev, void* out_dev, int M,
                            int N, int K, int lda, int ldo, const int32_t* pos_ids_dev, const float* cos_dev,
                            const float* sin_dev, const void* q_gamma_dev, const void* k_gamma_dev,
                            int head_dim, int q_cols, int k_cols, float eps, int dtype, int* status_dev,
                            void* stream);

/* tei_b200_op_linear on the first min(M, *m_rows_dev) rows only: M is the capacity of the
 * buffers, the row count lives on the device (the tokens routed to one expert,
 * backends/candle/src/models/nomic.rs:325-353, where the reference syncs to the host instead). */
int tei_b200_op_linear_rows_dev(const void* a_dev, const void* w_dev, const void* bias_dev,
                                void* out_dev, int M, int N, int K, int lda, int ldo, int act,
                                int dtype, const int32_t* m_rows_dev, int* status_dev, void* stream);

/* Mixture-of-experts routing (NomicRouter::forward, backends/candle/src/models/nomic.rs:229-243,
 * and the bookkeeping of NomicExperts::forward `:325-341`): per token the fp32 softmax over the
 * n_experts logits and its top_k largest entries (weights rounded to the model dtype), plus,
 * for every pick, the row it takes among the tokens of its expert.  counts_dev [n_experts] is
 * zeroed by the call, counts the picks per expert while the kernel runs and holds those counts
 * afterwards.  Rows within an expert are handed out in arrival order, so pos_dev may differ
 * between runs; everything computed from it per token does not.  n_experts <= 64, top_k <= 8. */
int tei_b200_op_moe_route(const void* logits_dev, int ld_logits, int n_tokens, int n_experts,
                          int top_k, int32_t* topk_expert_dev, float* topk_weight_dev,
                          int32_t* pos_dev, int32_t* counts_dev, int dtype, void* stream);

/* xg[(expert * cap + pos) * hidden ..] = x[token] for every pick (the index_select of
 * nomic.rs:343-345); cap = rows reserved per expert. */
int tei_b200_op_moe_gather(const void* x_dev, const int32_t* topk_expert_dev, const int32_t* pos_dev,
                           void* xg_dev, int n_tokens, int top_k, int hidden, long long cap,
                           int dtype, void* stream);

/* out[token] = sum over its picks of weight * yg[expert * cap + pos] + bias (the index_add and
 * broadcast_add of nomic.rs:346-355), accumulated in fp32.  bias may be NULL. */
int tei_b200_op_moe_combine(const void* yg_dev, const int32_t* topk_expert_dev,
                            const float* topk_weight_dev, const int32_t* pos_dev,
                            const void* bias_dev, void* out_dev, int n_tokens, int top_k, int hidden,
                            long long cap, int dtype, void* stream);

/* tei_b200_op_moe_route for callers that cannot allocate device memory.  It has no counterpart
 * in the reference.  The per-expert counters, which tei_b200_op_moe_route takes from the
 * caller, live in a 256-byte array inside the library instead (held by every GPU that loads
 * the library, until the process exits), so an embedding host that gave all device memory to
 * its own arena at start-up and forbids cudaMalloc on the request path - cudaMalloc
 * synchronises the device and can fail half-way through a request - or an operator plugin that
 * only receives the tensors of the one operator it implements, can still route.  The call
 * itself allocates and frees nothing.
 *   - n_experts <= 64 (the size of the built-in array); more returns an error and a message in
 *     `err` (may be NULL).
 *   - counts_out_dev [n_experts] receives the picks per expert; it may be NULL.
 *   - All calls on one GPU share the array: it is cleared at the start of each call, and calls
 *     that overlap on the GPU (two streams, two threads) corrupt each other's counts - order
 *     them.
 *   - The first call on a device looks up the array's device address; make it before any stream
 *     capture begins.
 * Outputs as for tei_b200_op_moe_route. */
int tei_b200_op_moe_route_noalloc(const void* logits_dev, int ld_logits, int n_tokens,
                                  int n_experts, int top_k, int32_t* topk_expert_dev,
                                  float* topk_weight_dev, int32_t* pos_dev,
                                  int32_t* counts_out_dev, int dtype, void* stream, char* err,
                                  size_t err_cap);

/* Self-test of the bounded waits; no counterpart in the reference.  Every wait inside the GEMM
 * and attention kernels gives up after a fixed number of probes, writes a code to *status_dev
 * and lets the kernel return.  This launches one CTA that waits, with that same primitive, on a
 * barrier nobody arrives at, with a limit of `limit` probes (1 .. 4096, a few microseconds to
 * milliseconds): afterwards *status_dev holds 101 and *gave_up_dev (optional) 1.  The kernel
 * cannot spin longer than its limit, trap or fault.  status_dev is mandatory here and in
 * tei_b200_op_linear / tei_b200_op_attention: a NULL status pointer is refused with
 * cudaErrorInvalidValue before anything is launched. */
int tei_b200_op_bounded_wait_probe(int* status_dev, int limit, int* gave_up_dev, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TEI_B200_OPS_H_ */
