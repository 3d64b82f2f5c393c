// Internal C++ interface between the host-side model code and the sm_100a kernels.
// Every launcher enqueues on the given stream, allocates nothing and returns a cudaError_t /
// status code; device-side failures (a bounded wait that ran out) are reported through the
// `status` word the caller passes and reads back after synchronising.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace tei {

enum DType : int { DT_F16 = 0, DT_BF16 = 1 };

// Activation fused into the GEMM epilogue.  ACT_SWIGLU and ACT_GEGLU expect the weight rows
// interleaved in blocks of 128 (128 gate rows, then the 128 matching up rows) and write N/2
// columns.
enum Act : int {
  ACT_NONE = 0,
  ACT_GELU = 1,        // tanh approximation, the only GELU the reference implements
  ACT_RELU = 2,
  ACT_TANH = 3,
  ACT_SWIGLU = 4,      // silu(gate) * up
  ACT_RELU_LOG1P = 5,  // log(1 + relu(x)), the SPLADE decoder activation
  ACT_GEGLU = 6,       // gelu_tanh(gate) * up, the JinaBERT feed-forward
};
inline bool act_is_glu(int act) { return act == ACT_SWIGLU || act == ACT_GEGLU; }

// Device status codes (0 = ok).
enum DevStatus : int {
  DEV_OK = 0,
  DEV_TIMEOUT_PRODUCER = 101,
  DEV_TIMEOUT_MMA = 102,
  DEV_TIMEOUT_EPILOGUE = 103,
  DEV_TIMEOUT_ATTN = 104,
  DEV_SMEM_ALIGN = 105,
};

// Optional epilogue of a fused q/k/v projection: per-head RMSNorm (when the gammas are given) and
// rotary embedding on the q and k heads of the output, the v columns untouched.  The output
// columns are [q heads | k heads | rest], heads of head_dim (32, 64 or 128) columns.
struct RopeFusion {
  const int* pos_ids;    // [M] position of every row
  const float* cos_tab;  // [max_pos, head_dim/2] fp32
  const float* sin_tab;
  const void* q_gamma;   // [head_dim] in the activation dtype, or nullptr: no norm
  const void* k_gamma;
  int head_dim;
  int q_cols, k_cols;    // widths of the q and of the k region in columns
  float eps;
};

struct GemmArgs {
  const void* a;        // [M, K] row-major activations, lda elements between rows
  const void* w;        // [N, K] row-major weights (as stored in safetensors)
  const void* bias;     // [N] or nullptr, same dtype as a
  const void* residual; // [M, N_out] or nullptr; added after the activation
  void* out;            // [M, N_out], ldo elements between rows
  int M, N, K;
  int lda, ldo, ldr;
  int act;
  int dtype;
  int* status;          // device int, stays 0 unless a wait ran out
  // Optional device int: the kernel works on min(M, *m_dev) rows.  M then is the capacity of the
  // buffers (what the tensor maps cover); the row count is only known on the device, as for the
  // tokens routed to one expert of a mixture-of-experts layer.
  const int* m_dev = nullptr;
  // Optional: q/k RMSNorm + RoPE in the epilogue (act must be ACT_NONE, no residual, output rows
  // 16-byte aligned).  Same bits as launch_qk_norm_rope applied to the plain projection.
  const RopeFusion* rope = nullptr;
};

// out = act(a @ w^T + bias) (+ residual).  tcgen05 + TMEM + TMA, persistent over 128x256 tiles.
int launch_gemm(const GemmArgs& g, cudaStream_t stream);
// Bytes of dynamic shared memory the GEMM kernel needs (for reporting).
int gemm_smem_bytes();
// The tiling launch_gemm picks for an M x N problem on `sms` SMs: 0 = CTA pairs (256 x 256 per
// pair), else the tile width of the single-CTA kernel (256, 128 or 64 columns; the narrow ones
// only where `narrow_ok`: plain epilogue, row count known on the host).  Host arithmetic only.
int gemm_tiling(int M, int N, int sms, bool narrow_ok);

struct AttnArgs {
  const void* q;  // token-major rows; head h of token t at q + t*ld_q + h*head_dim
  const void* k;
  const void* v;
  void* out;      // [T, n_heads*head_dim]
  const int* cu_seqlens;      // device, [n_seqs + 1]
  const int* work_items;      // device, [n_work][4] = {seq_start, seq_len, q0, first key}; see plan_attention
  int n_work;
  int total_tokens;
  int n_heads, n_kv_heads, head_dim;
  int ld_q, ld_k, ld_v, ld_o;  // row strides in elements
  int causal;
  // Sliding window (flash_attn.rs:82-95): key j counts for query i when
  // i - window_left <= j <= i + window_right; -1 = no limit on that side.  causal forces
  // window_right = 0.
  int window_left = -1, window_right = -1;
  float scale;
  const float* alibi_slopes;  // [n_heads] or nullptr
  int dtype;
  int* status;
};
int launch_attention(const AttnArgs& a, cudaStream_t stream);
// Host side: lists the (sequence, 128-row query tile) work items of a packed batch, most
// expensive first, as {seq_start, seq_len, q0, first key} quadruples (first key: the 64-aligned
// start of the keys the tile can see; 0 without a left window).  Returns the number of items
// needed; when that exceeds capacity_items (or work_out is null) nothing is written.
int plan_attention(const int* cu_seqlens, int n_seqs, int causal, int* work_out, int capacity_items,
                   int window_left = -1, int window_right = -1);

struct EmbedArgs {
  const int* ids;
  const int* type_ids;   // nullptr -> no token-type table
  const int* pos_ids;    // nullptr -> no position table
  const void* word;      // [V, H]
  const void* type_tab;  // [type_vocab, H] or nullptr
  const void* pos_tab;   // [max_pos, H] or nullptr
  const void* gamma;     // nullptr -> plain gather, no normalisation
  const void* beta;
  void* out;             // [T, H]
  int T, H;
  float eps;
  int dtype;
};
int launch_embed_layernorm(const EmbedArgs& e, cudaStream_t stream);

struct NormArgs {
  const void* x;         // [T, H]
  const void* residual;  // [T, H] or nullptr; model dtype for LayerNorm, fp32 for RMSNorm
  const void* gamma;
  const void* beta;      // LayerNorm only
  void* out;             // normalised rows
  float* sum_out;        // fp32 residual stream: x + residual written here (may alias residual); else nullptr
  int T, H;
  float eps;
  int rms;               // 0 LayerNorm, 1 RMSNorm
  int dtype;
  // 1: residual and sum_out are fp32 (pre-norm models), 0: residual in the model dtype and no
  // sum_out, -1: as RMSNorm implies.  gamma == nullptr leaves the sum un-normalised.
  int residual_f32 = -1;
};
int launch_add_norm(const NormArgs& n, cudaStream_t stream);
// One row per sequence of a [T, row_bytes] matrix, the first (last = 0: the CLS token) or the
// last one (last = 1), packed into [B, row_bytes] (scatter = 0) or written back from it
// (scatter = 1).  row_bytes is a multiple of 16.
int launch_first_rows(const void* src, void* dst, const int* cu_seqlens, int B, int row_bytes, int scatter,
                      int last, cudaStream_t stream);
// LayerNorm with bias over whole q rows and whole k rows (width H, stride ld), in place.
int launch_layernorm_qk(void* q, void* k, int ld, const void* gq, const void* bq, const void* gk,
                        const void* bk, int T, int H, float eps, int dtype, cudaStream_t stream);
// LayerNorm without bias over fp32 rows, in place.
int launch_layernorm_rows_f32(float* x, const void* gamma, int rows, int H, float eps, int dtype,
                              cudaStream_t stream);

struct RopeArgs {
  void* q;               // rows of n_heads*head_dim at stride ld_q
  void* k;               // rows of n_kv_heads*head_dim at stride ld_k
  const int* pos_ids;    // [T]
  const float* cos_tab;  // [max_pos, head_dim/2] fp32
  const float* sin_tab;
  const void* q_gamma;   // per-head RMSNorm weight [head_dim] or nullptr
  const void* k_gamma;
  int T, n_heads, n_kv_heads, head_dim, ld_q, ld_k;
  float eps;
  int dtype;
};
// Optional per-head RMSNorm followed by half-rotation RoPE, in place on q and k.
int launch_qk_norm_rope(const RopeArgs& r, cudaStream_t stream);

struct PoolArgs {
  const void* x;           // [T, H]
  const int* cu_seqlens;   // [n_seqs + 1]
  const int* seq_index;    // [n_out] batch positions to pool
  float* out;              // [n_out, H] fp32
  int n_out, H;
  int mode;                // 0 cls, 1 mean, 2 max (SPLADE), 3 last token
  int normalize;           // 1 -> L2-normalise each output row
  int dtype;
};
int launch_pool(const PoolArgs& p, cudaStream_t stream);

// In-place L2 normalisation of fp32 rows of width H.
int launch_l2_normalise(float* x, int rows, int H, cudaStream_t stream);

// Copies the token rows of the listed sequences, in order, to fp32.
int launch_gather_rows_f32(const void* x, const int* row_index, float* out, int n_rows, int H,
                           int dtype, cudaStream_t stream);

// Small dense head on pooled fp32 rows: out[r, n] = act(sum_k in[r,k] * w[n,k] + b[n]).
int launch_head_linear(const float* in, const void* w, const void* b, float* out, int rows, int N,
                       int K, int act, int dtype, cudaStream_t stream);

// Mixture-of-experts feed-forward of NomicBERT (backends/candle/src/models/nomic.rs:205-394),
// without a host round trip: the router's logits stay on the device, every expert gets a
// fixed-capacity segment of `cap` rows in the gathered buffers, and the expert GEMMs read their
// row count from `counts` (GemmArgs::m_dev).
//   route:   fp32 softmax over the E logits of a token, the k largest probabilities (ties: the
//            lower expert index), rounded to the model dtype as the reference does; for each
//            pick the expert, the weight and the row it takes in that expert's segment.
//   gather:  xg[(e * cap + pos) * H ..] = x[t] for every (token, pick).
//   combine: out[t] = sum over the picks of w * yg[e * cap + pos] + bias, accumulated in fp32.
int launch_moe_route(const void* logits, int ld_logits, int T, int E, int k, int* topk_e, float* topk_w,
                     int* pos, int* counts, int dtype, cudaStream_t stream);
int launch_moe_gather(const void* x, const int* topk_e, const int* pos, void* xg, int T, int k, int H,
                      long long cap, int dtype, cudaStream_t stream);
int launch_moe_combine(const void* yg, const int* topk_e, const float* topk_w, const int* pos,
                       const void* bias, void* out, int T, int k, int H, long long cap, int dtype,
                       cudaStream_t stream);

// Self-test of the failure path (selftest.cu): a kernel that only writes `code` to *status, as a
// kernel whose bounded wait ran out would, and a one-CTA kernel whose wait on a barrier nobody
// arrives at gives up after `limit` (<= 4096) probes and reports DEV_TIMEOUT_PRODUCER.
int launch_report_status(int* status, int code, cudaStream_t stream);
int launch_bounded_wait_probe(int* status, int limit, int* gave_up, cudaStream_t stream);

// Element-wise dtype conversion used at weight-load time.  src_kind: 0 fp32, 1 fp16, 2 bf16;
// dst dtype: DT_F16 / DT_BF16, or 2 for fp32.
int launch_convert(const void* src, int src_kind, void* dst, int dst_kind, size_t n,
                   cudaStream_t stream);

}  // namespace tei
