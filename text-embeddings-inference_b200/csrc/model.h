// One GPU replica of an encoder model: parsed config, device weights, workspace and the forward.
//
// Host-side counterpart of the reference's CandleBackend + Flash*Model
// (backends/candle/src/lib.rs:163-577, models/flash_bert.rs, flash_nomic.rs, flash_qwen3.rs):
// config.json -> architecture dispatch, safetensors -> fused device weights, packed Batch ->
// kernel sequence -> pooled / raw / score rows.
#pragma once
#include <cstddef>
#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include <cuda_runtime.h>

#include "json.h"
#include "safetensors.h"

namespace tei {

// The compute capability this library is built for (sm_100a), in the reference's notation
// (major * 10 + minor; backends/candle/src/compute_cap.rs:8-12).
constexpr int kCompileComputeCap = 100;
// Whether a binary built for `compile_cap` may run on a device of `runtime_cap`: the rule of
// backends/candle/src/compute_cap.rs:27-40, which `create` applies like lib.rs:240-248 does.
bool compute_cap_matching(int runtime_cap, int compile_cap);


struct RopeArgs;

// Error kinds that map onto the reference's BackendError (backends/core/src/lib.rs:84-95).
enum ErrKind : int {
  ERR_OK = 0,
  ERR_START = 1,
  ERR_INFERENCE = 2,
  ERR_UNHEALTHY = 3,
  ERR_WEIGHTS_NOT_FOUND = 4,
  ERR_TIMEOUT = 5,
};

struct TeiError : std::runtime_error {
  int kind;
  TeiError(int k, const std::string& m) : std::runtime_error(m), kind(k) {}
};

enum Arch { ARCH_BERT = 0, ARCH_NOMIC = 1, ARCH_QWEN3 = 2 };
// Kernel classes of the per-class device timing.
enum KernelClass { KC_EMBED = 0, KC_GEMM = 1, KC_ATTENTION = 2, KC_NORM = 3, KC_ROPE = 4, KC_POOL = 5, KC_COUNT = 6 };
enum PoolMode { POOL_CLS = 0, POOL_MEAN = 1, POOL_SPLADE = 2, POOL_LAST = 3 };

struct ModelSpec {
  Arch arch = ARCH_BERT;
  std::string model_type;
  bool roberta = false;
  bool gte = false;        // GTE ("new"): post-LN blocks with RoPE and a gated feed-forward (models/flash_gte.rs)
  float rope_ntk_factor = 0.f;  // RopeScaling::Ntk (layers/rotary.rs:86-93), 0: none
  // RopeScaling::Llama3 (layers/rotary.rs:46-85), factor 0: none
  float rope_l3_factor = 0.f, rope_l3_high = 0.f, rope_l3_low = 0.f, rope_l3_orig_max = 0.f;
  bool distil = false;     // DistilBERT: no token types, its own tensor names (models/flash_distilbert.rs)
  // What the router adds to every position id (router/src/lib.rs:184-192): pad_token_id + 1 for
  // model_type roberta / xlm-roberta / camembert, else 0.
  int position_offset = 0;
  bool jina = false;       // JinaBERT: gated feed-forward, optional ALiBi (models/flash_jina.rs)
  // JinaCodeBert (models/flash_jina_code.rs): LayerNorm on q and k, a second LayerNorm with the
  // layer's input as residual before the feed-forward, gate in the second half of the rows
  bool jina_code = false;
  bool alibi = false;      // ALiBi slopes instead of a position table
  int hidden = 0, layers = 0, heads = 0, kv_heads = 0, head_dim = 0, inter = 0;
  int vocab = 0, max_pos = 0, type_vocab = 0;
  float eps = 1e-12f;
  int act = 0;             // Act of the feed-forward
  bool gated = false;      // SwiGLU feed-forward
  bool qkv_bias = false, out_bias = false, fc1_bias = false, fc2_bias = false;
  bool causal = false;
  bool qk_norm = false;    // per-head RMSNorm on q and k before RoPE (Qwen3)
  int window_left = -1;    // sliding window of the decoder families (Mistral), -1: none
  // ModernBERT (models/flash_modernbert.rs): pre-LayerNorm blocks without biases on the norms,
  // LayerNorm after the embedding, every `global_every`-th layer attends globally with
  // rope_theta, the others within `local_window` keys on each side with `local_theta`.
  // NomicBERT mixture of experts (models/nomic.rs:205-421): layers with index % moe_every == 1
  // route every token to moe_top_k of num_experts feed-forwards.
  int moe_every = 0, num_experts = 0, moe_top_k = 0;
  bool modernbert = false;
  int global_every = 0, local_window = -1;
  float local_theta = 0.f;
  int head_act = 0;        // activation of the classification head's dense layer
  int cls_pool = POOL_CLS; // pooling in front of the classification head
  bool rope = false;
  float rope_theta = 10000.f;
  float rope_scaling_factor = 0.f;  // NomicBERT dynamic table switch (flash_nomic.rs:244-258)
  int rope_table_len = 0;           // rows of the cos / sin tables
  int nomic_max_pos = 0;            // max_position_embeddings used by that switch
  bool classifier = false;
  int n_classes = 0;
  int pool = POOL_CLS;
  int dtype = 0;  // DType

  int q_width() const { return heads * head_dim; }
  int kv_width() const { return kv_heads * head_dim; }
  int qkv_width() const { return q_width() + 2 * kv_width(); }
};

// Parses config.json the way backends/candle/src/lib.rs:124-154 + the per-model config structs
// do (models/bert.rs:11-30, nomic.rs:11-55, qwen3.rs:13-37).  model_type_flag: 0 classifier,
// 1 embedding.  Throws TeiError(ERR_START).
ModelSpec parse_model_spec(const Json& config, int model_type_flag, int pool, int dtype);

// The view of a packed batch the forward consumes (host pointers, borrowed).
struct HostBatch {
  const uint32_t* input_ids = nullptr;
  const uint32_t* token_type_ids = nullptr;
  const uint32_t* position_ids = nullptr;
  size_t n_tokens = 0;
  const uint32_t* cu_seqlens = nullptr;
  size_t n_seqs = 0;
  uint32_t max_length = 0;
  const uint32_t* pooled_indices = nullptr;
  size_t n_pooled = 0;
  const uint32_t* raw_indices = nullptr;
  size_t n_raw = 0;
};

struct ReplicaStats {
  double last_gpu_ms = 0.0;      // device time of the last forward (CUDA events)
  double last_h2d_bytes = 0.0;
  double last_d2h_bytes = 0.0;
  double last_launches = 0.0;    // kernels launched by the last forward
  double last_tokens = 0.0;
  double total_tokens = 0.0;
  double total_gpu_ms = 0.0;
  double calls = 0.0;
};

class Replica {
 public:
  Replica(int device, const ModelSpec& spec, const SafeTensors& st);
  ~Replica();
  Replica(const Replica&) = delete;
  Replica& operator=(const Replica&) = delete;

  const ModelSpec& spec() const { return spec_; }
  int device() const { return device_; }
  int output_dim() const;  // width of a pooled row (after the Dense modules, if any)
  int raw_dim() const;     // width of a raw (per-token) row

  // Appends a Sentence-Transformers Dense module (backends/candle/src/models/dense.rs:26-75,
  // loaded as in backends/candle/src/lib.rs:579-629): `<dir>/config.json` + `<dir>/model.safetensors`
  // with `linear.weight` [out, in] and optional `linear.bias`.  Modules run on the pooled rows in
  // the order they were added.  Throws TeiError(ERR_START).
  void add_dense(const std::string& dir);
  size_t dense_count() const { return dense_.size(); }

  // Validates the batch (throws TeiError(ERR_INFERENCE)), copies it to pinned memory and
  // enqueues the single host-to-device copy.  `predict` selects the classifier path (CLS rows of
  // every sequence -> head -> scores).
  void stage(const HostBatch& b, bool predict, bool normalize);
  // Enqueues the forward of the staged batch.
  void run();
  // Enqueues the device-to-host copy, waits, checks the device status word and copies the rows
  // to the caller's buffers (any of which may be null when the matching count is zero).
  void fetch(float* pooled_out, float* raw_out, float* scores_out);
  // Waits for everything enqueued so far and checks the device status word.
  void sync_and_check();

  // Per-kernel-class timing: when on, every launch is bracketed by a pair of events on the
  // launching stream (up to kMaxPairs launches between two synchronisations).
  void set_profiling(bool on);
  int kernel_times(double* ms, double* launches, int n) const;
  // Runs the staged forward `steps` times back to back and returns the device time of the whole
  // sequence, measured with events on the launching stream.
  double timed_runs(int steps);

  // The last-layer shortcut (on by default): when only one row per sequence leaves the model,
  // everything behind the last layer's scores runs on those rows alone.  Off: every row is
  // computed, as the reference does.  Takes effect with the next stage().
  void set_last_layer_shortcut(bool on) { last_layer_shortcut_ = on; }

  // RoPE (and the q/k RMSNorm) in the epilogue of the q/k/v projection (1), as a kernel of its own
  // behind it (0), or whichever is faster for the model (-1, the default: fused unless the model
  // has a q/k RMSNorm).  Same results bit for bit; takes effect with the next run().
  void set_fused_rope(int mode) { fused_rope_ = mode; }

  // The residual of the post-LN feed-forward added in the epilogue of its output projection (on;
  // only where the projection's K loop is long enough to hide it) or by the LayerNorm kernel
  // behind it (off, the default: the reference's form, layer_norm.rs with a residual).  Measured
  // on the 68,576-token BERT-base batch the two are level: the LayerNorm launches get 0.09 ms
  // shorter per forward, the projections 0.03 to 0.2 ms longer.  Takes effect with the next run().
  void set_fused_residual(bool on) { fused_residual_ = on; }

  // Self-test hook: the next run() ends with a kernel that writes `code` to the status word,
  // exactly what a kernel whose bounded wait ran out leaves behind.  One shot.
  void report_status_once(int code) { inject_status_ = code; }

  const ReplicaStats& stats() const { return stats_; }
  cudaStream_t stream() const { return stream_; }
  // Device pointers of the last outputs (valid until the next stage()).
  const float* pooled_dev() const { return d_pooled_; }
  size_t staged_tokens() const { return T_; }

 private:
  struct LayerW {
    void *wqkv = nullptr, *bqkv = nullptr, *wo = nullptr, *bo = nullptr;
    void *ln1_g = nullptr, *ln1_b = nullptr, *ln2_g = nullptr, *ln2_b = nullptr;
    void *w1 = nullptr, *b1 = nullptr, *w2 = nullptr, *b2 = nullptr;
    void *q_norm = nullptr, *k_norm = nullptr;
    // JinaCodeBert: LayerNorm of q, of k, and `layer_norm_1`
    void *lnq_g = nullptr, *lnq_b = nullptr, *lnk_g = nullptr, *lnk_b = nullptr;
    void *lnm_g = nullptr, *lnm_b = nullptr;
    // mixture-of-experts layers: router [E_pad, H], w1 [E*I, H], w2 transposed per expert
    // [E*H, I], bias [H]
    void *moe_router = nullptr, *moe_w1 = nullptr, *moe_w2t = nullptr, *moe_bias = nullptr;
  };

  struct DenseW {
    void* w = nullptr;
    void* b = nullptr;
    int in = 0, out = 0;
    int act = 0;  // ACT_NONE or ACT_TANH
  };

  void load_weights(const SafeTensors& st);
  void load_bert(const SafeTensors& st);
  void load_nomic(const SafeTensors& st);
  void load_qwen3(const SafeTensors& st);
  void load_modernbert(const SafeTensors& st);
  void load_gte(const SafeTensors& st);
  void build_rope_tables();
  void* dev_alloc(size_t bytes);
  // Converts `src` (any float dtype) into the model dtype at dst + dst_elem_off elements.
  void upload(void* dst, size_t dst_elem_off, const StTensor& src, int dst_kind = -1);
  void* upload_new(const StTensor& src, int dst_kind = -1);
  void upload_rows_interleaved(void* dst, const StTensor& gate, const StTensor& up);
  void ensure_workspace(size_t tokens, size_t seqs, size_t n_work, size_t n_pooled,
                        size_t raw_rows);
  void qkv_projection(const void* x, const LayerW& L, int T, int W, int H, const RopeArgs& r, int* status);
  void forward_bert();
  void forward_nomic();
  void forward_qwen3();
  void pool_and_heads();
  void launch(int rc, const char* what);
  void prof_begin();
  void prof_end(int cls);
  void prof_drain();
  size_t esize() const { return 2; }

  int device_;
  ModelSpec spec_;
  cudaStream_t stream_ = nullptr;
  cudaEvent_t ev_start_ = nullptr, ev_stop_ = nullptr;
  std::vector<void*> allocs_;
  ReplicaStats stats_;
  int launches_ = 0;
  static constexpr int kMaxPairs = 8192;
  bool profiling_ = false;
  std::vector<cudaEvent_t> ev_pool_;
  std::vector<int> pair_cls_;
  int n_pairs_ = 0;
  double class_ms_[KC_COUNT] = {0, 0, 0, 0, 0, 0};
  double class_launches_[KC_COUNT] = {0, 0, 0, 0, 0, 0};

  // weights
  void *word_ = nullptr, *pos_tab_ = nullptr, *type_tab_ = nullptr, *emb_g_ = nullptr,
       *emb_b_ = nullptr;
  std::vector<LayerW> layers_;
  void* final_norm_ = nullptr;
  void* projection_ = nullptr;  // optional Qwen3 `linear.weight`
  int projection_dim_ = 0;
  float *cos_ = nullptr, *sin_ = nullptr, *cos_scaled_ = nullptr, *sin_scaled_ = nullptr;
  float* alibi_slopes_ = nullptr;  // [heads], fp32 (alibi.rs:18-47)
  // classification heads
  void *cls_dense_w_ = nullptr, *cls_dense_b_ = nullptr, *cls_out_w_ = nullptr,
       *cls_out_b_ = nullptr, *cls_norm_g_ = nullptr;
  std::vector<DenseW> dense_;
  // SPLADE head
  void *sp_dense_w_ = nullptr, *sp_dense_b_ = nullptr, *sp_ln_g_ = nullptr, *sp_ln_b_ = nullptr,
       *sp_dec_w_ = nullptr, *sp_dec_b_ = nullptr;
  int sp_act_ = 0;
  // temporary device staging used while loading
  void* load_stage_ = nullptr;
  size_t load_stage_bytes_ = 0;

  // workspace (one arena, carved in ensure_workspace)
  void* arena_ = nullptr;
  size_t arena_bytes_ = 0;
  size_t cap_tokens_ = 0, cap_seqs_ = 0, cap_work_ = 0, cap_pooled_ = 0, cap_raw_rows_ = 0;
  int32_t* d_ints_ = nullptr;   // ids | types | pos | cu | pooled idx | raw row idx | work items
  int32_t* h_ints_ = nullptr;   // pinned mirror
  size_t ints_cap_ = 0;
  void *x_ = nullptr, *x1_ = nullptr, *qkv_ = nullptr, *attn_ = nullptr, *tmp_ = nullptr,
       *ffn_ = nullptr;
  float* resid_ = nullptr;
  // mixture-of-experts scratch: gathered inputs / hidden / outputs with `moe_cap_` rows per expert
  void *moe_xg_ = nullptr, *moe_hg_ = nullptr, *moe_yg_ = nullptr, *moe_logits_ = nullptr;
  int *moe_topk_e_ = nullptr, *moe_pos_ = nullptr, *moe_counts_ = nullptr;
  float* moe_topk_w_ = nullptr;
  size_t moe_cap_ = 0;
  void* splade_ = nullptr;
  float* d_out_ = nullptr;      // status word (as int) | pooled | raw | scores
  float* h_out_ = nullptr;      // pinned mirror
  size_t out_cap_floats_ = 0;
  float *d_pooled_ = nullptr, *d_raw_ = nullptr, *d_scores_ = nullptr, *d_cls_ = nullptr,
        *d_head_tmp_ = nullptr, *d_dense_a_ = nullptr, *d_dense_b_ = nullptr;
  size_t pooled_ld_ = 0;        // floats between pooled rows in the output block

  // staged batch
  size_t T_ = 0, B_ = 0, n_work_ = 0, n_pooled_ = 0, n_raw_rows_ = 0;
  uint32_t max_length_ = 0;
  bool predict_ = false, normalize_ = false;
  int32_t *d_ids_ = nullptr, *d_types_ = nullptr, *d_pos_ = nullptr, *d_cu_ = nullptr,
          *d_pooled_idx_ = nullptr, *d_raw_rows_ = nullptr, *d_work_ = nullptr, *d_all_idx_ = nullptr,
          *d_work_local_ = nullptr;  // work list of the layers with the two-sided local window
  // When only the first row of every sequence leaves the model (CLS pooling or a classifier head,
  // no raw rows), the last layer needs its keys and values for every token but everything after
  // the scores only for that row: a work list with just the first query tile of every sequence.
  int32_t* d_work_first_ = nullptr;
  size_t n_work_first_ = 0;
  bool first_rows_only_ = false;
  bool last_layer_shortcut_ = true;
  int fused_rope_ = -1;
  bool fused_residual_ = false;
  int inject_status_ = 0;
  size_t out_floats_ = 0;
};

}  // namespace tei
