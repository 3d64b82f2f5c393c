// extern "C" wrappers of the kernel launchers (declared in include/tei_b200_ops.h).
#include "../../include/tei_b200_ops.h"

#include "kernels.h"

using namespace tei;

extern "C" {

int tei_b200_gemm_tiling(int M, int N, int sms, int narrow_ok) {
  if (M <= 0 || N <= 0 || sms <= 0) return -1;
  return tei::gemm_tiling(M, N, sms, narrow_ok != 0);
}

int tei_b200_op_linear(const void* a_dev, const void* w_dev, const void* bias_dev,
                       const void* residual_dev, void* out_dev, int M, int N, int K, int lda,
                       int ldo, int ldr, int act, int dtype, int* status_dev, void* stream) {
  GemmArgs g;
  g.a = a_dev;
  g.w = w_dev;
  g.bias = bias_dev;
  g.residual = residual_dev;
  g.out = out_dev;
  g.M = M;
  g.N = N;
  g.K = K;
  g.lda = lda;
  g.ldo = ldo;
  g.ldr = ldr;
  g.act = act;
  g.dtype = dtype;
  g.status = status_dev;
  return launch_gemm(g, static_cast<cudaStream_t>(stream));
}

int tei_b200_attention_plan(const int32_t* cu_seqlens_host, int n_seqs, int causal,
                            int32_t* work_out, int capacity_items) {
  return plan_attention(cu_seqlens_host, n_seqs, causal, work_out, capacity_items);
}

int tei_b200_attention_plan_windowed(const int32_t* cu_seqlens_host, int n_seqs, int causal,
                                     int window_left, int window_right, int32_t* work_out,
                                     int capacity_items) {
  return plan_attention(cu_seqlens_host, n_seqs, causal, work_out, capacity_items, window_left,
                        window_right);
}

int tei_b200_op_attention(const void* q_dev, const void* k_dev, const void* v_dev, void* out_dev,
                          const int32_t* work_dev, int n_work, int total_tokens, int n_heads,
                          int n_kv_heads, int head_dim, int ld_q, int ld_k, int ld_v, int ld_o,
                          int causal, float softmax_scale, const float* alibi_slopes_dev,
                          int dtype, int* status_dev, void* stream) {
  return tei_b200_op_attention_windowed(q_dev, k_dev, v_dev, out_dev, work_dev, n_work, total_tokens,
                                        n_heads, n_kv_heads, head_dim, ld_q, ld_k, ld_v, ld_o, causal,
                                        -1, -1, softmax_scale, alibi_slopes_dev, dtype, status_dev,
                                        stream);
}

int tei_b200_op_attention_windowed(const void* q_dev, const void* k_dev, const void* v_dev,
                                   void* out_dev, const int32_t* work_dev, int n_work,
                                   int total_tokens, int n_heads, int n_kv_heads, int head_dim,
                                   int ld_q, int ld_k, int ld_v, int ld_o, int causal,
                                   int window_left, int window_right, float softmax_scale,
                                   const float* alibi_slopes_dev, int dtype, int* status_dev,
                                   void* stream) {
  AttnArgs a;
  a.window_left = window_left;
  a.window_right = window_right;
  a.q = q_dev;
  a.k = k_dev;
  a.v = v_dev;
  a.out = out_dev;
  a.cu_seqlens = nullptr;
  a.work_items = work_dev;
  a.n_work = n_work;
  a.total_tokens = total_tokens;
  a.n_heads = n_heads;
  a.n_kv_heads = n_kv_heads;
  a.head_dim = head_dim;
  a.ld_q = ld_q;
  a.ld_k = ld_k;
  a.ld_v = ld_v;
  a.ld_o = ld_o;
  a.causal = causal;
  a.scale = softmax_scale;
  a.alibi_slopes = alibi_slopes_dev;
  a.dtype = dtype;
  a.status = status_dev;
  return launch_attention(a, static_cast<cudaStream_t>(stream));
}

int tei_b200_op_embed_layernorm(const int32_t* ids_dev, const int32_t* type_ids_dev,
                                const int32_t* pos_ids_dev, const void* word_dev,
                                const void* type_dev, const void* pos_dev, const void* gamma_dev,
                                const void* beta_dev, void* out_dev, int n_tokens, int hidden,
                                float eps, int dtype, void* stream) {
  EmbedArgs e;
  e.ids = ids_dev;
  e.type_ids = type_ids_dev;
  e.pos_ids = pos_ids_dev;
  e.word = word_dev;
  e.type_tab = type_dev;
  e.pos_tab = pos_dev;
  e.gamma = gamma_dev;
  e.beta = beta_dev;
  e.out = out_dev;
  e.T = n_tokens;
  e.H = hidden;
  e.eps = eps;
  e.dtype = dtype;
  return launch_embed_layernorm(e, static_cast<cudaStream_t>(stream));
}

int tei_b200_op_add_norm(const void* x_dev, const void* residual_dev, const void* gamma_dev,
                         const void* beta_dev, void* out_dev, float* sum_out_dev, int n_tokens,
                         int hidden, float eps, int rms, int dtype, void* stream) {
  NormArgs n;
  n.x = x_dev;
  n.residual = residual_dev;
  n.gamma = gamma_dev;
  n.beta = beta_dev;
  n.out = out_dev;
  n.sum_out = sum_out_dev;
  n.T = n_tokens;
  n.H = hidden;
  n.eps = eps;
  n.rms = rms;
  n.dtype = dtype;
  return launch_add_norm(n, static_cast<cudaStream_t>(stream));
}

int tei_b200_op_qk_norm_rope(void* q_dev, void* k_dev, const int32_t* pos_ids_dev,
                             const float* cos_dev, const float* sin_dev, const void* q_gamma_dev,
                             const void* k_gamma_dev, int n_tokens, int n_heads, int n_kv_heads,
                             int head_dim, int ld_q, int ld_k, float eps, int dtype,
                             void* stream) {
  RopeArgs r;
  r.q = q_dev;
  r.k = k_dev;
  r.pos_ids = pos_ids_dev;
  r.cos_tab = cos_dev;
  r.sin_tab = sin_dev;
  r.q_gamma = q_gamma_dev;
  r.k_gamma = k_gamma_dev;
  r.T = n_tokens;
  r.n_heads = n_heads;
  r.n_kv_heads = n_kv_heads;
  r.head_dim = head_dim;
  r.ld_q = ld_q;
  r.ld_k = ld_k;
  r.eps = eps;
  r.dtype = dtype;
  return launch_qk_norm_rope(r, static_cast<cudaStream_t>(stream));
}

int tei_b200_op_pool(const void* x_dev, const int32_t* cu_seqlens_dev,
                     const int32_t* seq_index_dev, float* out_dev, int n_out, int hidden, int mode,
                     int normalize, int dtype, void* stream) {
  PoolArgs p;
  p.x = x_dev;
  p.cu_seqlens = cu_seqlens_dev;
  p.seq_index = seq_index_dev;
  p.out = out_dev;
  p.n_out = n_out;
  p.H = hidden;
  p.mode = mode;
  p.normalize = normalize;
  p.dtype = dtype;
  return launch_pool(p, static_cast<cudaStream_t>(stream));
}

int tei_b200_op_gather_rows_f32(const void* x_dev, const int32_t* row_index_dev, float* out_dev,
                                int n_rows, int hidden, int dtype, void* stream) {
  return launch_gather_rows_f32(x_dev, row_index_dev, out_dev, n_rows, hidden, dtype,
                                static_cast<cudaStream_t>(stream));
}

int tei_b200_op_head_linear(const float* in_dev, const void* w_dev, const void* b_dev,
                            float* out_dev, int rows, int N, int K, int act, int dtype,
                            void* stream) {
  return launch_head_linear(in_dev, w_dev, b_dev, out_dev, rows, N, K, act, dtype,
                            static_cast<cudaStream_t>(stream));
}

int tei_b200_op_linear_rows_dev(const void* a_dev, const void* w_dev, const void* bias_dev,
                                void* out_dev, int M, int N, int K, int lda, int ldo, int act,
                                int dtype, const int32_t* m_rows_dev, int* status_dev, void* stream) {
  GemmArgs g;
  g.a = a_dev;
  g.w = w_dev;
  g.bias = bias_dev;
  g.residual = nullptr;
  g.out = out_dev;
  g.M = M;
  g.N = N;
  g.K = K;
  g.lda = lda;
  g.ldo = ldo;
  g.ldr = 0;
  g.act = act;
  g.dtype = dtype;
  g.status = status_dev;
  g.m_dev = m_rows_dev;
  return launch_gemm(g, static_cast<cudaStream_t>(stream));
}

int tei_b200_op_moe_route(const void* logits_dev, int ld_logits, int n_tokens, int n_experts,
                          int top_k, int32_t* topk_expert_dev, float* topk_weight_dev,
                          int32_t* pos_dev, int32_t* counts_dev, int dtype, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (n_experts <= 0 || n_experts > 64) return static_cast<int>(cudaErrorInvalidValue);
  cudaError_t e = cudaMemsetAsync(counts_dev, 0, static_cast<size_t>(n_experts) * 4, st);
  if (e != cudaSuccess) return static_cast<int>(e);
  return launch_moe_route(logits_dev, ld_logits, n_tokens, n_experts, top_k, topk_expert_dev,
                          topk_weight_dev, pos_dev, counts_dev, dtype, st);
}

int tei_b200_op_moe_gather(const void* x_dev, const int32_t* topk_expert_dev, const int32_t* pos_dev,
                           void* xg_dev, int n_tokens, int top_k, int hidden, long long cap,
                           int dtype, void* stream) {
  return launch_moe_gather(x_dev, topk_expert_dev, pos_dev, xg_dev, n_tokens, top_k, hidden, cap, dtype,
                           static_cast<cudaStream_t>(stream));
}

int tei_b200_op_moe_combine(const void* yg_dev, const int32_t* topk_expert_dev,
                            const float* topk_weight_dev, const int32_t* pos_dev,
                            const void* bias_dev, void* out_dev, int n_tokens, int top_k, int hidden,
                            long long cap, int dtype, void* stream) {
  return launch_moe_combine(yg_dev, topk_expert_dev, topk_weight_dev, pos_dev, bias_dev, out_dev, n_tokens,
                            top_k, hidden, cap, dtype, static_cast<cudaStream_t>(stream));
}

int tei_b200_op_linear_rope(const void* a_dev, const void* w_dev, const void* bias_dev, void* out_dev, int M,
                            int N, int K, int lda, int ldo, const int32_t* pos_ids_dev, const float* cos_dev,
                            const float* sin_dev, const void* q_gamma_dev, const void* k_gamma_dev,
                            int head_dim, int q_cols, int k_cols, float eps, int dtype, int* status_dev,
                            void* stream) {
  RopeFusion r;
  r.pos_ids = pos_ids_dev;
  r.cos_tab = cos_dev;
  r.sin_tab = sin_dev;
  r.q_gamma = q_gamma_dev;
  r.k_gamma = k_gamma_dev;
  r.head_dim = head_dim;
  r.q_cols = q_cols;
  r.k_cols = k_cols;
  r.eps = eps;
  GemmArgs g;
  g.a = a_dev;
  g.w = w_dev;
  g.bias = bias_dev;
  g.residual = nullptr;
  g.out = out_dev;
  g.M = M;
  g.N = N;
  g.K = K;
  g.lda = lda;
  g.ldo = ldo;
  g.ldr = 0;
  g.act = ACT_NONE;
  g.dtype = dtype;
  g.status = status_dev;
  g.rope = &r;
  return launch_gemm(g, static_cast<cudaStream_t>(stream));
}

int tei_b200_op_bounded_wait_probe(int* status_dev, int limit, int* gave_up_dev, void* stream) {
  return launch_bounded_wait_probe(status_dev, limit, gave_up_dev, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
