#include "model.h"

#include <cstdlib>

#include "kernels.h"
#include "plan.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>

namespace tei {
namespace {

#define TEI_CUDA(expr)                                                                      \
  do {                                                                                      \
    cudaError_t e__ = (expr);                                                               \
    if (e__ != cudaSuccess) {                                                               \
      throw TeiError(ERR_INFERENCE, std::string(#expr) + ": " + cudaGetErrorString(e__));   \
    }                                                                                       \
  } while (0)

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Brackets one kernel launch with a pair of events when per-class timing is switched on.
#define LAUNCH(cls, call, what) \
  do {                          \
    prof_begin();               \
    launch((call), what);       \
    prof_end(cls);              \
  } while (0)

int parse_act(const std::string& s) {
  // layers/linear.rs:5-17: every GELU spelling means the tanh approximation.
  if (s == "gelu" || s == "gelu_new" || s == "gelu_pytorch_tanh") return ACT_GELU;
  if (s == "relu") return ACT_RELU;
  if (s == "tanh") return ACT_TANH;
  if (s == "swiglu") return ACT_SWIGLU;
  if (s == "silu") return -2;
  return -1;
}

int64_t need_int(const Json& c, const char* key) {
  if (!c[key].is_number()) throw TeiError(ERR_START, std::string("config.json: missing field `") + key + "`");
  return c[key].as_int();
}
double need_double(const Json& c, const char* key) {
  if (!c[key].is_number()) throw TeiError(ERR_START, std::string("config.json: missing field `") + key + "`");
  return c[key].as_double();
}
std::string need_string(const Json& c, const char* key) {
  if (!c[key].is_string()) throw TeiError(ERR_START, std::string("config.json: missing field `") + key + "`");
  return c[key].as_string();
}
bool need_bool(const Json& c, const char* key) {
  if (!c[key].is_bool()) throw TeiError(ERR_START, std::string("config.json: missing field `") + key + "`");
  return c[key].as_bool();
}

}  // namespace

ModelSpec parse_model_spec(const Json& c, int model_type_flag, int pool, int dtype) {
  ModelSpec s;
  s.dtype = dtype;
  s.model_type = need_string(c, "model_type");
  s.classifier = (model_type_flag == 0);
  s.pool = s.classifier ? POOL_CLS : pool;  // classifiers always pool CLS (flash_bert.rs:247-249)
  const std::string& mt = s.model_type;
  if (mt == "bert" || mt == "roberta" || mt == "xlm-roberta" || mt == "camembert") {
    s.arch = ARCH_BERT;
    s.roberta = mt != "bert";
    if (s.roberta) s.position_offset = static_cast<int>(c.get_int("pad_token_id", 0)) + 1;
    s.vocab = static_cast<int>(need_int(c, "vocab_size"));
    s.hidden = static_cast<int>(need_int(c, "hidden_size"));
    s.layers = static_cast<int>(need_int(c, "num_hidden_layers"));
    s.heads = static_cast<int>(need_int(c, "num_attention_heads"));
    s.inter = static_cast<int>(need_int(c, "intermediate_size"));
    s.max_pos = static_cast<int>(need_int(c, "max_position_embeddings"));
    s.type_vocab = static_cast<int>(need_int(c, "type_vocab_size"));
    s.eps = static_cast<float>(need_double(c, "layer_norm_eps"));
    // BertConfigWrapper (backends/candle/src/lib.rs:83-121): `_name_or_path` or
    // `auto_map.AutoConfig` select the JinaBERT implementations for model_type "bert".
    const std::string name_or_path = c.get_string("_name_or_path", "");
    const std::string auto_config = c["auto_map"].is_object() ? c["auto_map"].get_string("AutoConfig", "") : "";
    const std::string pos_type = c.get_string("position_embedding_type", "absolute");
    if (mt == "bert" && (name_or_path == "jinaai/jina-bert-implementation" ||
                         auto_config.find("jinaai/jina-bert-implementation") != std::string::npos)) {
      s.jina = true;
      if (pos_type == "alibi") s.alibi = true;
      else if (pos_type != "absolute") throw TeiError(ERR_START, "not supported");  // flash_jina.rs:243
      if (s.pool == POOL_SPLADE) throw TeiError(ERR_START, "`splade` is not supported for Jina");
    } else if (mt == "bert" && (name_or_path == "jinaai/jina-bert-v2-qk-post-norm" ||
                                auto_config.find("jinaai/jina-bert-v2-qk-post-norm") != std::string::npos)) {
      s.jina = s.jina_code = true;
      if (pos_type == "alibi") s.alibi = true;
      else if (pos_type != "absolute") throw TeiError(ERR_START, "not supported");  // flash_jina_code.rs:296
      if (s.classifier) throw TeiError(ERR_START, "`classifier` model type is not supported for Jina Code");
      if (s.pool == POOL_SPLADE) throw TeiError(ERR_START, "`splade` is not supported for Jina Code");
    } else if (pos_type != "absolute") {
      throw TeiError(ERR_START, "FlashBert only supports absolute position embeddings");
    }
    s.act = parse_act(need_string(c, "hidden_act"));
    if (s.jina) {
      // gated feed-forward: act(first half) * second half (flash_jina.rs:177-182)
      if (s.act != ACT_GELU) throw TeiError(ERR_START, "unsupported hidden_act for the JinaBERT feed-forward");
      s.gated = true;
      s.act = ACT_GEGLU;
    } else if (s.act != ACT_GELU && s.act != ACT_RELU && s.act != ACT_TANH) {
      throw TeiError(ERR_START, "unsupported hidden_act for a BERT feed-forward");
    }
    if (s.heads <= 0 || s.hidden % s.heads != 0) throw TeiError(ERR_START, "hidden_size is not a multiple of num_attention_heads");
    s.kv_heads = s.heads;
    s.head_dim = s.hidden / s.heads;
    s.qkv_bias = s.out_bias = s.fc1_bias = s.fc2_bias = true;
    if (s.jina) s.fc1_bias = false;
    if (s.classifier) {
      if (!c["id2label"].is_object()) throw TeiError(ERR_START, "`id2label` must be set for classifier models");
      s.n_classes = static_cast<int>(c["id2label"].size());
    }
  } else if (mt == "distilbert") {
    // DistilBertConfig (models/distilbert.rs:9-21); BERT blocks without token types and with a
    // fixed LayerNorm epsilon of 1e-12 (flash_distilbert.rs:113-115).
    s.arch = ARCH_BERT;
    s.distil = true;
    if (s.classifier) throw TeiError(ERR_START, "`classifier` model type is not supported for DistilBert");
    if (s.pool == POOL_SPLADE) throw TeiError(ERR_START, "`splade` for DistilBert is outside this backend");
    s.vocab = static_cast<int>(need_int(c, "vocab_size"));
    s.hidden = static_cast<int>(need_int(c, "dim"));
    s.layers = static_cast<int>(need_int(c, "n_layers"));
    s.heads = s.kv_heads = static_cast<int>(need_int(c, "n_heads"));
    s.inter = static_cast<int>(need_int(c, "hidden_dim"));
    s.max_pos = static_cast<int>(need_int(c, "max_position_embeddings"));
    s.type_vocab = 0;
    s.eps = 1e-12f;
    s.act = parse_act(need_string(c, "activation"));
    if (s.act != ACT_GELU && s.act != ACT_RELU) throw TeiError(ERR_START, "unsupported activation for DistilBert");
    if (s.heads <= 0 || s.hidden % s.heads != 0) throw TeiError(ERR_START, "dim is not a multiple of n_heads");
    s.head_dim = s.hidden / s.heads;
    s.qkv_bias = s.out_bias = s.fc1_bias = s.fc2_bias = true;
  } else if (mt == "gte" || mt == "new") {
    // GTEConfig (models/gte.rs:14-36); runs on the NomicBERT skeleton (post-LN, RoPE, gated FFN).
    s.arch = ARCH_NOMIC;
    s.gte = true;
    if (s.pool == POOL_SPLADE) throw TeiError(ERR_START, "`splade` is not supported for GTE");
    if (c.get_bool("logn_attention_clip1", false)) throw TeiError(ERR_START, "`logn_attention_clip1` is not supported");
    if (c.get_bool("logn_attention_scale", false)) throw TeiError(ERR_START, "`logn_attention_scale` is not supported");
    if (need_string(c, "position_embedding_type") != "rope") throw TeiError(ERR_START, "Only `PositionEmbeddingType::Rope` is supported");
    s.vocab = static_cast<int>(need_int(c, "vocab_size"));
    s.hidden = static_cast<int>(need_int(c, "hidden_size"));
    s.layers = static_cast<int>(need_int(c, "num_hidden_layers"));
    s.heads = s.kv_heads = static_cast<int>(need_int(c, "num_attention_heads"));
    s.inter = static_cast<int>(need_int(c, "intermediate_size"));
    s.max_pos = static_cast<int>(need_int(c, "max_position_embeddings"));
    s.type_vocab = static_cast<int>(need_int(c, "type_vocab_size"));
    s.eps = static_cast<float>(need_double(c, "layer_norm_eps"));
    if (parse_act(need_string(c, "hidden_act")) != ACT_GELU) throw TeiError(ERR_START, "GTE expects a GELU hidden_act");
    s.gated = true;
    s.act = ACT_GEGLU;  // act(second half) * first half (gte.rs:216-227)
    s.qkv_bias = s.out_bias = true;
    s.fc1_bias = false;
    s.fc2_bias = true;
    if (s.heads <= 0 || s.hidden % s.heads != 0) throw TeiError(ERR_START, "hidden_size is not a multiple of num_attention_heads");
    s.head_dim = s.hidden / s.heads;
    s.rope = true;
    if (c["rope_theta"].is_number()) s.rope_theta = static_cast<float>(c["rope_theta"].as_double());
    else if (c["rope_parameters"]["rope_theta"].is_number()) s.rope_theta = static_cast<float>(c["rope_parameters"]["rope_theta"].as_double());
    else throw TeiError(ERR_START, "Neither `rope_theta` nor `rope_parameters.rope_theta` are defined in the `config.json`");
    if (c["rope_scaling"].is_object()) {
      const std::string rt = c["rope_scaling"].get_string("type", c["rope_scaling"].get_string("rope_type", ""));
      if (rt != "ntk") throw TeiError(ERR_START, "only the `ntk` rope_scaling of GTE is supported");
      s.rope_ntk_factor = static_cast<float>(need_double(c["rope_scaling"], "factor"));
    }
    s.rope_table_len = s.max_pos;
    s.nomic_max_pos = s.max_pos;
    if (s.classifier) {
      if (!c["id2label"].is_object()) throw TeiError(ERR_START, "`id2label` must be set for classifier models");
      s.n_classes = static_cast<int>(c["id2label"].size());
    }
  } else if (mt == "nomic_bert") {
    s.arch = ARCH_NOMIC;
    if (s.classifier) throw TeiError(ERR_START, "`classifier` model type is not supported for Nomic");
    if (s.pool == POOL_SPLADE) throw TeiError(ERR_START, "`splade` is not supported for Nomic");
    const bool prenorm = need_bool(c, "prenorm");
    const double frac = need_double(c, "rotary_emb_fraction");
    const bool interleaved = need_bool(c, "rotary_emb_interleaved");
    s.type_vocab = static_cast<int>(need_int(c, "type_vocab_size"));
    if (prenorm || frac != 1.0 || interleaved || s.type_vocab <= 0) {
      throw TeiError(ERR_START, "config is not supported");  // NomicConfig::valid(), nomic.rs:49-54
    }
    s.moe_every = static_cast<int>(c.get_int("moe_every_n_layers", 0));
    if (s.moe_every > 0) {  // NomicRouter::load unwraps both (nomic.rs:213-215)
      s.num_experts = static_cast<int>(need_int(c, "num_experts"));
      s.moe_top_k = static_cast<int>(need_int(c, "moe_top_k"));
      if (s.num_experts < 1 || s.num_experts > 64 || s.moe_top_k < 1 || s.moe_top_k > 8 || s.moe_top_k > s.num_experts) {
        throw TeiError(ERR_START, "mixture of experts: up to 64 experts and a top-k of up to 8 are supported");
      }
    }
    s.vocab = static_cast<int>(need_int(c, "vocab_size"));
    s.hidden = static_cast<int>(need_int(c, "n_embd"));
    s.layers = static_cast<int>(need_int(c, "n_layer"));
    s.heads = static_cast<int>(need_int(c, "n_head"));
    s.inter = static_cast<int>(need_int(c, "n_inner"));
    s.eps = static_cast<float>(need_double(c, "layer_norm_epsilon"));
    s.qkv_bias = s.out_bias = need_bool(c, "qkv_proj_bias");
    s.fc1_bias = need_bool(c, "mlp_fc1_bias");
    s.fc2_bias = need_bool(c, "mlp_fc2_bias");
    const int act = parse_act(need_string(c, "activation_function"));
    if (act == ACT_SWIGLU) {
      s.gated = true;
      s.act = ACT_SWIGLU;
    } else if (act == ACT_GELU || act == ACT_RELU) {
      s.act = act;
    } else {
      throw TeiError(ERR_START, "unsupported activation_function for NomicBERT");
    }
    if (s.heads <= 0 || s.hidden % s.heads != 0) throw TeiError(ERR_START, "n_embd is not a multiple of n_head");
    s.kv_heads = s.heads;
    s.head_dim = s.hidden / s.heads;
    s.rope = true;
    s.rope_theta = static_cast<float>(need_double(c, "rotary_emb_base"));
    s.rope_table_len = static_cast<int>(need_int(c, "n_positions"));
    s.max_pos = s.rope_table_len;
    s.rope_scaling_factor = static_cast<float>(c.get_double("rotary_scaling_factor", 0.0));
    s.nomic_max_pos = static_cast<int>(
        c.get_int("max_position_embeddings", c.get_int("max_trained_positions", 2048)));
  } else if (mt == "qwen3" || mt == "qwen2" || mt == "mistral" || mt == "llama") {
    // One decoder skeleton (pre-RMSNorm, GQA, RoPE, SiLU-gated feed-forward) serves
    // flash_qwen3.rs, flash_qwen2.rs and flash_mistral.rs (Llama configs are run as Mistral,
    // backends/candle/src/lib.rs:549-575); the differences are flags.
    s.arch = ARCH_QWEN3;
    const std::string family = mt == "qwen3" ? "Qwen3" : mt == "qwen2" ? "Qwen2" : "Mistral";
    if (s.classifier) throw TeiError(ERR_START, "`classifier` model type is not supported for " + family);
    if (s.pool == POOL_SPLADE) throw TeiError(ERR_START, "`splade` is not supported for " + family);
    s.vocab = static_cast<int>(need_int(c, "vocab_size"));
    s.hidden = static_cast<int>(need_int(c, "hidden_size"));
    s.inter = static_cast<int>(need_int(c, "intermediate_size"));
    s.layers = static_cast<int>(need_int(c, "num_hidden_layers"));
    s.heads = static_cast<int>(need_int(c, "num_attention_heads"));
    s.kv_heads = static_cast<int>(need_int(c, "num_key_value_heads"));
    s.max_pos = static_cast<int>(need_int(c, "max_position_embeddings"));
    s.eps = static_cast<float>(need_double(c, "rms_norm_eps"));
    if (parse_act(need_string(c, "hidden_act")) != -2) throw TeiError(ERR_START, family + " expects hidden_act = silu");
    if (mt == "qwen3") {
      if (c.get_bool("use_sliding_window", false)) throw TeiError(ERR_START, "sliding window is not supported");
      if (need_bool(c, "attention_bias")) throw TeiError(ERR_START, "attention_bias = true is not supported");
      s.head_dim = static_cast<int>(c.get_int("head_dim", s.heads > 0 ? s.hidden / s.heads : 0));
      s.qk_norm = true;
      s.causal = !c.get_bool("use_bidirectional_attention", false);
    } else if (mt == "qwen2") {
      // flash_qwen2.rs:26-29,36-57: q/k/v carry biases, no sliding window, `is_causal`
      // defaults to true (qwen2.rs:4-7,26-27).
      if (need_bool(c, "use_sliding_window")) throw TeiError(ERR_START, "Sliding window is not supported for Qwen2");
      s.head_dim = s.heads > 0 ? s.hidden / s.heads : 0;
      s.qkv_bias = true;
      s.causal = c.get_bool("is_causal", true);
    } else {
      // flash_mistral.rs:56,95-110: `sliding_window` is the left window of the attention.
      // Llama's rope_scaling is refused (lib.rs:549-553); Mistral hands its own to get_inv_freqs
      // (flash_mistral.rs:278-283), whose untagged enum picks the variant by the fields present
      // (layers/rotary.rs:11-27): Llama3 with all four numbers, NTK with `factor` alone.
      if (!c["rope_scaling"].is_null()) {
        if (mt == "llama") throw TeiError(ERR_START, "Rope scaling is not supported for FlashLlama yet");
        const Json& rs = c["rope_scaling"];
        if (!rs.is_object() || !rs["factor"].is_number()) throw TeiError(ERR_START, "config.json: unsupported `rope_scaling`");
        const float factor = static_cast<float>(rs["factor"].as_double());
        if (rs["high_freq_factor"].is_number() && rs["low_freq_factor"].is_number() &&
            rs["original_max_position_embeddings"].is_number()) {
          s.rope_l3_factor = factor;
          s.rope_l3_high = static_cast<float>(rs["high_freq_factor"].as_double());
          s.rope_l3_low = static_cast<float>(rs["low_freq_factor"].as_double());
          s.rope_l3_orig_max = static_cast<float>(rs["original_max_position_embeddings"].as_double());
        } else {
          s.rope_ntk_factor = factor;
        }
      }
      s.head_dim = s.heads > 0 ? s.hidden / s.heads : 0;
      if (mt == "mistral" && c["sliding_window"].is_number()) s.window_left = static_cast<int>(c["sliding_window"].as_int());
      s.causal = !c.get_bool("use_bidirectional_attention", false);
    }
    if (c["rope_theta"].is_number()) {
      s.rope_theta = static_cast<float>(c["rope_theta"].as_double());
    } else if (c["rope_parameters"]["rope_theta"].is_number()) {
      s.rope_theta = static_cast<float>(c["rope_parameters"]["rope_theta"].as_double());
    } else {
      throw TeiError(ERR_START, "Neither `rope_theta` nor `rope_parameters.rope_theta` are defined in the `config.json`");
    }
    s.gated = true;
    s.act = ACT_SWIGLU;
    s.rope = true;
    s.rope_table_len = s.max_pos;
    s.type_vocab = 0;
  } else if (mt == "modernbert") {
    // ModernBertConfig (models/modernbert.rs:12-49); it runs on the pre-norm decoder skeleton.
    s.arch = ARCH_QWEN3;
    s.modernbert = true;
    if (s.pool == POOL_SPLADE) throw TeiError(ERR_START, "`splade` is not supported for ModernBert");
    s.vocab = static_cast<int>(need_int(c, "vocab_size"));
    s.hidden = static_cast<int>(need_int(c, "hidden_size"));
    s.inter = static_cast<int>(need_int(c, "intermediate_size"));
    s.layers = static_cast<int>(need_int(c, "num_hidden_layers"));
    s.heads = s.kv_heads = static_cast<int>(need_int(c, "num_attention_heads"));
    s.max_pos = static_cast<int>(need_int(c, "max_position_embeddings"));
    s.eps = static_cast<float>(need_double(c, "norm_eps"));
    if (parse_act(need_string(c, "hidden_activation")) != ACT_GELU) {
      throw TeiError(ERR_START, "ModernBert expects a GELU hidden_activation");
    }
    s.head_dim = s.heads > 0 ? s.hidden / s.heads : 0;
    s.rope_theta = static_cast<float>(need_double(c, "global_rope_theta"));
    s.local_theta = static_cast<float>(need_double(c, "local_rope_theta"));
    s.global_every = static_cast<int>(need_int(c, "global_attn_every_n_layers"));
    s.local_window = static_cast<int>(need_int(c, "local_attention")) / 2;  // flash_modernbert.rs:61
    if (s.global_every <= 0) throw TeiError(ERR_START, "global_attn_every_n_layers must be positive");
    s.gated = true;
    s.act = ACT_GEGLU;  // act(first half) * second half (modernbert.rs:115-127)
    s.rope = true;
    s.rope_table_len = s.max_pos;
    s.causal = false;
    s.type_vocab = 0;
    if (s.classifier) {
      // modernbert.rs:425-432,482-483: `num_labels` rows (1 when absent), pooling from the config
      s.n_classes = static_cast<int>(c.get_int("num_labels", c["id2label"].is_object() ? static_cast<int64_t>(c["id2label"].size()) : 1));
      const std::string cp = c.get_string("classifier_pooling", "cls");
      if (cp == "cls") s.cls_pool = POOL_CLS;
      else if (cp == "mean") s.cls_pool = POOL_MEAN;
      else throw TeiError(ERR_START, "unknown classifier_pooling " + cp);
      s.head_act = parse_act(need_string(c, "classifier_activation"));
      if (s.head_act < 0 || s.head_act == ACT_SWIGLU) throw TeiError(ERR_START, "unsupported classifier_activation");
    }
  } else {
    // backends/candle/src/lib.rs:537-542: the reference itself refuses this model in half precision
    if (mt == "bidirectional_pplx_qwen3") throw TeiError(ERR_START, "Pplx1 is only supported in fp32 precision");
    throw TeiError(ERR_START, "model_type `" + mt + "` is not served by this backend");
  }
  if (s.head_dim != 32 && s.head_dim != 64 && s.head_dim != 128) {
    throw TeiError(ERR_START, "head_dim must be 32, 64 or 128 for the sm_100a attention kernel");
  }
  if (s.kv_heads <= 0 || s.heads % s.kv_heads != 0) throw TeiError(ERR_START, "heads must be a multiple of kv heads");
  if (s.hidden % 8 != 0 || s.inter % 8 != 0 || s.hidden > 4096) {
    throw TeiError(ERR_START, "hidden / intermediate sizes must be multiples of 8 and hidden <= 4096");
  }
  if (s.gated && s.inter % 128 != 0) throw TeiError(ERR_START, "gated feed-forward needs intermediate_size % 128 == 0");
  if (s.pool == POOL_SPLADE && s.arch != ARCH_BERT) throw TeiError(ERR_START, "splade needs a BERT-family masked-LM checkpoint");
  return s;
}

// A build runs on its own architecture and on the later ones of its family:
// Turing 75 on 75; Ampere 80 on 80..89; 86 on 86..89; Ada 89 on 89; Hopper 90 on 90; Blackwell
// 100 on 100; 120 on 120..121; 121 on 121 (compute_cap.rs:27-40).
bool compute_cap_matching(int runtime_cap, int compile_cap) {
  struct Range { int compile, lo, hi; };
  static const Range kRanges[] = {{75, 75, 75}, {80, 80, 89}, {86, 86, 89}, {89, 89, 89},
                                  {90, 90, 90}, {100, 100, 100}, {120, 120, 121}, {121, 121, 121}};
  // builds between two listed Ampere targets (81..85) run where the 86 build would, as the
  // reference's second arm says: runtime 86..89 with compile 80..=86
  if (compile_cap > 80 && compile_cap < 86) return runtime_cap >= 86 && runtime_cap <= 89;
  for (const Range& r : kRanges) {
    if (r.compile == compile_cap) return runtime_cap >= r.lo && runtime_cap <= r.hi;
  }
  return false;
}

// ------------------------------------------------------------------------------ Replica
Replica::Replica(int device, const ModelSpec& spec, const SafeTensors& st)
    : device_(device), spec_(spec) {
  cudaError_t e = cudaSetDevice(device_);
  if (e != cudaSuccess) throw TeiError(ERR_START, std::string("cudaSetDevice: ") + cudaGetErrorString(e));
  int major = 0, minor = 0;
  cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device_);
  cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device_);
  const int runtime_cap = major * 10 + minor;
  if (!compute_cap_matching(runtime_cap, kCompileComputeCap)) {  // the refusal of lib.rs:240-248
    throw TeiError(ERR_START, "Runtime compute cap " + std::to_string(runtime_cap) +
                                  " is not compatible with compile time compute cap " +
                                  std::to_string(kCompileComputeCap) + " (this backend needs an sm_100 device)");
  }
  TEI_CUDA(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
  TEI_CUDA(cudaEventCreate(&ev_start_));
  TEI_CUDA(cudaEventCreate(&ev_stop_));
  try {
    load_weights(st);
    if (spec_.rope) build_rope_tables();
    TEI_CUDA(cudaStreamSynchronize(stream_));
    if (load_stage_) {
      cudaFree(load_stage_);
      load_stage_ = nullptr;
      load_stage_bytes_ = 0;
    }
  } catch (const TeiError&) {
    throw;
  } catch (const std::exception& ex) {
    const std::string m = ex.what();
    throw TeiError(m.rfind("weights not found", 0) == 0 ? ERR_WEIGHTS_NOT_FOUND : ERR_START, m);
  }
}

Replica::~Replica() {
  cudaSetDevice(device_);
  if (stream_) cudaStreamSynchronize(stream_);
  for (void* p : allocs_) cudaFree(p);
  if (load_stage_) cudaFree(load_stage_);
  if (arena_) cudaFree(arena_);
  if (d_ints_) cudaFree(d_ints_);
  if (h_ints_) cudaFreeHost(h_ints_);
  if (d_out_) cudaFree(d_out_);
  if (h_out_) cudaFreeHost(h_out_);
  for (auto& e : ev_pool_) cudaEventDestroy(e);
  if (ev_start_) cudaEventDestroy(ev_start_);
  if (ev_stop_) cudaEventDestroy(ev_stop_);
  if (stream_) cudaStreamDestroy(stream_);
}

int Replica::raw_dim() const {
  if (spec_.pool == POOL_SPLADE) return spec_.vocab;
  if (projection_) return projection_dim_;
  return spec_.hidden;
}

int Replica::output_dim() const { return dense_.empty() ? raw_dim() : dense_.back().out; }

void Replica::add_dense(const std::string& dir) {
  TEI_CUDA(cudaSetDevice(device_));
  if (spec_.classifier) throw TeiError(ERR_START, "Dense modules apply to embedding models only");
  if (spec_.pool == POOL_SPLADE) throw TeiError(ERR_START, "Dense modules cannot follow SPLADE pooling");
  std::string text;
  {
    std::FILE* f = std::fopen((dir + "/config.json").c_str(), "rb");
    if (!f) throw TeiError(ERR_START, "Unable to read `" + dir + "/config.json` file");
    char buf[4096];
    size_t n;
    while ((n = std::fread(buf, 1, sizeof(buf), f)) > 0) text.append(buf, n);
    std::fclose(f);
  }
  Json cfg;
  try {
    cfg = Json::parse(text);
  } catch (const std::exception& e) {
    throw TeiError(ERR_START, "Unable to parse `" + dir + "/config.json`: " + e.what());
  }
  // DenseConfig (dense.rs:26-32): in_features, out_features and bias are required.
  if (!cfg["in_features"].is_number() || !cfg["out_features"].is_number() || !cfg["bias"].is_bool()) {
    throw TeiError(ERR_START, "Unable to parse `" + dir + "/config.json`: in_features, out_features and bias are required");
  }
  DenseW d;
  d.in = static_cast<int>(cfg["in_features"].as_int());
  d.out = static_cast<int>(cfg["out_features"].as_int());
  d.act = ACT_NONE;
  if (cfg["activation_function"].is_string()) {
    const std::string a = cfg["activation_function"].as_string();
    if (a == "torch.nn.modules.activation.Tanh") d.act = ACT_TANH;
    else if (a == "torch.nn.modules.linear.Identity") d.act = ACT_NONE;
    else throw TeiError(ERR_START, "Unable to parse `" + dir + "/config.json`: unknown activation_function " + a);
  }
  if (d.in <= 0 || d.out <= 0) throw TeiError(ERR_START, "Dense module with an empty dimension");
  if (d.in != output_dim()) {
    throw TeiError(ERR_START, "Dense module expects " + std::to_string(d.in) + " input features, the model gives " +
                                  std::to_string(output_dim()));
  }
  SafeTensors st;
  try {
    st.open_file(dir + "/model.safetensors");
  } catch (const std::exception& e) {
    throw TeiError(ERR_START, std::string("Dense module weights: ") + e.what());
  }
  if (!st.contains("linear.weight")) throw TeiError(ERR_START, "Dense module without `linear.weight`");
  const StTensor& w = st.get("linear.weight");
  if (w.shape.size() != 2 || w.shape[0] != static_cast<size_t>(d.out) || w.shape[1] != static_cast<size_t>(d.in)) {
    throw TeiError(ERR_START, "Dense module `linear.weight` does not have the shape [out_features, in_features]");
  }
  d.w = upload_new(w);
  if (cfg["bias"].as_bool()) {
    if (!st.contains("linear.bias")) throw TeiError(ERR_START, "Dense module without `linear.bias`");
    const StTensor& b = st.get("linear.bias");
    if (b.shape.size() != 1 || b.shape[0] != static_cast<size_t>(d.out)) {
      throw TeiError(ERR_START, "Dense module `linear.bias` does not have the shape [out_features]");
    }
    d.b = upload_new(b);
  }
  TEI_CUDA(cudaStreamSynchronize(stream_));
  dense_.push_back(d);
}

void* Replica::dev_alloc(size_t bytes) {
  void* p = nullptr;
  TEI_CUDA(cudaMalloc(&p, std::max<size_t>(bytes, 16)));
  allocs_.push_back(p);
  return p;
}

void Replica::set_profiling(bool on) {
  TEI_CUDA(cudaSetDevice(device_));
  if (on && ev_pool_.empty()) {
    ev_pool_.resize(2 * kMaxPairs);
    for (auto& e : ev_pool_) TEI_CUDA(cudaEventCreate(&e));
    pair_cls_.resize(kMaxPairs);
  }
  profiling_ = on;
  n_pairs_ = 0;
  for (int i = 0; i < KC_COUNT; ++i) {
    class_ms_[i] = 0.0;
    class_launches_[i] = 0.0;
  }
}

void Replica::prof_begin() {
  if (profiling_ && n_pairs_ < kMaxPairs) cudaEventRecord(ev_pool_[2 * n_pairs_], stream_);
}

void Replica::prof_end(int cls) {
  if (profiling_ && n_pairs_ < kMaxPairs) {
    cudaEventRecord(ev_pool_[2 * n_pairs_ + 1], stream_);
    pair_cls_[n_pairs_] = cls;
    ++n_pairs_;
  }
}

// Called after a stream synchronise: folds the recorded event pairs into the per-class totals.
void Replica::prof_drain() {
  for (int i = 0; i < n_pairs_; ++i) {
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, ev_pool_[2 * i], ev_pool_[2 * i + 1]) == cudaSuccess) {
      class_ms_[pair_cls_[i]] += ms;
      class_launches_[pair_cls_[i]] += 1.0;
    }
  }
  n_pairs_ = 0;
}

int Replica::kernel_times(double* ms, double* launches, int n) const {
  const int m = n < KC_COUNT ? n : KC_COUNT;
  for (int i = 0; i < m; ++i) {
    ms[i] = class_ms_[i];
    launches[i] = class_launches_[i];
  }
  return m;
}

double Replica::timed_runs(int steps) {
  TEI_CUDA(cudaSetDevice(device_));
  cudaEvent_t a, b;
  TEI_CUDA(cudaEventCreate(&a));
  TEI_CUDA(cudaEventCreate(&b));
  TEI_CUDA(cudaStreamSynchronize(stream_));
  TEI_CUDA(cudaEventRecord(a, stream_));
  int launches = 0;
  for (int i = 0; i < steps; ++i) {
    run();
    launches += launches_;
  }
  TEI_CUDA(cudaEventRecord(b, stream_));
  sync_and_check();
  float ms = 0.f;
  cudaEventElapsedTime(&ms, a, b);
  cudaEventDestroy(a);
  cudaEventDestroy(b);
  stats_.last_launches = launches;
  return ms;
}

void Replica::launch(int rc, const char* what) {
  if (rc != 0) {
    throw TeiError(ERR_INFERENCE, std::string(what) + " launch failed with code " + std::to_string(rc));
  }
  ++launches_;
}

void Replica::upload(void* dst, size_t dst_elem_off, const StTensor& src, int dst_kind) {
  if (dst_kind < 0) dst_kind = spec_.dtype;
  int src_kind;
  switch (src.dtype) {
    case StDType::F32: src_kind = 0; break;
    case StDType::F16: src_kind = 1; break;
    case StDType::BF16: src_kind = 2; break;
    default: throw TeiError(ERR_START, "unsupported tensor dtype in safetensors (need F32, F16 or BF16)");
  }
  if (src.nbytes > load_stage_bytes_) {
    TEI_CUDA(cudaStreamSynchronize(stream_));
    if (load_stage_) cudaFree(load_stage_);
    load_stage_bytes_ = align_up(src.nbytes, 1 << 20);
    TEI_CUDA(cudaMalloc(&load_stage_, load_stage_bytes_));
  }
  TEI_CUDA(cudaMemcpyAsync(load_stage_, src.data, src.nbytes, cudaMemcpyHostToDevice, stream_));
  const size_t es = dst_kind == 2 ? 4 : 2;
  int rc = launch_convert(load_stage_, src_kind, static_cast<uint8_t*>(dst) + dst_elem_off * es,
                          dst_kind, static_cast<size_t>(src.numel()), stream_);
  if (rc) throw TeiError(ERR_START, "dtype conversion kernel failed");
}

void* Replica::upload_new(const StTensor& src, int dst_kind) {
  const size_t es = (dst_kind == 2) ? 4 : 2;
  void* p = dev_alloc(static_cast<size_t>(src.numel()) * es);
  upload(p, 0, src, dst_kind);
  return p;
}

// dst rows: [gate 0..127 | up 0..127 | gate 128..255 | up 128..255 | ...] (the layout the SwiGLU
// epilogue of the GEMM expects).  Works for matrices [I, K] and for bias vectors [I].
void Replica::upload_rows_interleaved(void* dst, const StTensor& gate, const StTensor& up) {
  if (gate.shape != up.shape || gate.shape.empty() || gate.shape[0] % 128 != 0) {
    throw TeiError(ERR_START, "gate / up shapes do not allow the 128-row interleave");
  }
  const size_t rows = static_cast<size_t>(gate.shape[0]);
  const size_t cols = static_cast<size_t>(gate.numel()) / rows;
  void* tg = nullptr;
  void* tu = nullptr;
  TEI_CUDA(cudaMalloc(&tg, rows * cols * 2));
  TEI_CUDA(cudaMalloc(&tu, rows * cols * 2));
  try {
    upload(tg, 0, gate);
    upload(tu, 0, up);
    const size_t blk = 128 * cols * 2;
    TEI_CUDA(cudaMemcpy2DAsync(dst, 2 * blk, tg, blk, blk, rows / 128, cudaMemcpyDeviceToDevice, stream_));
    TEI_CUDA(cudaMemcpy2DAsync(static_cast<uint8_t*>(dst) + blk, 2 * blk, tu, blk, blk, rows / 128,
                               cudaMemcpyDeviceToDevice, stream_));
    TEI_CUDA(cudaStreamSynchronize(stream_));
  } catch (...) {
    cudaFree(tg);
    cudaFree(tu);
    throw;
  }
  cudaFree(tg);
  cudaFree(tu);
}

namespace {

struct Names {
  const SafeTensors& st;
  std::string prefix;
  bool has(const std::string& n) const { return st.contains(prefix + n); }
  const StTensor& get(const std::string& n) const {
    if (!st.contains(prefix + n)) throw TeiError(ERR_START, "cannot find tensor " + prefix + n);
    return st.get(prefix + n);
  }
  // LayerNorm::load accepts weight|gamma and bias|beta (layers/layer_norm.rs:93-98).
  const StTensor& ln_w(const std::string& p) const { return has(p + ".weight") ? get(p + ".weight") : get(p + ".gamma"); }
  const StTensor& ln_b(const std::string& p) const { return has(p + ".bias") ? get(p + ".bias") : get(p + ".beta"); }
};

// A vector parameter (bias, norm weight) must have exactly the length the kernels will read.
const StTensor& vec(const StTensor& t, int64_t n, const char* what) {
  if (t.numel() != n) {
    throw TeiError(ERR_START, std::string("unexpected shape for a ") + what + " vector: " + std::to_string(t.numel()) +
                                  " elements where the config implies " + std::to_string(n));
  }
  return t;
}

void expect_shape(const StTensor& t, std::initializer_list<int64_t> shape, const std::string& name) {
  if (t.shape != std::vector<int64_t>(shape)) {
    throw TeiError(ERR_START, "unexpected shape for tensor " + name);
  }
}

}  // namespace

void Replica::load_weights(const SafeTensors& st) {
  layers_.resize(spec_.layers);
  switch (spec_.arch) {
    case ARCH_BERT: load_bert(st); break;
    case ARCH_NOMIC:
      if (spec_.gte) load_gte(st);
      else load_nomic(st);
      break;
    case ARCH_QWEN3:
      if (spec_.modernbert) load_modernbert(st);
      else load_qwen3(st);
      break;
  }
}

void Replica::load_bert(const SafeTensors& st) {
  const ModelSpec& s = spec_;
  const int H = s.hidden, I = s.inter;
  if (s.distil) {
    // flash_distilbert.rs:205-226: `embeddings` + `encoder`, `distilbert.embeddings` +
    // `distilbert.transformer`, or `embeddings` + `transformer`.
    std::string emb, enc;
    if (st.contains("embeddings.word_embeddings.weight") && st.contains("encoder.layer.0.attention.q_lin.weight")) {
      emb = "embeddings."; enc = "encoder.";
    } else if (st.contains("distilbert.embeddings.word_embeddings.weight")) {
      emb = "distilbert.embeddings."; enc = "distilbert.transformer.";
    } else if (st.contains("embeddings.word_embeddings.weight")) {
      emb = "embeddings."; enc = "transformer.";
    } else {
      throw TeiError(ERR_START, "cannot find tensor embeddings.word_embeddings.weight");
    }
    Names n{st, ""};
    expect_shape(n.get(emb + "word_embeddings.weight"), {s.vocab, H}, emb + "word_embeddings.weight");
    expect_shape(n.get(emb + "position_embeddings.weight"), {s.max_pos, H}, emb + "position_embeddings.weight");
    word_ = upload_new(n.get(emb + "word_embeddings.weight"));
    pos_tab_ = upload_new(n.get(emb + "position_embeddings.weight"));
    emb_g_ = upload_new(vec(n.ln_w(emb + "LayerNorm"), H, "hidden-size"));
    emb_b_ = upload_new(vec(n.ln_b(emb + "LayerNorm"), H, "hidden-size"));
    for (int i = 0; i < s.layers; ++i) {
      LayerW& L = layers_[i];
      const std::string p = enc + "layer." + std::to_string(i) + ".";
      L.wqkv = dev_alloc(static_cast<size_t>(3) * H * H * 2);
      L.bqkv = dev_alloc(static_cast<size_t>(3) * H * 2);
      const char* qkv[3] = {"q_lin", "k_lin", "v_lin"};
      for (int j = 0; j < 3; ++j) {
        const StTensor& w = n.get(p + "attention." + qkv[j] + ".weight");
        expect_shape(w, {H, H}, p + "attention." + qkv[j] + ".weight");
        upload(L.wqkv, static_cast<size_t>(j) * H * H, w);
        upload(L.bqkv, static_cast<size_t>(j) * H, vec(n.get(p + "attention." + qkv[j] + ".bias"), H, "q/k/v bias"));
      }
      expect_shape(n.get(p + "attention.out_lin.weight"), {H, H}, p + "attention.out_lin.weight");
      L.wo = upload_new(n.get(p + "attention.out_lin.weight"));
      L.bo = upload_new(vec(n.get(p + "attention.out_lin.bias"), H, "hidden-size"));
      L.ln1_g = upload_new(vec(n.ln_w(p + "sa_layer_norm"), H, "hidden-size"));
      L.ln1_b = upload_new(vec(n.ln_b(p + "sa_layer_norm"), H, "hidden-size"));
      expect_shape(n.get(p + "ffn.lin1.weight"), {I, H}, p + "ffn.lin1.weight");
      L.w1 = upload_new(n.get(p + "ffn.lin1.weight"));
      L.b1 = upload_new(vec(n.get(p + "ffn.lin1.bias"), I, "feed-forward bias"));
      expect_shape(n.get(p + "ffn.lin2.weight"), {H, I}, p + "ffn.lin2.weight");
      L.w2 = upload_new(n.get(p + "ffn.lin2.weight"));
      L.b2 = upload_new(vec(n.get(p + "ffn.lin2.bias"), H, "hidden-size"));
      L.ln2_g = upload_new(vec(n.ln_w(p + "output_layer_norm"), H, "hidden-size"));
      L.ln2_b = upload_new(vec(n.ln_b(p + "output_layer_norm"), H, "hidden-size"));
    }
    return;
  }
  // flash_bert.rs:264-279 (bert) and :331-356 (roberta family): bare names, then known prefixes.
  std::vector<std::string> cand = s.roberta ? std::vector<std::string>{"", "roberta.", "xlm-roberta.", "camembert."}
                                            : std::vector<std::string>{"", "bert."};
  std::string prefix;
  bool found = false;
  for (const auto& p : cand) {
    if (st.contains(p + "embeddings.word_embeddings.weight")) {
      prefix = p;
      found = true;
      break;
    }
  }
  if (!found) throw TeiError(ERR_START, "cannot find tensor embeddings.word_embeddings.weight");
  Names n{st, prefix};
  Names root{st, ""};
  expect_shape(n.get("embeddings.word_embeddings.weight"), {s.vocab, H}, "embeddings.word_embeddings.weight");
  expect_shape(n.get("embeddings.token_type_embeddings.weight"), {s.type_vocab, H}, "embeddings.token_type_embeddings.weight");
  word_ = upload_new(n.get("embeddings.word_embeddings.weight"));
  if (!s.alibi) {  // JinaEmbeddings::load, jina.rs:20-31
    expect_shape(n.get("embeddings.position_embeddings.weight"), {s.max_pos, H}, "embeddings.position_embeddings.weight");
    pos_tab_ = upload_new(n.get("embeddings.position_embeddings.weight"));
  } else {
    // alibi_head_slopes (alibi.rs:18-47), f64 on the host, fp32 on the device as flash_jina.rs:237-241
    auto pow2_slopes = [](int k) {
      const double start = std::pow(2.0, -std::pow(2.0, -(std::log2(static_cast<double>(k)) - 3.0)));
      std::vector<double> v(k);
      for (int i = 0; i < k; ++i) v[i] = start * std::pow(start, i);
      return v;
    };
    std::vector<double> sl;
    const double lg = std::log2(static_cast<double>(s.heads));
    if (lg == std::floor(lg)) {
      sl = pow2_slopes(s.heads);
    } else {
      const int closest = 1 << static_cast<int>(std::floor(lg));
      sl = pow2_slopes(closest);
      const std::vector<double> extra = pow2_slopes(2 * closest);
      for (int i = 0; static_cast<int>(sl.size()) < s.heads; i += 2) sl.push_back(extra[i]);
    }
    std::vector<float> slf(sl.begin(), sl.end());
    alibi_slopes_ = static_cast<float*>(dev_alloc(slf.size() * 4));
    TEI_CUDA(cudaMemcpy(alibi_slopes_, slf.data(), slf.size() * 4, cudaMemcpyHostToDevice));
  }
  type_tab_ = upload_new(n.get("embeddings.token_type_embeddings.weight"));
  emb_g_ = upload_new(vec(n.ln_w("embeddings.LayerNorm"), H, "hidden-size"));
  emb_b_ = upload_new(vec(n.ln_b("embeddings.LayerNorm"), H, "hidden-size"));
  for (int i = 0; i < s.layers; ++i) {
    LayerW& L = layers_[i];
    const std::string p = "encoder.layer." + std::to_string(i) + ".";
    // q, k, v fused by concatenating rows (flash_bert.rs:43-44).
    L.wqkv = dev_alloc(static_cast<size_t>(3) * H * H * 2);
    L.bqkv = dev_alloc(static_cast<size_t>(3) * H * 2);
    const char* qkv[3] = {"query", "key", "value"};
    for (int j = 0; j < 3; ++j) {
      const StTensor& w = n.get(p + "attention.self." + qkv[j] + ".weight");
      expect_shape(w, {H, H}, p + "attention.self." + qkv[j] + ".weight");
      upload(L.wqkv, static_cast<size_t>(j) * H * H, w);
      upload(L.bqkv, static_cast<size_t>(j) * H, vec(n.get(p + "attention.self." + qkv[j] + ".bias"), H, "q/k/v bias"));
    }
    expect_shape(n.get(p + "attention.output.dense.weight"), {H, H}, p + "attention.output.dense.weight");
    L.wo = upload_new(n.get(p + "attention.output.dense.weight"));
    L.bo = upload_new(vec(n.get(p + "attention.output.dense.bias"), H, "hidden-size"));
    L.ln1_g = upload_new(vec(n.ln_w(p + "attention.output.LayerNorm"), H, "hidden-size"));
    L.ln1_b = upload_new(vec(n.ln_b(p + "attention.output.LayerNorm"), H, "hidden-size"));
    if (s.jina_code) {
      // JinaCodeAttention::load / JinaCodeBertLayer::load (flash_jina_code.rs:27-90,170-212):
      // `attention.self.layer_norm_q` / `_k` over the whole hidden width; `mlp.up_gated_layer`
      // [2I, H] without bias whose rows [0, I) are NOT gated and rows [I, 2I) go through the
      // activation (:236-240); `mlp.down_layer`; `layer_norm_1`, `layer_norm_2`.
      L.lnq_g = upload_new(vec(n.ln_w(p + "attention.self.layer_norm_q"), H, "hidden-size"));
      L.lnq_b = upload_new(vec(n.ln_b(p + "attention.self.layer_norm_q"), H, "hidden-size"));
      L.lnk_g = upload_new(vec(n.ln_w(p + "attention.self.layer_norm_k"), H, "hidden-size"));
      L.lnk_b = upload_new(vec(n.ln_b(p + "attention.self.layer_norm_k"), H, "hidden-size"));
      const StTensor& gw = n.get(p + "mlp.up_gated_layer.weight");
      expect_shape(gw, {2 * I, H}, p + "mlp.up_gated_layer.weight");
      StTensor gate = gw, up = gw;
      gate.shape = {I, H};
      up.shape = {I, H};
      gate.nbytes = up.nbytes = gw.nbytes / 2;
      gate.data = gw.data + gw.nbytes / 2;
      L.w1 = dev_alloc(static_cast<size_t>(2) * I * H * 2);
      upload_rows_interleaved(L.w1, gate, up);
      expect_shape(n.get(p + "mlp.down_layer.weight"), {H, I}, p + "mlp.down_layer.weight");
      L.w2 = upload_new(n.get(p + "mlp.down_layer.weight"));
      L.b2 = upload_new(vec(n.get(p + "mlp.down_layer.bias"), H, "hidden-size"));
      L.lnm_g = upload_new(vec(n.ln_w(p + "layer_norm_1"), H, "hidden-size"));
      L.lnm_b = upload_new(vec(n.ln_b(p + "layer_norm_1"), H, "hidden-size"));
      L.ln2_g = upload_new(vec(n.ln_w(p + "layer_norm_2"), H, "hidden-size"));
      L.ln2_b = upload_new(vec(n.ln_b(p + "layer_norm_2"), H, "hidden-size"));
      continue;
    }
    if (s.jina) {
      // JinaBertLayer::load (flash_jina.rs:133-155): `mlp.gated_layers.weight` [2I, H] without
      // bias, rows [0, I) gated by the activation, rows [I, 2I) not; `mlp.wo`; `mlp.layernorm`.
      const StTensor& gw = n.get(p + "mlp.gated_layers.weight");
      expect_shape(gw, {2 * I, H}, p + "mlp.gated_layers.weight");
      StTensor gate = gw, up = gw;
      gate.shape = {I, H};
      up.shape = {I, H};
      gate.nbytes = up.nbytes = gw.nbytes / 2;
      up.data = gw.data + gw.nbytes / 2;
      L.w1 = dev_alloc(static_cast<size_t>(2) * I * H * 2);
      upload_rows_interleaved(L.w1, gate, up);
      expect_shape(n.get(p + "mlp.wo.weight"), {H, I}, p + "mlp.wo.weight");
      L.w2 = upload_new(n.get(p + "mlp.wo.weight"));
      L.b2 = upload_new(vec(n.get(p + "mlp.wo.bias"), H, "hidden-size"));
      L.ln2_g = upload_new(vec(n.ln_w(p + "mlp.layernorm"), H, "hidden-size"));
      L.ln2_b = upload_new(vec(n.ln_b(p + "mlp.layernorm"), H, "hidden-size"));
      continue;
    }
    expect_shape(n.get(p + "intermediate.dense.weight"), {I, H}, p + "intermediate.dense.weight");
    L.w1 = upload_new(n.get(p + "intermediate.dense.weight"));
    L.b1 = upload_new(vec(n.get(p + "intermediate.dense.bias"), I, "feed-forward bias"));
    expect_shape(n.get(p + "output.dense.weight"), {H, I}, p + "output.dense.weight");
    L.w2 = upload_new(n.get(p + "output.dense.weight"));
    L.b2 = upload_new(vec(n.get(p + "output.dense.bias"), H, "hidden-size"));
    L.ln2_g = upload_new(vec(n.ln_w(p + "output.LayerNorm"), H, "hidden-size"));
    L.ln2_b = upload_new(vec(n.ln_b(p + "output.LayerNorm"), H, "hidden-size"));
  }
  if (s.classifier) {
    if (s.roberta) {  // RobertaClassificationHead, bert.rs:434-444
      expect_shape(root.get("classifier.dense.weight"), {H, H}, "classifier.dense.weight");
      expect_shape(root.get("classifier.out_proj.weight"), {s.n_classes, H}, "classifier.out_proj.weight");
      cls_dense_w_ = upload_new(root.get("classifier.dense.weight"));
      cls_dense_b_ = upload_new(vec(root.get("classifier.dense.bias"), H, "hidden-size"));
      cls_out_w_ = upload_new(root.get("classifier.out_proj.weight"));
      cls_out_b_ = upload_new(vec(root.get("classifier.out_proj.bias"), s.n_classes, "classifier bias"));
    } else {  // BertClassificationHead, bert.rs:381-395
      if (root.has("bert.pooler.dense.weight")) {
        expect_shape(root.get("bert.pooler.dense.weight"), {H, H}, "bert.pooler.dense.weight");
        cls_dense_w_ = upload_new(root.get("bert.pooler.dense.weight"));
        cls_dense_b_ = upload_new(vec(root.get("bert.pooler.dense.bias"), H, "hidden-size"));
      }
      expect_shape(root.get("classifier.weight"), {s.n_classes, H}, "classifier.weight");
      cls_out_w_ = upload_new(root.get("classifier.weight"));
      cls_out_b_ = upload_new(vec(root.get("classifier.bias"), s.n_classes, "classifier bias"));
    }
  }
  if (s.pool == POOL_SPLADE) {
    if (s.roberta) {  // bert.rs:519-541
      expect_shape(root.get("lm_head.dense.weight"), {H, H}, "lm_head.dense.weight");
      expect_shape(root.get("lm_head.decoder.weight"), {s.vocab, H}, "lm_head.decoder.weight");
      sp_dense_w_ = upload_new(root.get("lm_head.dense.weight"));
      sp_dense_b_ = upload_new(vec(root.get("lm_head.dense.bias"), H, "hidden-size"));
      sp_ln_g_ = upload_new(vec(root.ln_w("lm_head.layer_norm"), H, "hidden-size"));
      sp_ln_b_ = upload_new(vec(root.ln_b("lm_head.layer_norm"), H, "hidden-size"));
      sp_dec_w_ = upload_new(root.get("lm_head.decoder.weight"));
      sp_dec_b_ = upload_new(vec(root.get("lm_head.bias"), s.vocab, "decoder bias"));
      sp_act_ = ACT_GELU;
    } else {  // bert.rs:477-509
      expect_shape(root.get("cls.predictions.transform.dense.weight"), {H, H}, "cls.predictions.transform.dense.weight");
      {
        const char* dec = root.has("cls.predictions.decoder.weight") ? "cls.predictions.decoder.weight"
                                                                      : "bert.embeddings.word_embeddings.weight";
        expect_shape(root.get(dec), {s.vocab, H}, dec);
      }
      sp_dense_w_ = upload_new(root.get("cls.predictions.transform.dense.weight"));
      sp_dense_b_ = upload_new(vec(root.get("cls.predictions.transform.dense.bias"), H, "hidden-size"));
      sp_ln_g_ = upload_new(vec(root.ln_w("cls.predictions.transform.LayerNorm"), H, "hidden-size"));
      sp_ln_b_ = upload_new(vec(root.ln_b("cls.predictions.transform.LayerNorm"), H, "hidden-size"));
      sp_dec_w_ = root.has("cls.predictions.decoder.weight")
                      ? upload_new(root.get("cls.predictions.decoder.weight"))
                      : upload_new(root.get("bert.embeddings.word_embeddings.weight"));
      sp_dec_b_ = upload_new(vec(root.get("cls.predictions.bias"), s.vocab, "decoder bias"));
      sp_act_ = s.act;
    }
  }
}

void Replica::load_nomic(const SafeTensors& st) {
  const ModelSpec& s = spec_;
  const int H = s.hidden, I = s.inter;
  Names n{st, ""};
  expect_shape(n.get("embeddings.word_embeddings.weight"), {s.vocab, H}, "embeddings.word_embeddings.weight");
  word_ = upload_new(n.get("embeddings.word_embeddings.weight"));
  expect_shape(n.get("embeddings.token_type_embeddings.weight"), {s.type_vocab, H}, "embeddings.token_type_embeddings.weight");
  type_tab_ = upload_new(n.get("embeddings.token_type_embeddings.weight"));
  emb_g_ = upload_new(vec(n.ln_w("emb_ln"), H, "hidden-size"));
  emb_b_ = upload_new(vec(n.ln_b("emb_ln"), H, "hidden-size"));
  for (int i = 0; i < s.layers; ++i) {
    LayerW& L = layers_[i];
    const std::string p = "encoder.layers." + std::to_string(i) + ".";
    expect_shape(n.get(p + "attn.Wqkv.weight"), {3 * H, H}, p + "attn.Wqkv.weight");
    L.wqkv = upload_new(n.get(p + "attn.Wqkv.weight"));
    if (s.qkv_bias) L.bqkv = upload_new(vec(n.get(p + "attn.Wqkv.bias"), s.qkv_width(), "qkv bias"));
    expect_shape(n.get(p + "attn.out_proj.weight"), {H, H}, p + "attn.out_proj.weight");
    L.wo = upload_new(n.get(p + "attn.out_proj.weight"));
    if (s.out_bias) L.bo = upload_new(vec(n.get(p + "attn.out_proj.bias"), H, "hidden-size"));
    if (s.moe_every > 0 && i % s.moe_every == 1) {
      // NomicMoELayer (nomic.rs:205-296): router.layer.weight [E, H] (rows padded to a multiple
      // of 8 for the logits' row stride), experts.mlp.w1 / w2 [E * I, H], experts.bias [H].  w2
      // is used as h [n, I] x w2_e [I, H] (`:268-275`), so each expert's block is transposed
      // once here to the [N, K] form the GEMM takes.
      const int E = s.num_experts, Epad = static_cast<int>(align_up(static_cast<size_t>(E), 8));
      const StTensor& rw = n.get(p + "mlp.router.layer.weight");
      expect_shape(rw, {E, H}, p + "mlp.router.layer.weight");
      L.moe_router = dev_alloc(static_cast<size_t>(Epad) * H * 2);
      TEI_CUDA(cudaMemsetAsync(L.moe_router, 0, static_cast<size_t>(Epad) * H * 2, stream_));
      upload(L.moe_router, 0, rw);
      const StTensor& w1 = n.get(p + "mlp.experts.mlp.w1");
      const StTensor& w2 = n.get(p + "mlp.experts.mlp.w2");
      expect_shape(w1, {static_cast<int64_t>(E) * I, H}, p + "mlp.experts.mlp.w1");
      expect_shape(w2, {static_cast<int64_t>(E) * I, H}, p + "mlp.experts.mlp.w2");
      L.moe_w1 = upload_new(w1);
      const size_t es = w2.nbytes / static_cast<size_t>(w2.numel());
      std::vector<uint8_t> tr(w2.nbytes);
      for (int e = 0; e < E; ++e) {
        const uint8_t* src = w2.data + static_cast<size_t>(e) * I * H * es;
        uint8_t* dst = tr.data() + static_cast<size_t>(e) * I * H * es;
        for (int r = 0; r < I; ++r) {
          for (int cidx = 0; cidx < H; ++cidx) {
            std::memcpy(dst + (static_cast<size_t>(cidx) * I + r) * es, src + (static_cast<size_t>(r) * H + cidx) * es, es);
          }
        }
      }
      StTensor w2t = w2;
      w2t.data = tr.data();
      w2t.shape = {static_cast<int64_t>(E) * H, I};
      L.moe_w2t = upload_new(w2t);
      TEI_CUDA(cudaStreamSynchronize(stream_));  // `tr` goes out of scope
      L.moe_bias = upload_new(vec(n.get(p + "mlp.experts.bias"), H, "hidden-size"));
      L.ln1_g = upload_new(vec(n.ln_w(p + "norm1"), H, "hidden-size"));
      L.ln1_b = upload_new(vec(n.ln_b(p + "norm1"), H, "hidden-size"));
      L.ln2_g = upload_new(vec(n.ln_w(p + "norm2"), H, "hidden-size"));
      L.ln2_b = upload_new(vec(n.ln_b(p + "norm2"), H, "hidden-size"));
      continue;
    }
    if (s.gated) {
      // fc1 = cat[fc12; fc11] and swiglu = silu(first half) * second half (nomic.rs:109-121):
      // fc12 is the gate, fc11 the up projection.
      expect_shape(n.get(p + "mlp.fc11.weight"), {I, H}, p + "mlp.fc11.weight");
      expect_shape(n.get(p + "mlp.fc12.weight"), {I, H}, p + "mlp.fc12.weight");
      L.w1 = dev_alloc(static_cast<size_t>(2) * I * H * 2);
      upload_rows_interleaved(L.w1, n.get(p + "mlp.fc12.weight"), n.get(p + "mlp.fc11.weight"));
      if (s.fc1_bias) {
        L.b1 = dev_alloc(static_cast<size_t>(2) * I * 2);
        upload_rows_interleaved(L.b1, vec(n.get(p + "mlp.fc12.bias"), I, "fc12 bias"), vec(n.get(p + "mlp.fc11.bias"), I, "fc11 bias"));
      }
    } else {
      expect_shape(n.get(p + "mlp.fc1.weight"), {I, H}, p + "mlp.fc1.weight");
      L.w1 = upload_new(n.get(p + "mlp.fc1.weight"));
      if (s.fc1_bias) L.b1 = upload_new(vec(n.get(p + "mlp.fc1.bias"), I, "feed-forward bias"));
    }
    expect_shape(n.get(p + "mlp.fc2.weight"), {H, I}, p + "mlp.fc2.weight");
    L.w2 = upload_new(n.get(p + "mlp.fc2.weight"));
    if (s.fc2_bias) L.b2 = upload_new(vec(n.get(p + "mlp.fc2.bias"), H, "hidden-size"));
    L.ln1_g = upload_new(vec(n.ln_w(p + "norm1"), H, "hidden-size"));
    L.ln1_b = upload_new(vec(n.ln_b(p + "norm1"), H, "hidden-size"));
    L.ln2_g = upload_new(vec(n.ln_w(p + "norm2"), H, "hidden-size"));
    L.ln2_b = upload_new(vec(n.ln_b(p + "norm2"), H, "hidden-size"));
  }
}

void Replica::load_gte(const SafeTensors& st) {
  const ModelSpec& s = spec_;
  const int H = s.hidden, I = s.inter;
  // flash_gte.rs:197-199: names under `new.` or bare.
  Names n{st, st.contains("new.embeddings.word_embeddings.weight") ? "new." : ""};
  Names root{st, ""};
  expect_shape(n.get("embeddings.word_embeddings.weight"), {s.vocab, H}, "embeddings.word_embeddings.weight");
  word_ = upload_new(n.get("embeddings.word_embeddings.weight"));
  if (s.type_vocab > 0) {
    expect_shape(n.get("embeddings.token_type_embeddings.weight"), {s.type_vocab, H}, "embeddings.token_type_embeddings.weight");
    type_tab_ = upload_new(n.get("embeddings.token_type_embeddings.weight"));
  }
  emb_g_ = upload_new(vec(n.ln_w("embeddings.LayerNorm"), H, "hidden-size"));
  emb_b_ = upload_new(vec(n.ln_b("embeddings.LayerNorm"), H, "hidden-size"));
  for (int i = 0; i < s.layers; ++i) {
    LayerW& L = layers_[i];
    const std::string p = "encoder.layer." + std::to_string(i) + ".";
    expect_shape(n.get(p + "attention.qkv_proj.weight"), {3 * H, H}, p + "attention.qkv_proj.weight");
    L.wqkv = upload_new(n.get(p + "attention.qkv_proj.weight"));
    L.bqkv = upload_new(vec(n.get(p + "attention.qkv_proj.bias"), s.qkv_width(), "qkv bias"));
    expect_shape(n.get(p + "attention.o_proj.weight"), {H, H}, p + "attention.o_proj.weight");
    L.wo = upload_new(n.get(p + "attention.o_proj.weight"));
    L.bo = upload_new(vec(n.get(p + "attention.o_proj.bias"), H, "hidden-size"));
    // mlp.up_gate_proj [2I, H]: rows [0, I) are `up`, rows [I, 2I) the gate that goes through the
    // activation (gte.rs:219-226).
    const StTensor& ug = n.get(p + "mlp.up_gate_proj.weight");
    expect_shape(ug, {2 * I, H}, p + "mlp.up_gate_proj.weight");
    StTensor up = ug, gate = ug;
    up.shape = {I, H};
    gate.shape = {I, H};
    up.nbytes = gate.nbytes = ug.nbytes / 2;
    gate.data = ug.data + ug.nbytes / 2;
    L.w1 = dev_alloc(static_cast<size_t>(2) * I * H * 2);
    upload_rows_interleaved(L.w1, gate, up);
    expect_shape(n.get(p + "mlp.down_proj.weight"), {H, I}, p + "mlp.down_proj.weight");
    L.w2 = upload_new(n.get(p + "mlp.down_proj.weight"));
    L.b2 = upload_new(vec(n.get(p + "mlp.down_proj.bias"), H, "hidden-size"));
    L.ln1_g = upload_new(vec(n.ln_w(p + "attn_ln"), H, "hidden-size"));
    L.ln1_b = upload_new(vec(n.ln_b(p + "attn_ln"), H, "hidden-size"));
    L.ln2_g = upload_new(vec(n.ln_w(p + "mlp_ln"), H, "hidden-size"));
    L.ln2_b = upload_new(vec(n.ln_b(p + "mlp_ln"), H, "hidden-size"));
  }
  if (s.classifier) {  // GTEClassificationHead, gte.rs:282-340: optional pooler.dense + tanh, classifier
    if (n.has("pooler.dense.weight") && n.has("pooler.dense.bias")) {
      expect_shape(n.get("pooler.dense.weight"), {H, H}, "pooler.dense.weight");
      cls_dense_w_ = upload_new(n.get("pooler.dense.weight"));
      cls_dense_b_ = upload_new(vec(n.get("pooler.dense.bias"), H, "hidden-size"));
    }
    expect_shape(root.get("classifier.weight"), {s.n_classes, H}, "classifier.weight");
    cls_out_w_ = upload_new(root.get("classifier.weight"));
    cls_out_b_ = upload_new(vec(root.get("classifier.bias"), s.n_classes, "classifier bias"));
  }
}

void Replica::load_qwen3(const SafeTensors& st) {
  const ModelSpec& s = spec_;
  const int H = s.hidden, I = s.inter, Q = s.q_width(), KV = s.kv_width();
  // Optional `model.` prefix (flash_qwen3.rs:322-326).
  Names n{st, st.contains("model.embed_tokens.weight") ? "model." : ""};
  expect_shape(n.get("embed_tokens.weight"), {s.vocab, H}, "embed_tokens.weight");
  word_ = upload_new(n.get("embed_tokens.weight"));
  for (int i = 0; i < s.layers; ++i) {
    LayerW& L = layers_[i];
    const std::string p = "layers." + std::to_string(i) + ".";
    // The reference runs q, k and v as three GEMMs (flash_qwen3.rs:119-121); their weights are
    // stacked here so that one GEMM produces the [T, Q + 2 KV] activation.
    expect_shape(n.get(p + "self_attn.q_proj.weight"), {Q, H}, p + "self_attn.q_proj.weight");
    expect_shape(n.get(p + "self_attn.k_proj.weight"), {KV, H}, p + "self_attn.k_proj.weight");
    expect_shape(n.get(p + "self_attn.v_proj.weight"), {KV, H}, p + "self_attn.v_proj.weight");
    L.wqkv = dev_alloc(static_cast<size_t>(Q + 2 * KV) * H * 2);
    upload(L.wqkv, 0, n.get(p + "self_attn.q_proj.weight"));
    upload(L.wqkv, static_cast<size_t>(Q) * H, n.get(p + "self_attn.k_proj.weight"));
    upload(L.wqkv, static_cast<size_t>(Q + KV) * H, n.get(p + "self_attn.v_proj.weight"));
    expect_shape(n.get(p + "self_attn.o_proj.weight"), {H, Q}, p + "self_attn.o_proj.weight");
    L.wo = upload_new(n.get(p + "self_attn.o_proj.weight"));
    if (s.qkv_bias) {  // flash_qwen2.rs:37-57
      L.bqkv = dev_alloc(static_cast<size_t>(Q + 2 * KV) * 2);
      upload(L.bqkv, 0, vec(n.get(p + "self_attn.q_proj.bias"), Q, "q bias"));
      upload(L.bqkv, static_cast<size_t>(Q), vec(n.get(p + "self_attn.k_proj.bias"), KV, "k bias"));
      upload(L.bqkv, static_cast<size_t>(Q + KV), vec(n.get(p + "self_attn.v_proj.bias"), KV, "v bias"));
    }
    if (s.qk_norm) {
      L.q_norm = upload_new(vec(n.get(p + "self_attn.q_norm.weight"), s.head_dim, "q_norm"));
      L.k_norm = upload_new(vec(n.get(p + "self_attn.k_norm.weight"), s.head_dim, "k_norm"));
    }
    expect_shape(n.get(p + "mlp.gate_proj.weight"), {I, H}, p + "mlp.gate_proj.weight");
    expect_shape(n.get(p + "mlp.up_proj.weight"), {I, H}, p + "mlp.up_proj.weight");
    L.w1 = dev_alloc(static_cast<size_t>(2) * I * H * 2);
    upload_rows_interleaved(L.w1, n.get(p + "mlp.gate_proj.weight"), n.get(p + "mlp.up_proj.weight"));
    expect_shape(n.get(p + "mlp.down_proj.weight"), {H, I}, p + "mlp.down_proj.weight");
    L.w2 = upload_new(n.get(p + "mlp.down_proj.weight"));
    L.ln1_g = upload_new(vec(n.get(p + "input_layernorm.weight"), H, "hidden-size"));
    L.ln2_g = upload_new(vec(n.get(p + "post_attention_layernorm.weight"), H, "hidden-size"));
  }
  final_norm_ = upload_new(vec(n.get("norm.weight"), H, "hidden-size"));
  if (st.contains("linear.weight")) {  // flash_qwen3.rs:344-357
    const StTensor& w = st.get("linear.weight");
    if (w.shape.size() != 2 || w.shape[1] != H) throw TeiError(ERR_START, "unexpected shape for tensor linear.weight");
    if (w.shape[0] % 8 != 0 || w.shape[0] > H) throw TeiError(ERR_START, "projection width must be a multiple of 8 and at most hidden_size");
    projection_ = upload_new(w);
    projection_dim_ = static_cast<int>(w.shape[0]);
  }
}

void Replica::load_modernbert(const SafeTensors& st) {
  const ModelSpec& s = spec_;
  const int H = s.hidden, I = s.inter;
  // flash_modernbert.rs:279-293: names under `model.` or bare.
  Names n{st, st.contains("model.embeddings.tok_embeddings.weight") ? "model." : ""};
  Names root{st, ""};
  expect_shape(n.get("embeddings.tok_embeddings.weight"), {s.vocab, H}, "embeddings.tok_embeddings.weight");
  word_ = upload_new(n.get("embeddings.tok_embeddings.weight"));
  emb_g_ = upload_new(vec(n.get("embeddings.norm.weight"), H, "hidden-size"));  // LayerNormNoBias: weight only
  for (int i = 0; i < s.layers; ++i) {
    LayerW& L = layers_[i];
    const std::string p = "layers." + std::to_string(i) + ".";
    if (i != 0) L.ln1_g = upload_new(vec(n.get(p + "attn_norm.weight"), H, "hidden-size"));  // layer 0 has none (:131-139)
    expect_shape(n.get(p + "attn.Wqkv.weight"), {3 * H, H}, p + "attn.Wqkv.weight");
    L.wqkv = upload_new(n.get(p + "attn.Wqkv.weight"));
    if (n.has(p + "attn.Wqkv.bias")) L.bqkv = upload_new(vec(n.get(p + "attn.Wqkv.bias"), s.qkv_width(), "qkv bias"));
    expect_shape(n.get(p + "attn.Wo.weight"), {H, H}, p + "attn.Wo.weight");
    L.wo = upload_new(n.get(p + "attn.Wo.weight"));
    if (n.has(p + "attn.Wo.bias")) L.bo = upload_new(vec(n.get(p + "attn.Wo.bias"), H, "hidden-size"));
    L.ln2_g = upload_new(vec(n.get(p + "mlp_norm.weight"), H, "hidden-size"));
    // mlp.Wi [2I, H]: rows [0, I) go through the activation, rows [I, 2I) gate them.
    const StTensor& wi = n.get(p + "mlp.Wi.weight");
    expect_shape(wi, {2 * I, H}, p + "mlp.Wi.weight");
    auto halves = [](const StTensor& t, StTensor& a, StTensor& b) {
      a = t;
      b = t;
      a.shape[0] = b.shape[0] = t.shape[0] / 2;
      a.nbytes = b.nbytes = t.nbytes / 2;
      b.data = t.data + t.nbytes / 2;
    };
    StTensor ga, up;
    halves(wi, ga, up);
    L.w1 = dev_alloc(static_cast<size_t>(2) * I * H * 2);
    upload_rows_interleaved(L.w1, ga, up);
    if (n.has(p + "mlp.Wi.bias")) {
      StTensor ba, bu;
      halves(vec(n.get(p + "mlp.Wi.bias"), 2 * I, "Wi bias"), ba, bu);
      L.b1 = dev_alloc(static_cast<size_t>(2) * I * 2);
      upload_rows_interleaved(L.b1, ba, bu);
    }
    expect_shape(n.get(p + "mlp.Wo.weight"), {H, I}, p + "mlp.Wo.weight");
    L.w2 = upload_new(n.get(p + "mlp.Wo.weight"));
    if (n.has(p + "mlp.Wo.bias")) L.b2 = upload_new(vec(n.get(p + "mlp.Wo.bias"), H, "hidden-size"));
  }
  final_norm_ = upload_new(vec(n.get("final_norm.weight"), H, "hidden-size"));
  if (s.classifier) {  // ModernBertClassificationHead::load, modernbert.rs:408-440
    expect_shape(root.get("head.dense.weight"), {H, H}, "head.dense.weight");
    cls_dense_w_ = upload_new(root.get("head.dense.weight"));
    cls_norm_g_ = upload_new(vec(root.get("head.norm.weight"), H, "hidden-size"));
    expect_shape(root.get("classifier.weight"), {s.n_classes, H}, "classifier.weight");
    cls_out_w_ = upload_new(root.get("classifier.weight"));
    cls_out_b_ = upload_new(vec(root.get("classifier.bias"), s.n_classes, "classifier bias"));
  }
}

void Replica::build_rope_tables() {
  // layers/rotary.rs:29-116: inv_freq_i = 1 / base^(i / dim) for even i, angle = pos * inv_freq,
  // all in f32.  The tables stay in fp32 on the device.
  const int dh = spec_.head_dim, half = dh / 2, len = spec_.rope_table_len;
  auto fill = [&](float base, float** d_cos, float** d_sin) {
    std::vector<float> inv(half);
    for (int i = 0; i < half; ++i) inv[i] = 1.0f / std::pow(base, static_cast<float>(2 * i) / static_cast<float>(dh));
    if (spec_.rope_ntk_factor > 0.f) {
      // RopeScaling::Ntk (layers/rotary.rs:86-93): base * factor, then divided by factor^(2 / dim)
      const float f = spec_.rope_ntk_factor;
      const float sdiv = std::pow(f, 2.0f / static_cast<float>(dh));
      for (int i = 0; i < half; ++i) {
        inv[i] = (1.0f / std::pow(base * f, static_cast<float>(2 * i) / static_cast<float>(dh))) / sdiv;
      }
    }
    if (spec_.rope_l3_factor > 0.f) {
      // RopeScaling::Llama3 (layers/rotary.rs:46-85): short wavelengths keep their frequency,
      // long ones are divided by the factor, the band between is blended; all in f32.
      const float old_len = spec_.rope_l3_orig_max;
      const float low_wavelen = old_len / spec_.rope_l3_low, high_wavelen = old_len / spec_.rope_l3_high;
      for (int i = 0; i < half; ++i) {
        const float inv_base = inv[i];
        const float wavelen = 2.0f * 3.14159265358979323846f / inv_base;
        if (wavelen < high_wavelen) continue;
        if (wavelen > low_wavelen) {
          inv[i] = inv_base / spec_.rope_l3_factor;
        } else {
          const float smooth = (old_len / wavelen - spec_.rope_l3_low) / (spec_.rope_l3_high - spec_.rope_l3_low);
          inv[i] = (1.0f - smooth) * (inv_base / spec_.rope_l3_factor) + smooth * inv_base;
        }
      }
    }
    std::vector<float> c(static_cast<size_t>(len) * half), s(static_cast<size_t>(len) * half);
    for (int p = 0; p < len; ++p) {
      for (int i = 0; i < half; ++i) {
        const float a = static_cast<float>(p) * inv[i];
        c[static_cast<size_t>(p) * half + i] = std::cos(a);
        s[static_cast<size_t>(p) * half + i] = std::sin(a);
      }
    }
    *d_cos = static_cast<float*>(dev_alloc(c.size() * 4));
    *d_sin = static_cast<float*>(dev_alloc(s.size() * 4));
    TEI_CUDA(cudaMemcpy(*d_cos, c.data(), c.size() * 4, cudaMemcpyHostToDevice));
    TEI_CUDA(cudaMemcpy(*d_sin, s.data(), s.size() * 4, cudaMemcpyHostToDevice));
  };
  fill(spec_.rope_theta, &cos_, &sin_);
  // ModernBERT: a second pair of tables for the local-attention layers (flash_modernbert.rs:299-313)
  if (spec_.modernbert) fill(spec_.local_theta, &cos_scaled_, &sin_scaled_);
  if (spec_.arch == ARCH_NOMIC && spec_.rope_scaling_factor > 0.f) {
    // flash_nomic.rs:244-258, including its integer exponent: powi((dim / (dim - 2)) as i32).
    const float sf = spec_.rope_scaling_factor;
    const float inner = spec_.rope_theta * ((sf * static_cast<float>(spec_.rope_table_len) /
                                             static_cast<float>(spec_.nomic_max_pos)) - (sf - 1.0f));
    const int expo = static_cast<int>(static_cast<float>(dh) / (static_cast<float>(dh) - 2.0f));
    float nb = 1.0f;
    for (int i = 0; i < expo; ++i) nb *= inner;
    fill(nb, &cos_scaled_, &sin_scaled_);
  }
}

// ------------------------------------------------------------------------------ workspace
void Replica::ensure_workspace(size_t tokens, size_t seqs, size_t n_work, size_t n_pooled,
                               size_t raw_rows) {
  const ModelSpec& s = spec_;
  // integer inputs
  const size_t ints_need = 3 * tokens + (seqs + 1) + 2 * seqs + raw_rows + 12 * n_work + 64;  // up to three work lists
  if (ints_need > ints_cap_) {
    TEI_CUDA(cudaStreamSynchronize(stream_));
    if (d_ints_) cudaFree(d_ints_);
    if (h_ints_) cudaFreeHost(h_ints_);
    d_ints_ = nullptr;
    h_ints_ = nullptr;
    ints_cap_ = ints_need + ints_need / 4;
    TEI_CUDA(cudaMalloc(&d_ints_, ints_cap_ * 4));
    TEI_CUDA(cudaMallocHost(&h_ints_, ints_cap_ * 4));
  }
  // outputs (+ head scratch after them)
  const size_t D = static_cast<size_t>(output_dim());
  const size_t Dpad = align_up(D, 8);
  const size_t Draw = align_up(static_cast<size_t>(raw_dim()), 8);
  size_t dense_w = 0;  // widest row of the Dense chain (two ping-pong buffers of pooled rows)
  if (!dense_.empty()) {
    dense_w = Draw;
    for (const DenseW& d : dense_) dense_w = std::max(dense_w, align_up(static_cast<size_t>(d.out), 8));
  }
  const size_t out_need = 64 + n_pooled * Dpad + raw_rows * Draw +
                          seqs * static_cast<size_t>(std::max(s.n_classes, 1)) +
                          2 * seqs * static_cast<size_t>(s.hidden) + 2 * n_pooled * dense_w + 64;
  if (out_need > out_cap_floats_) {
    TEI_CUDA(cudaStreamSynchronize(stream_));
    if (d_out_) cudaFree(d_out_);
    if (h_out_) cudaFreeHost(h_out_);
    d_out_ = nullptr;
    h_out_ = nullptr;
    out_cap_floats_ = out_need + out_need / 4;
    TEI_CUDA(cudaMalloc(&d_out_, out_cap_floats_ * 4));
    TEI_CUDA(cudaMallocHost(&h_out_, out_cap_floats_ * 4));
  }
  if (tokens <= cap_tokens_) return;
  TEI_CUDA(cudaStreamSynchronize(stream_));
  if (arena_) cudaFree(arena_);
  arena_ = nullptr;
  const size_t cap = align_up(tokens, 256);
  const size_t H = s.hidden;
  const size_t sz_h = align_up(cap * H * 2, 1024);
  const size_t sz_qkv = align_up(cap * static_cast<size_t>(s.qkv_width()) * 2, 1024);
  const size_t sz_attn = align_up(cap * static_cast<size_t>(s.q_width()) * 2, 1024);
  const size_t sz_ffn = align_up(cap * static_cast<size_t>(s.inter) * 2, 1024);
  const size_t sz_res = s.arch == ARCH_QWEN3 ? align_up(cap * H * 4, 1024) : 0;
  const size_t vpad = align_up(static_cast<size_t>(s.vocab), 8);
  const size_t sz_spl = s.pool == POOL_SPLADE ? align_up(cap * vpad * 2, 1024) : 0;
  // mixture of experts: every expert owns `cap` rows of the gathered buffers (a token goes to an
  // expert at most once, so cap rows always suffice)
  const size_t E = static_cast<size_t>(s.num_experts), topk = static_cast<size_t>(s.moe_top_k);
  const bool moe = s.moe_every > 0;
  const size_t sz_xg = moe ? align_up(E * cap * H * 2, 1024) : 0;
  const size_t sz_hg = moe ? align_up(E * cap * static_cast<size_t>(s.inter) * 2, 1024) : 0;
  const size_t sz_lg = moe ? align_up(cap * align_up(E, 8) * 2, 1024) : 0;
  const size_t sz_tk = moe ? align_up(cap * topk * 4, 1024) : 0;
  const size_t total = 3 * sz_h + sz_qkv + sz_attn + sz_ffn + sz_res + sz_spl + 2 * sz_xg + sz_hg + sz_lg +
                       3 * sz_tk + (moe ? 1024 : 0);
  TEI_CUDA(cudaMalloc(&arena_, total));
  arena_bytes_ = total;
  uint8_t* p = static_cast<uint8_t*>(arena_);
  x_ = p; p += sz_h;
  x1_ = p; p += sz_h;
  tmp_ = p; p += sz_h;
  qkv_ = p; p += sz_qkv;
  attn_ = p; p += sz_attn;
  ffn_ = p; p += sz_ffn;
  resid_ = sz_res ? reinterpret_cast<float*>(p) : nullptr; p += sz_res;
  splade_ = sz_spl ? p : nullptr; p += sz_spl;
  if (sz_spl) TEI_CUDA(cudaMemsetAsync(splade_, 0, sz_spl, stream_));
  if (moe) {
    moe_xg_ = p; p += sz_xg;
    moe_yg_ = p; p += sz_xg;
    moe_hg_ = p; p += sz_hg;
    moe_logits_ = p; p += sz_lg;
    moe_topk_e_ = reinterpret_cast<int*>(p); p += sz_tk;
    moe_pos_ = reinterpret_cast<int*>(p); p += sz_tk;
    moe_topk_w_ = reinterpret_cast<float*>(p); p += sz_tk;
    moe_counts_ = reinterpret_cast<int*>(p); p += 1024;
    moe_cap_ = cap;
  }
  cap_tokens_ = cap;
}

// ------------------------------------------------------------------------------ stage
void Replica::stage(const HostBatch& b, bool predict, bool normalize) {
  TEI_CUDA(cudaSetDevice(device_));
  // The pinned block is rewritten below: an earlier batch's copy or forward that is still in
  // flight (stage, run, stage again without a sync or fetch between) must be through with it.
  // After a fetch or sync the stream is idle and this returns at once.
  TEI_CUDA(cudaStreamSynchronize(stream_));
  const ModelSpec& s = spec_;
  if (b.n_seqs == 0 || b.n_tokens == 0) throw TeiError(ERR_INFERENCE, "empty batch");
  if (!b.input_ids || !b.cu_seqlens || !b.position_ids) throw TeiError(ERR_INFERENCE, "null batch pointer");
  if (b.n_tokens > 0x7fffffffu / 8) throw TeiError(ERR_INFERENCE, "batch too large");
  if (predict && !s.classifier) throw TeiError(ERR_INFERENCE, "`predict` is not implemented for this model");
  if (b.cu_seqlens[0] != 0 || b.cu_seqlens[b.n_seqs] != b.n_tokens) {
    throw TeiError(ERR_INFERENCE, "cumulative_seq_lengths must start at 0 and end at the token count");
  }
  uint32_t max_len = 0;
  for (size_t i = 0; i < b.n_seqs; ++i) {
    if (b.cu_seqlens[i + 1] <= b.cu_seqlens[i]) {
      throw TeiError(ERR_INFERENCE, "cumulative_seq_lengths must be strictly increasing");
    }
    max_len = std::max(max_len, b.cu_seqlens[i + 1] - b.cu_seqlens[i]);
  }
  // ALiBi models have no position table to index (flash_jina.rs never reads position_ids then).
  const uint32_t pos_limit = s.alibi ? 0xffffffffu : static_cast<uint32_t>(s.arch == ARCH_BERT ? s.max_pos : s.rope_table_len);
  const bool use_types = s.arch != ARCH_QWEN3 && s.type_vocab > 0;  // DistilBERT and the decoders have no token types
  if (use_types && !b.token_type_ids) throw TeiError(ERR_INFERENCE, "null token_type_ids");
  // Branch-free passes (they vectorise): the largest value of each array is compared once.
  uint32_t max_id = 0, max_pos = 0, max_type = 0;
  for (size_t t = 0; t < b.n_tokens; ++t) max_id = std::max(max_id, b.input_ids[t]);
  for (size_t t = 0; t < b.n_tokens; ++t) max_pos = std::max(max_pos, b.position_ids[t]);
  if (use_types) {
    for (size_t t = 0; t < b.n_tokens; ++t) max_type = std::max(max_type, b.token_type_ids[t]);
  }
  if (max_id >= static_cast<uint32_t>(s.vocab)) throw TeiError(ERR_INFERENCE, "input id out of the vocabulary");
  if (max_pos >= pos_limit) throw TeiError(ERR_INFERENCE, "position id beyond the position table");
  if (use_types && max_type >= static_cast<uint32_t>(s.type_vocab)) {
    throw TeiError(ERR_INFERENCE, "token type id out of range");
  }
  size_t n_pooled = predict ? 0 : b.n_pooled;
  size_t n_raw = predict ? 0 : b.n_raw;
  for (size_t i = 0; i < n_pooled; ++i) {
    if (b.pooled_indices[i] >= b.n_seqs) throw TeiError(ERR_INFERENCE, "pooled index out of range");
  }
  size_t raw_rows = 0;
  for (size_t i = 0; i < n_raw; ++i) {
    if (b.raw_indices[i] >= b.n_seqs) throw TeiError(ERR_INFERENCE, "raw index out of range");
    raw_rows += b.cu_seqlens[b.raw_indices[i] + 1] - b.cu_seqlens[b.raw_indices[i]];
  }
  if (s.pool == POOL_SPLADE && n_raw > 0) throw TeiError(ERR_INFERENCE, "raw embeddings are not available with splade pooling");

  std::vector<int> cu_i(b.n_seqs + 1);
  for (size_t i = 0; i <= b.n_seqs; ++i) cu_i[i] = static_cast<int>(b.cu_seqlens[i]);
  const size_t n_work = static_cast<size_t>(count_attention_items(cu_i.data(), static_cast<int>(b.n_seqs)));
  ensure_workspace(b.n_tokens, b.n_seqs, n_work, n_pooled, raw_rows);

  T_ = b.n_tokens;
  B_ = b.n_seqs;
  n_work_ = n_work;
  n_pooled_ = n_pooled;
  n_raw_rows_ = raw_rows;
  max_length_ = max_len;
  predict_ = predict;
  normalize_ = normalize;

  // One pinned block, one copy: ids | types | pos | cu | pooled idx | all idx | raw rows | work.
  int32_t* h = h_ints_;
  size_t off = 0;
  auto put_u32 = [&](const uint32_t* src, size_t n) {
    size_t o = off;
    if (src) std::memcpy(h + off, src, n * 4);
    else std::memset(h + off, 0, n * 4);
    off += n;
    return o;
  };
  const size_t o_ids = put_u32(b.input_ids, T_);
  const size_t o_types = put_u32(use_types ? b.token_type_ids : nullptr, T_);
  const size_t o_pos = put_u32(b.position_ids, T_);
  const size_t o_cu = put_u32(b.cu_seqlens, B_ + 1);
  const size_t o_pidx = put_u32(n_pooled ? b.pooled_indices : nullptr, n_pooled);
  const size_t o_all = off;
  for (size_t i = 0; i < B_; ++i) h[off++] = static_cast<int32_t>(i);
  const size_t o_raw = off;
  for (size_t i = 0; i < n_raw; ++i) {
    const uint32_t sidx = b.raw_indices[i];
    for (uint32_t r = b.cu_seqlens[sidx]; r < b.cu_seqlens[sidx + 1]; ++r) h[off++] = static_cast<int32_t>(r);
  }
  off = align_up(off, 4);
  const size_t o_work = off;
  const int n_planned = plan_attention(cu_i.data(), static_cast<int>(B_), s.causal ? 1 : 0, h + off,
                                       static_cast<int>(n_work), s.window_left, -1);
  if (static_cast<size_t>(n_planned) != n_work) throw TeiError(ERR_INFERENCE, "attention planning mismatch");
  off += 4 * n_work;
  size_t o_work_local = 0;
  if (s.local_window >= 0) {  // the layers with the two-sided window walk their own list
    o_work_local = off;
    const int n_local = plan_attention(cu_i.data(), static_cast<int>(B_), 0, h + off, static_cast<int>(n_work),
                                       s.local_window, s.local_window);
    if (static_cast<size_t>(n_local) != n_work) throw TeiError(ERR_INFERENCE, "attention planning mismatch");
    off += 4 * n_work;
  }
  // Last-layer shortcut of the post-LN BERT family (see forward_bert): needs room for five packed
  // [B, H] blocks inside one [T, H] buffer.
  size_t o_work_first = 0;
  const bool first_rows_enabled = last_layer_shortcut_;
  const bool post_ln_family = (s.arch == ARCH_BERT && !s.jina_code) ||
                              (s.arch == ARCH_NOMIC && !layers_.empty() && !layers_.back().moe_router);
  first_rows_only_ = first_rows_enabled && post_ln_family && s.layers > 0 && s.local_window < 0 &&
                     n_raw == 0 && (predict || s.pool == POOL_CLS) && 5 * B_ <= T_;
  // The pre-norm decoders (forward_qwen3) do the same for CLS and last-token pooling; their
  // packed blocks are [B, Q] + four [B, H] inside x1_ and [B, 2I] + an fp32 [B, H] inside ffn_.
  const bool one_row_decoder =
      first_rows_enabled && s.arch == ARCH_QWEN3 && !projection_ && s.layers > 0 && n_raw == 0 &&
      !predict && (s.pool == POOL_CLS || s.pool == POOL_LAST) &&
      B_ * (static_cast<size_t>(s.q_width()) + 4 * s.hidden) <= T_ * static_cast<size_t>(s.hidden) &&
      B_ * (static_cast<size_t>(s.inter) * 4 + static_cast<size_t>(s.hidden) * 4 + 64) <= T_ * static_cast<size_t>(s.inter) * 2;
  const bool last_row = one_row_decoder && s.pool == POOL_LAST;
  first_rows_only_ = first_rows_only_ || one_row_decoder;
  n_work_first_ = 0;
  if (first_rows_only_) {
    o_work_first = off;
    // ModernBERT: the last layer may be one of those with the two-sided window and its own list
    const bool last_is_local = s.modernbert && s.local_window >= 0 && ((s.layers - 1) % s.global_every != 0);
    const int32_t* all = h + (last_is_local ? o_work_local : o_work);
    for (size_t i = 0; i < n_work; ++i) {
      // keep the query tile that holds the row: the first one, or the last one of the sequence
      const bool keep = last_row ? all[4 * i + 2] + 128 >= all[4 * i + 1] : all[4 * i + 2] == 0;
      if (!keep) continue;
      std::memcpy(h + off, all + 4 * i, 16);
      off += 4;
      ++n_work_first_;
    }
  }
  TEI_CUDA(cudaMemcpyAsync(d_ints_, h_ints_, off * 4, cudaMemcpyHostToDevice, stream_));
  stats_.last_h2d_bytes = static_cast<double>(off * 4);
  d_work_first_ = first_rows_only_ ? d_ints_ + o_work_first : nullptr;
  d_ids_ = d_ints_ + o_ids;
  d_types_ = d_ints_ + o_types;
  d_pos_ = d_ints_ + o_pos;
  d_cu_ = d_ints_ + o_cu;
  d_pooled_idx_ = d_ints_ + o_pidx;
  d_all_idx_ = d_ints_ + o_all;
  d_raw_rows_ = d_ints_ + o_raw;
  d_work_ = d_ints_ + o_work;
  d_work_local_ = s.local_window >= 0 ? d_ints_ + o_work_local : nullptr;

  // Output block: [0,64) status word | pooled | raw | scores || scratch (not copied back).
  const size_t D = static_cast<size_t>(output_dim());
  // The Dense chain writes rows of exactly D floats; the pooling kernel rows of Dpad.
  pooled_ld_ = dense_.empty() ? align_up(D, 8) : D;
  size_t oo = 64;
  d_pooled_ = d_out_ + oo; oo += align_up(n_pooled * pooled_ld_, 8);
  d_raw_ = d_out_ + oo; oo += raw_rows * static_cast<size_t>(raw_dim());
  d_scores_ = d_out_ + oo; oo += predict ? B_ * static_cast<size_t>(s.n_classes) : 0;
  out_floats_ = oo;
  oo = align_up(oo, 8);
  d_cls_ = d_out_ + oo; oo += B_ * s.hidden;
  d_head_tmp_ = d_out_ + oo; oo += B_ * s.hidden;
  if (!dense_.empty()) {
    size_t dense_w = align_up(static_cast<size_t>(raw_dim()), 8);
    for (const DenseW& d : dense_) dense_w = std::max(dense_w, align_up(static_cast<size_t>(d.out), 8));
    d_dense_a_ = d_out_ + oo; oo += n_pooled * dense_w;
    d_dense_b_ = d_out_ + oo;
  }
  TEI_CUDA(cudaMemsetAsync(d_out_, 0, 256, stream_));
}

// ------------------------------------------------------------------------------ forward
void Replica::run() {
  TEI_CUDA(cudaSetDevice(device_));
  launches_ = 0;
  TEI_CUDA(cudaEventRecord(ev_start_, stream_));
  switch (spec_.arch) {
    case ARCH_BERT: forward_bert(); break;
    case ARCH_NOMIC: forward_nomic(); break;
    case ARCH_QWEN3: forward_qwen3(); break;
  }
  pool_and_heads();
  if (inject_status_ != 0) {
    const int code = inject_status_;
    inject_status_ = 0;
    launch(launch_report_status(reinterpret_cast<int*>(d_out_), code, stream_), "status report");
  }
  TEI_CUDA(cudaEventRecord(ev_stop_, stream_));
  stats_.last_launches = launches_;
  stats_.last_tokens = static_cast<double>(T_);
}

namespace {
GemmArgs gemm_args(const void* a, const void* w, const void* bias, void* out, int M, int N, int K,
                   int lda, int ldo, int act, int dtype, int* status) {
  GemmArgs g;
  g.a = a; g.w = w; g.bias = bias; g.residual = nullptr; g.out = out;
  g.M = M; g.N = N; g.K = K; g.lda = lda; g.ldo = ldo; g.ldr = 0;
  g.act = act; g.dtype = dtype; g.status = status;
  return g;
}
// The feed-forward output projection of the post-LN models: with a long K loop (the tile's main
// loop then hides the epilogue's wait for the residual rows) the residual is added in the GEMM
// and the LayerNorm behind it reads one tensor instead of two.  The model runs the same form on
// every path (all rows or the last layer's first rows), so both keep giving the same bits.
bool residual_fits_epilogue(int N, int K) { return K >= 2048 && N % 64 == 0; }
}  // namespace

// The fused q/k/v projection of the rotary models.  q/k RMSNorm and RoPE run in the epilogue of
// the GEMM (head sizes 32, 64, 128); otherwise, or with the fusion switched off, as a second
// in-place kernel over the q and k columns.  Both give the same bits.
void Replica::qkv_projection(const void* x, const LayerW& L, int T, int W, int H, const RopeArgs& r, int* status) {
  const ModelSpec& s = spec_;
  GemmArgs g = gemm_args(x, L.wqkv, L.bqkv, qkv_, T, W, H, H, W, ACT_NONE, s.dtype, status);
  // By default the fused form runs where it is the faster one: RoPE alone.  With the q/k RMSNorm
  // of Qwen3 the epilogue needs the cos / sin rows and the norm weights of a whole head per thread
  // and outlasts the tile's main loop (1024 -> 4096 columns at 131,072 rows: 1.33 ms fused against
  // 0.79 + 0.27 ms), so there the second kernel stays unless the fusion is asked for.
  const bool want = fused_rope_ < 0 ? r.q_gamma == nullptr : fused_rope_ > 0;
  const bool fuse = want && (r.head_dim == 32 || r.head_dim == 64 || r.head_dim == 128);
  RopeFusion f;
  if (fuse) {
    f.pos_ids = r.pos_ids; f.cos_tab = r.cos_tab; f.sin_tab = r.sin_tab;
    f.q_gamma = r.q_gamma; f.k_gamma = r.k_gamma; f.head_dim = r.head_dim;
    f.q_cols = r.n_heads * r.head_dim; f.k_cols = r.n_kv_heads * r.head_dim; f.eps = r.eps;
    g.rope = &f;
  }
  LAUNCH(KC_GEMM, launch_gemm(g, stream_), "qkv projection");
  if (!fuse) LAUNCH(KC_ROPE, launch_qk_norm_rope(r, stream_), "q/k RMSNorm + rotary embedding");
}

void Replica::forward_bert() {
  const ModelSpec& s = spec_;
  const int T = static_cast<int>(T_), H = s.hidden, I = s.inter;
  int* status = reinterpret_cast<int*>(d_out_);
  EmbedArgs e;
  e.ids = d_ids_; e.type_ids = type_tab_ ? d_types_ : nullptr; e.pos_ids = pos_tab_ ? d_pos_ : nullptr;
  e.word = word_; e.type_tab = type_tab_; e.pos_tab = pos_tab_;
  e.gamma = emb_g_; e.beta = emb_b_; e.out = x_; e.T = T; e.H = H; e.eps = s.eps; e.dtype = s.dtype;
  LAUNCH(KC_EMBED, launch_embed_layernorm(e, stream_), "embeddings");
  uint8_t* qkv = static_cast<uint8_t*>(qkv_);
  for (int i = 0; i < s.layers; ++i) {
    const LayerW& L = layers_[i];
    LAUNCH(KC_GEMM, launch_gemm(gemm_args(x_, L.wqkv, L.bqkv, qkv_, T, 3 * H, H, H, 3 * H, ACT_NONE, s.dtype, status), stream_), "qkv projection");
    if (first_rows_only_ && i + 1 == s.layers) {
      // Only the first row of every sequence is read after this layer.  Keys and values are
      // there for every token; the scores are taken for the first query tile of each sequence
      // only, and the output projection, both LayerNorms and the feed-forward run on the B
      // first rows, packed into x1_ (five [B, H] blocks) and ffn_; the result goes back to the
      // rows' places in x_, where pooling and the heads look for it.
      const int B = static_cast<int>(B_);
      const size_t blk = static_cast<size_t>(B) * H * 2;
      uint8_t* c0 = static_cast<uint8_t*>(x1_);
      void *attn_c = c0, *res_c = c0 + blk, *tmp_c = c0 + 2 * blk, *x1_c = c0 + 3 * blk, *out_c = c0 + 4 * blk;
      AttnArgs a;
      a.q = qkv; a.k = qkv + static_cast<size_t>(H) * 2; a.v = qkv + static_cast<size_t>(2 * H) * 2;
      a.out = attn_; a.cu_seqlens = d_cu_; a.work_items = d_work_first_; a.n_work = static_cast<int>(n_work_first_);
      a.total_tokens = T; a.n_heads = s.heads; a.n_kv_heads = s.kv_heads; a.head_dim = s.head_dim;
      a.ld_q = a.ld_k = a.ld_v = 3 * H; a.ld_o = H; a.causal = 0;
      a.scale = static_cast<float>(1.0 / std::sqrt(static_cast<double>(s.head_dim)));
      a.alibi_slopes = alibi_slopes_; a.dtype = s.dtype; a.status = status;
      LAUNCH(KC_ATTENTION, launch_attention(a, stream_), "attention, first query tiles");
      LAUNCH(KC_POOL, launch_first_rows(attn_, attn_c, d_cu_, B, H * 2, 0, 0, stream_), "first rows of the attention output");
      LAUNCH(KC_POOL, launch_first_rows(x_, res_c, d_cu_, B, H * 2, 0, 0, stream_), "first rows of the layer input");
      LAUNCH(KC_GEMM, launch_gemm(gemm_args(attn_c, L.wo, L.bo, tmp_c, B, H, H, H, H, ACT_NONE, s.dtype, status), stream_), "attention output projection");
      NormArgs n1;
      n1.x = tmp_c; n1.residual = res_c; n1.gamma = L.ln1_g; n1.beta = L.ln1_b; n1.out = x1_c; n1.sum_out = nullptr;
      n1.T = B; n1.H = H; n1.eps = s.eps; n1.rms = 0; n1.dtype = s.dtype;
      LAUNCH(KC_NORM, launch_add_norm(n1, stream_), "attention LayerNorm");
      if (s.gated) {  // JinaBERT
        LAUNCH(KC_GEMM, launch_gemm(gemm_args(x1_c, L.w1, nullptr, ffn_, B, 2 * I, H, H, I, s.act, s.dtype, status), stream_), "gated projection");
      } else {
        LAUNCH(KC_GEMM, launch_gemm(gemm_args(x1_c, L.w1, L.b1, ffn_, B, I, H, H, I, s.act, s.dtype, status), stream_), "intermediate projection");
      }
      GemmArgs g2 = gemm_args(ffn_, L.w2, L.b2, tmp_c, B, H, I, I, H, ACT_NONE, s.dtype, status);
      const bool res_in_gemm = fused_residual_ && residual_fits_epilogue(H, I);
      if (res_in_gemm) g2.residual = x1_c, g2.ldr = H;
      LAUNCH(KC_GEMM, launch_gemm(g2, stream_), "output projection");
      NormArgs n2 = n1;
      n2.x = tmp_c; n2.residual = res_in_gemm ? nullptr : x1_c; n2.gamma = L.ln2_g; n2.beta = L.ln2_b; n2.out = out_c;
      LAUNCH(KC_NORM, launch_add_norm(n2, stream_), "output LayerNorm");
      LAUNCH(KC_POOL, launch_first_rows(out_c, x_, d_cu_, B, H * 2, 1, 0, stream_), "first rows back in place");
      break;
    }
    AttnArgs a;
    a.q = qkv; a.k = qkv + static_cast<size_t>(H) * 2; a.v = qkv + static_cast<size_t>(2 * H) * 2;
    a.out = attn_; a.cu_seqlens = d_cu_; a.work_items = d_work_; a.n_work = static_cast<int>(n_work_);
    a.total_tokens = T; a.n_heads = s.heads; a.n_kv_heads = s.kv_heads; a.head_dim = s.head_dim;
    a.ld_q = a.ld_k = a.ld_v = 3 * H; a.ld_o = H; a.causal = 0;
    a.scale = static_cast<float>(1.0 / std::sqrt(static_cast<double>(s.head_dim)));
    a.alibi_slopes = alibi_slopes_; a.dtype = s.dtype; a.status = status;
    if (s.jina_code) {
      LAUNCH(KC_NORM, launch_layernorm_qk(qkv, qkv + static_cast<size_t>(H) * 2, 3 * H, L.lnq_g, L.lnq_b, L.lnk_g,
                                          L.lnk_b, T, H, s.eps, s.dtype, stream_), "q / k LayerNorm");
    }
    LAUNCH(KC_ATTENTION, launch_attention(a, stream_), "attention");
    LAUNCH(KC_GEMM, launch_gemm(gemm_args(attn_, L.wo, L.bo, tmp_, T, H, H, H, H, ACT_NONE, s.dtype, status), stream_), "attention output projection");
    NormArgs n1;
    n1.x = tmp_; n1.residual = x_; n1.gamma = L.ln1_g; n1.beta = L.ln1_b; n1.out = x1_; n1.sum_out = nullptr;
    n1.T = T; n1.H = H; n1.eps = s.eps; n1.rms = 0; n1.dtype = s.dtype;
    LAUNCH(KC_NORM, launch_add_norm(n1, stream_), "attention LayerNorm");
    if (s.jina_code) {
      // flash_jina_code.rs:226-247: h = layer_norm_1(attention block output + layer input), the
      // gated feed-forward on h, then layer_norm_2(down + h).  h goes to tmp_ (free again), the
      // down projection to x1_ (consumed by then).
      NormArgs nm = n1;
      nm.x = x1_; nm.residual = x_; nm.gamma = L.lnm_g; nm.beta = L.lnm_b; nm.out = tmp_;
      LAUNCH(KC_NORM, launch_add_norm(nm, stream_), "pre-MLP LayerNorm");
      LAUNCH(KC_GEMM, launch_gemm(gemm_args(tmp_, L.w1, nullptr, ffn_, T, 2 * I, H, H, I, s.act, s.dtype, status), stream_), "gated projection");
      LAUNCH(KC_GEMM, launch_gemm(gemm_args(ffn_, L.w2, L.b2, x1_, T, H, I, I, H, ACT_NONE, s.dtype, status), stream_), "down projection");
      NormArgs n2 = n1;
      n2.x = x1_; n2.residual = tmp_; n2.gamma = L.ln2_g; n2.beta = L.ln2_b; n2.out = x_;
      LAUNCH(KC_NORM, launch_add_norm(n2, stream_), "post-MLP LayerNorm");
      continue;
    }
    if (s.gated) {  // JinaBERT: act(gate) * up in the epilogue of one [T, 2I] projection
      LAUNCH(KC_GEMM, launch_gemm(gemm_args(x1_, L.w1, nullptr, ffn_, T, 2 * I, H, H, I, s.act, s.dtype, status), stream_), "gated projection");
    } else {
      LAUNCH(KC_GEMM, launch_gemm(gemm_args(x1_, L.w1, L.b1, ffn_, T, I, H, H, I, s.act, s.dtype, status), stream_), "intermediate projection");
    }
    GemmArgs g2 = gemm_args(ffn_, L.w2, L.b2, tmp_, T, H, I, I, H, ACT_NONE, s.dtype, status);
    const bool res_in_gemm = fused_residual_ && residual_fits_epilogue(H, I);
    if (res_in_gemm) g2.residual = x1_, g2.ldr = H;
    LAUNCH(KC_GEMM, launch_gemm(g2, stream_), "output projection");
    NormArgs n2 = n1;
    n2.x = tmp_; n2.residual = res_in_gemm ? nullptr : x1_; n2.gamma = L.ln2_g; n2.beta = L.ln2_b; n2.out = x_;
    LAUNCH(KC_NORM, launch_add_norm(n2, stream_), "output LayerNorm");
  }
}

void Replica::forward_nomic() {
  const ModelSpec& s = spec_;
  const int T = static_cast<int>(T_), H = s.hidden, I = s.inter;
  int* status = reinterpret_cast<int*>(d_out_);
  EmbedArgs e;
  e.ids = d_ids_; e.type_ids = d_types_; e.pos_ids = nullptr;
  e.word = word_; e.type_tab = type_tab_; e.pos_tab = nullptr;
  e.gamma = emb_g_; e.beta = emb_b_; e.out = x_; e.T = T; e.H = H; e.eps = s.eps; e.dtype = s.dtype;
  LAUNCH(KC_EMBED, launch_embed_layernorm(e, stream_), "embeddings");
  // flash_nomic.rs:288-306: the NTK-scaled table is used only when the batch is longer than the
  // trained context.
  const bool scaled = cos_scaled_ && max_length_ > static_cast<uint32_t>(s.nomic_max_pos);
  uint8_t* qkv = static_cast<uint8_t*>(qkv_);
  for (int i = 0; i < s.layers; ++i) {
    const LayerW& L = layers_[i];
    RopeArgs r;
    r.q = qkv; r.k = qkv + static_cast<size_t>(H) * 2; r.pos_ids = d_pos_;
    r.cos_tab = scaled ? cos_scaled_ : cos_; r.sin_tab = scaled ? sin_scaled_ : sin_;
    r.q_gamma = nullptr; r.k_gamma = nullptr; r.T = T; r.n_heads = s.heads; r.n_kv_heads = s.kv_heads;
    r.head_dim = s.head_dim; r.ld_q = 3 * H; r.ld_k = 3 * H; r.eps = 0.f; r.dtype = s.dtype;
    qkv_projection(x_, L, T, 3 * H, H, r, status);  // flash_nomic.rs:60-81
    AttnArgs a;
    a.q = qkv; a.k = qkv + static_cast<size_t>(H) * 2; a.v = qkv + static_cast<size_t>(2 * H) * 2;
    a.out = attn_; a.cu_seqlens = d_cu_; a.work_items = d_work_; a.n_work = static_cast<int>(n_work_);
    a.total_tokens = T; a.n_heads = s.heads; a.n_kv_heads = s.kv_heads; a.head_dim = s.head_dim;
    a.ld_q = a.ld_k = a.ld_v = 3 * H; a.ld_o = H; a.causal = 0;
    a.scale = static_cast<float>(1.0 / std::sqrt(static_cast<double>(s.head_dim)));
    a.alibi_slopes = nullptr; a.dtype = s.dtype; a.status = status;
    if (first_rows_only_ && i + 1 == s.layers) {
      // Only the first row of every sequence is read after this layer (see forward_bert): scores
      // for the first query tiles, everything behind them on the B first rows, packed into x1_.
      const int B = static_cast<int>(B_);
      const size_t blk = static_cast<size_t>(B) * H * 2;
      uint8_t* c0 = static_cast<uint8_t*>(x1_);
      void *attn_c = c0, *res_c = c0 + blk, *tmp_c = c0 + 2 * blk, *x1_c = c0 + 3 * blk, *out_c = c0 + 4 * blk;
      a.work_items = d_work_first_;
      a.n_work = static_cast<int>(n_work_first_);
      LAUNCH(KC_ATTENTION, launch_attention(a, stream_), "attention, first query tiles");
      LAUNCH(KC_POOL, launch_first_rows(attn_, attn_c, d_cu_, B, H * 2, 0, 0, stream_), "first rows of the attention output");
      LAUNCH(KC_POOL, launch_first_rows(x_, res_c, d_cu_, B, H * 2, 0, 0, stream_), "first rows of the layer input");
      LAUNCH(KC_GEMM, launch_gemm(gemm_args(attn_c, L.wo, L.bo, tmp_c, B, H, H, H, H, ACT_NONE, s.dtype, status), stream_), "attention output projection");
      NormArgs m1;
      m1.x = tmp_c; m1.residual = res_c; m1.gamma = L.ln1_g; m1.beta = L.ln1_b; m1.out = x1_c; m1.sum_out = nullptr;
      m1.T = B; m1.H = H; m1.eps = s.eps; m1.rms = 0; m1.dtype = s.dtype;
      LAUNCH(KC_NORM, launch_add_norm(m1, stream_), "norm1");
      if (s.gated) {
        LAUNCH(KC_GEMM, launch_gemm(gemm_args(x1_c, L.w1, L.b1, ffn_, B, 2 * I, H, H, I, s.act, s.dtype, status), stream_), "gated fc1");
      } else {
        LAUNCH(KC_GEMM, launch_gemm(gemm_args(x1_c, L.w1, L.b1, ffn_, B, I, H, H, I, s.act, s.dtype, status), stream_), "fc1");
      }
      GemmArgs g2 = gemm_args(ffn_, L.w2, L.b2, tmp_c, B, H, I, I, H, ACT_NONE, s.dtype, status);
      const bool res_in_gemm = fused_residual_ && residual_fits_epilogue(H, I);
      if (res_in_gemm) g2.residual = x1_c, g2.ldr = H;
      LAUNCH(KC_GEMM, launch_gemm(g2, stream_), "fc2");
      NormArgs m2 = m1;
      m2.x = tmp_c; m2.residual = res_in_gemm ? nullptr : x1_c; m2.gamma = L.ln2_g; m2.beta = L.ln2_b; m2.out = out_c;
      LAUNCH(KC_NORM, launch_add_norm(m2, stream_), "norm2");
      LAUNCH(KC_POOL, launch_first_rows(out_c, x_, d_cu_, B, H * 2, 1, 0, stream_), "first rows back in place");
      break;
    }
    LAUNCH(KC_ATTENTION, launch_attention(a, stream_), "attention");
    LAUNCH(KC_GEMM, launch_gemm(gemm_args(attn_, L.wo, L.bo, tmp_, T, H, H, H, H, ACT_NONE, s.dtype, status), stream_), "attention output projection");
    NormArgs n1;
    n1.x = tmp_; n1.residual = x_; n1.gamma = L.ln1_g; n1.beta = L.ln1_b; n1.out = x1_; n1.sum_out = nullptr;
    n1.T = T; n1.H = H; n1.eps = s.eps; n1.rms = 0; n1.dtype = s.dtype;
    LAUNCH(KC_NORM, launch_add_norm(n1, stream_), "norm1");
    bool res_in_gemm = false;  // the experts' outputs are combined first: their residual stays with the LayerNorm
    if (L.moe_router) {
      // NomicMoELayer::forward (nomic.rs:384-393): router logits -> fp32 softmax -> top-k; every
      // expert runs act(x w1_e^T) w2_e on the tokens routed to it; the outputs are summed with
      // the routing weights and the shared bias.  No host round trip: the expert GEMMs take
      // their row count from the device.
      const int E = s.num_experts, K = s.moe_top_k, Epad = static_cast<int>(align_up(static_cast<size_t>(E), 8));
      const long long cap = static_cast<long long>(moe_cap_);
      LAUNCH(KC_GEMM, launch_gemm(gemm_args(x1_, L.moe_router, nullptr, moe_logits_, T, Epad, H, H, Epad, ACT_NONE, s.dtype, status), stream_), "router");
      TEI_CUDA(cudaMemsetAsync(moe_counts_, 0, static_cast<size_t>(E) * 4, stream_));
      LAUNCH(KC_POOL, launch_moe_route(moe_logits_, Epad, T, E, K, moe_topk_e_, moe_topk_w_, moe_pos_, moe_counts_, s.dtype, stream_), "expert routing");
      LAUNCH(KC_POOL, launch_moe_gather(x1_, moe_topk_e_, moe_pos_, moe_xg_, T, K, H, cap, s.dtype, stream_), "expert gather");
      for (int e = 0; e < E; ++e) {
        uint8_t* xg = static_cast<uint8_t*>(moe_xg_) + static_cast<size_t>(e) * cap * H * 2;
        uint8_t* hg = static_cast<uint8_t*>(moe_hg_) + static_cast<size_t>(e) * cap * I * 2;
        uint8_t* yg = static_cast<uint8_t*>(moe_yg_) + static_cast<size_t>(e) * cap * H * 2;
        const uint8_t* w1 = static_cast<const uint8_t*>(L.moe_w1) + static_cast<size_t>(e) * I * H * 2;
        const uint8_t* w2 = static_cast<const uint8_t*>(L.moe_w2t) + static_cast<size_t>(e) * H * I * 2;
        GemmArgs g1 = gemm_args(xg, w1, nullptr, hg, static_cast<int>(cap), I, H, H, I, s.act, s.dtype, status);
        g1.m_dev = moe_counts_ + e;
        LAUNCH(KC_GEMM, launch_gemm(g1, stream_), "expert fc1");
        GemmArgs g2 = gemm_args(hg, w2, nullptr, yg, static_cast<int>(cap), H, I, I, H, ACT_NONE, s.dtype, status);
        g2.m_dev = moe_counts_ + e;
        LAUNCH(KC_GEMM, launch_gemm(g2, stream_), "expert fc2");
      }
      LAUNCH(KC_POOL, launch_moe_combine(moe_yg_, moe_topk_e_, moe_topk_w_, moe_pos_, L.moe_bias, tmp_, T, K, H, cap, s.dtype, stream_), "expert combine");
    } else {
      if (s.gated) {
        LAUNCH(KC_GEMM, launch_gemm(gemm_args(x1_, L.w1, L.b1, ffn_, T, 2 * I, H, H, I, s.act, s.dtype, status), stream_), "gated fc1");
      } else {
        LAUNCH(KC_GEMM, launch_gemm(gemm_args(x1_, L.w1, L.b1, ffn_, T, I, H, H, I, s.act, s.dtype, status), stream_), "fc1");
      }
      GemmArgs g2 = gemm_args(ffn_, L.w2, L.b2, tmp_, T, H, I, I, H, ACT_NONE, s.dtype, status);
      res_in_gemm = fused_residual_ && residual_fits_epilogue(H, I);
      if (res_in_gemm) g2.residual = x1_, g2.ldr = H;
      LAUNCH(KC_GEMM, launch_gemm(g2, stream_), "fc2");
    }
    NormArgs n2 = n1;
    n2.x = tmp_; n2.residual = res_in_gemm ? nullptr : x1_; n2.gamma = L.ln2_g; n2.beta = L.ln2_b; n2.out = x_;
    LAUNCH(KC_NORM, launch_add_norm(n2, stream_), "norm2");
  }
}

void Replica::forward_qwen3() {
  // The pre-norm skeleton: x = x + attn(norm(x)); x = x + mlp(norm(x)), with the running sum in
  // fp32.  RMSNorm decoders (flash_qwen3.rs, flash_qwen2.rs, flash_mistral.rs) and ModernBERT
  // (flash_modernbert.rs: LayerNorm without bias, LayerNorm after the embedding, no norm in front
  // of the first attention, GeGLU, local / global layers) differ by the flags of the spec.
  const ModelSpec& s = spec_;
  const int T = static_cast<int>(T_), H = s.hidden, I = s.inter, Q = s.q_width(), KV = s.kv_width();
  const int W = Q + 2 * KV;
  const int rms = s.modernbert ? 0 : 1;
  int* status = reinterpret_cast<int*>(d_out_);
  EmbedArgs e;
  e.ids = d_ids_; e.type_ids = nullptr; e.pos_ids = nullptr;
  e.word = word_; e.type_tab = nullptr; e.pos_tab = nullptr;
  e.gamma = emb_g_; e.beta = nullptr; e.out = tmp_; e.T = T; e.H = H; e.eps = s.eps; e.dtype = s.dtype;
  LAUNCH(KC_EMBED, launch_embed_layernorm(e, stream_), "embeddings");
  uint8_t* qkv = static_cast<uint8_t*>(qkv_);
  // h (the branch output waiting to be added) lives in tmp_; the fp32 running sum in resid_.
  for (int i = 0; i < s.layers; ++i) {
    const LayerW& L = layers_[i];
    const bool local = s.modernbert && (i % s.global_every != 0);
    NormArgs n1;
    n1.x = tmp_; n1.residual = (i == 0) ? nullptr : resid_; n1.gamma = L.ln1_g; n1.beta = nullptr;
    n1.out = x_; n1.sum_out = resid_; n1.T = T; n1.H = H; n1.eps = s.eps; n1.rms = rms; n1.dtype = s.dtype;
    n1.residual_f32 = 1;
    LAUNCH(KC_NORM, launch_add_norm(n1, stream_), "input norm");
    RopeArgs r;
    r.q = qkv; r.k = qkv + static_cast<size_t>(Q) * 2; r.pos_ids = d_pos_;
    r.cos_tab = local ? cos_scaled_ : cos_; r.sin_tab = local ? sin_scaled_ : sin_;
    r.q_gamma = L.q_norm; r.k_gamma = L.k_norm; r.T = T; r.n_heads = s.heads; r.n_kv_heads = s.kv_heads;
    r.head_dim = s.head_dim; r.ld_q = W; r.ld_k = W; r.eps = s.eps; r.dtype = s.dtype;
    qkv_projection(x_, L, T, W, H, r, status);  // flash_qwen3.rs:119-153
    AttnArgs a;
    a.q = qkv; a.k = qkv + static_cast<size_t>(Q) * 2; a.v = qkv + static_cast<size_t>(Q + KV) * 2;
    a.out = attn_; a.cu_seqlens = d_cu_; a.work_items = local ? d_work_local_ : d_work_;
    a.n_work = static_cast<int>(n_work_);
    a.total_tokens = T; a.n_heads = s.heads; a.n_kv_heads = s.kv_heads; a.head_dim = s.head_dim;
    a.ld_q = a.ld_k = a.ld_v = W; a.ld_o = Q; a.causal = s.causal ? 1 : 0;
    a.window_left = local ? s.local_window : s.window_left;
    a.window_right = local ? s.local_window : -1;
    a.scale = static_cast<float>(1.0 / std::sqrt(static_cast<double>(s.head_dim)));
    a.alibi_slopes = nullptr; a.dtype = s.dtype; a.status = status;
    if (first_rows_only_ && i + 1 == s.layers) {
      // Only one row per sequence is pooled (the first or the last token) and nothing else is
      // read after this layer: scores for the query tile that holds the row, then the output
      // projection, the post-attention norm, the feed-forward and the final norm on the B rows,
      // packed into x1_ / ffn_, and back to the rows' places in x_.
      const int B = static_cast<int>(B_);
      const int last = s.pool == POOL_LAST ? 1 : 0;
      uint8_t* c0 = static_cast<uint8_t*>(x1_);
      const size_t blk = static_cast<size_t>(B) * H * 2;
      void* attn_c = c0;
      uint8_t* c1 = c0 + static_cast<size_t>(B) * Q * 2;
      void *tmp_c = c1, *x1_c = c1 + blk, *out_c = c1 + 2 * blk;
      float* resid_c = reinterpret_cast<float*>(static_cast<uint8_t*>(ffn_) +
                                                align_up(static_cast<size_t>(B) * 2 * I * 2, 64));
      a.work_items = d_work_first_;
      a.n_work = static_cast<int>(n_work_first_);
      LAUNCH(KC_ATTENTION, launch_attention(a, stream_), "attention, one query tile per sequence");
      LAUNCH(KC_POOL, launch_first_rows(attn_, attn_c, d_cu_, B, Q * 2, 0, last, stream_), "rows of the attention output");
      LAUNCH(KC_POOL, launch_first_rows(resid_, resid_c, d_cu_, B, H * 4, 0, last, stream_), "rows of the running sum");
      LAUNCH(KC_GEMM, launch_gemm(gemm_args(attn_c, L.wo, L.bo, tmp_c, B, H, Q, Q, H, ACT_NONE, s.dtype, status), stream_), "o projection");
      NormArgs m2 = n1;
      m2.x = tmp_c; m2.residual = resid_c; m2.gamma = L.ln2_g; m2.out = x1_c; m2.sum_out = resid_c; m2.T = B;
      LAUNCH(KC_NORM, launch_add_norm(m2, stream_), "post-attention norm");
      LAUNCH(KC_GEMM, launch_gemm(gemm_args(x1_c, L.w1, L.b1, ffn_, B, 2 * I, H, H, I, s.act, s.dtype, status), stream_), "gate/up projection");
      LAUNCH(KC_GEMM, launch_gemm(gemm_args(ffn_, L.w2, L.b2, tmp_c, B, H, I, I, H, ACT_NONE, s.dtype, status), stream_), "down projection");
      NormArgs mf = m2;
      mf.x = tmp_c; mf.gamma = final_norm_; mf.out = out_c;
      LAUNCH(KC_NORM, launch_add_norm(mf, stream_), "final norm");
      LAUNCH(KC_POOL, launch_first_rows(out_c, x_, d_cu_, B, H * 2, 1, last, stream_), "rows back in place");
      return;
    }
    LAUNCH(KC_ATTENTION, launch_attention(a, stream_), "attention");
    LAUNCH(KC_GEMM, launch_gemm(gemm_args(attn_, L.wo, L.bo, tmp_, T, H, Q, Q, H, ACT_NONE, s.dtype, status), stream_), "o projection");
    NormArgs n2 = n1;
    n2.x = tmp_; n2.residual = resid_; n2.gamma = L.ln2_g; n2.out = x1_; n2.sum_out = resid_;
    LAUNCH(KC_NORM, launch_add_norm(n2, stream_), "post-attention norm");
    LAUNCH(KC_GEMM, launch_gemm(gemm_args(x1_, L.w1, L.b1, ffn_, T, 2 * I, H, H, I, s.act, s.dtype, status), stream_), "gate/up projection");
    LAUNCH(KC_GEMM, launch_gemm(gemm_args(ffn_, L.w2, L.b2, tmp_, T, H, I, I, H, ACT_NONE, s.dtype, status), stream_), "down projection");
  }
  NormArgs nf;
  nf.x = tmp_; nf.residual = resid_; nf.gamma = final_norm_; nf.beta = nullptr; nf.out = x_; nf.sum_out = resid_;
  nf.T = T; nf.H = H; nf.eps = s.eps; nf.rms = rms; nf.dtype = s.dtype; nf.residual_f32 = 1;
  LAUNCH(KC_NORM, launch_add_norm(nf, stream_), "final norm");
  if (projection_) {
    // Optional `linear.weight` projection applied to every token row (flash_qwen3.rs:430-435).
    if (projection_dim_ > H) throw TeiError(ERR_INFERENCE, "projection wider than the hidden size is not supported");
    LAUNCH(KC_GEMM, launch_gemm(gemm_args(x_, projection_, nullptr, x1_, T, projection_dim_, H, H, projection_dim_, ACT_NONE, s.dtype, status), stream_), "projection");
    std::swap(x_, x1_);
  }
}

void Replica::pool_and_heads() {
  const ModelSpec& s = spec_;
  const int T = static_cast<int>(T_), H = s.hidden;
  int* status = reinterpret_cast<int*>(d_out_);
  const int D = raw_dim();
  if (predict_) {
    PoolArgs p;
    p.x = x_; p.cu_seqlens = d_cu_; p.seq_index = d_all_idx_; p.out = d_cls_;
    p.n_out = static_cast<int>(B_); p.H = H; p.mode = s.modernbert ? s.cls_pool : POOL_CLS; p.normalize = 0;
    p.dtype = s.dtype;
    LAUNCH(KC_POOL, launch_pool(p, stream_), "pooling for the head");
    const float* head_in = d_cls_;
    if (s.modernbert) {  // dense (no bias) + activation -> LayerNorm -> classifier, modernbert.rs:443-456
      LAUNCH(KC_POOL, launch_head_linear(d_cls_, cls_dense_w_, nullptr, d_head_tmp_, static_cast<int>(B_), H, H, s.head_act, s.dtype, stream_), "head dense");
      LAUNCH(KC_POOL, launch_layernorm_rows_f32(d_head_tmp_, cls_norm_g_, static_cast<int>(B_), H, s.eps, s.dtype, stream_), "head norm");
      head_in = d_head_tmp_;
    } else if (cls_dense_w_) {  // dense + tanh (RobertaClassificationHead / BERT pooler, bert.rs:405-465)
      LAUNCH(KC_POOL, launch_head_linear(d_cls_, cls_dense_w_, cls_dense_b_, d_head_tmp_, static_cast<int>(B_), H, H, ACT_TANH, s.dtype, stream_), "classifier dense");
      head_in = d_head_tmp_;
    }
    LAUNCH(KC_POOL, launch_head_linear(head_in, cls_out_w_, cls_out_b_, d_scores_, static_cast<int>(B_), s.n_classes, H, ACT_NONE, s.dtype, stream_), "classifier output");
    return;
  }
  if (n_pooled_ > 0) {
    PoolArgs p;
    p.cu_seqlens = d_cu_; p.seq_index = d_pooled_idx_; p.out = d_pooled_;
    p.n_out = static_cast<int>(n_pooled_); p.dtype = s.dtype;
    if (s.pool == POOL_SPLADE) {
      // BertSpladeHead (bert.rs:551-558): dense + act -> LayerNorm -> decoder + ReLU -> log(1 + x),
      // then the per-sequence maximum (flash_bert.rs:464-490).
      const int V = s.vocab, Vpad = static_cast<int>(align_up(V, 8));
      LAUNCH(KC_GEMM, launch_gemm(gemm_args(x_, sp_dense_w_, sp_dense_b_, tmp_, T, H, H, H, H, sp_act_, s.dtype, status), stream_), "splade transform");
      NormArgs n;
      n.x = tmp_; n.residual = nullptr; n.gamma = sp_ln_g_; n.beta = sp_ln_b_; n.out = x1_; n.sum_out = nullptr;
      n.T = T; n.H = H; n.eps = s.eps; n.rms = 0; n.dtype = s.dtype;
      LAUNCH(KC_NORM, launch_add_norm(n, stream_), "splade LayerNorm");
      LAUNCH(KC_GEMM, launch_gemm(gemm_args(x1_, sp_dec_w_, sp_dec_b_, splade_, T, V, H, H, Vpad, ACT_RELU_LOG1P, s.dtype, status), stream_), "splade decoder");
      p.x = splade_; p.H = Vpad; p.mode = POOL_SPLADE; p.normalize = 0;
    } else {
      p.x = x_; p.H = D; p.mode = s.pool; p.normalize = (normalize_ && dense_.empty()) ? 1 : 0;
      if (!dense_.empty()) p.out = d_dense_a_;
    }
    LAUNCH(KC_POOL, launch_pool(p, stream_), "pooling");
    if (!dense_.empty() && s.pool != POOL_SPLADE) {
      // Dense modules on the pooled rows, in order (backends/candle/src/lib.rs:672-680); the
      // last one writes into the output block.
      const float* in = d_dense_a_;
      for (size_t i = 0; i < dense_.size(); ++i) {
        const DenseW& d = dense_[i];
        float* out = i + 1 == dense_.size() ? d_pooled_ : (in == d_dense_a_ ? d_dense_b_ : d_dense_a_);
        LAUNCH(KC_POOL, launch_head_linear(in, d.w, d.b, out, static_cast<int>(n_pooled_), d.out, d.in, d.act, s.dtype, stream_), "dense module");
        in = out;
      }
      if (normalize_) {
        LAUNCH(KC_POOL, launch_l2_normalise(d_pooled_, static_cast<int>(n_pooled_), dense_.back().out, stream_), "normalise");
      }
    }
  }
  if (n_raw_rows_ > 0) {
    LAUNCH(KC_POOL, launch_gather_rows_f32(x_, d_raw_rows_, d_raw_, static_cast<int>(n_raw_rows_), D, s.dtype, stream_), "raw rows");
  }
}

// ------------------------------------------------------------------------------ fetch
void Replica::sync_and_check() {
  TEI_CUDA(cudaSetDevice(device_));
  int status = 0;
  TEI_CUDA(cudaMemcpyAsync(h_out_, d_out_, 4, cudaMemcpyDeviceToHost, stream_));
  TEI_CUDA(cudaStreamSynchronize(stream_));
  prof_drain();
  std::memcpy(&status, h_out_, 4);
  if (status != 0) {
    throw TeiError(ERR_TIMEOUT, "a kernel's bounded wait ran out (device status " + std::to_string(status) + ")");
  }
  float ms = 0.f;
  if (cudaEventElapsedTime(&ms, ev_start_, ev_stop_) == cudaSuccess) {
    stats_.last_gpu_ms = ms;
  }
}

void Replica::fetch(float* pooled_out, float* raw_out, float* scores_out) {
  TEI_CUDA(cudaSetDevice(device_));
  TEI_CUDA(cudaMemcpyAsync(h_out_, d_out_, out_floats_ * 4, cudaMemcpyDeviceToHost, stream_));
  TEI_CUDA(cudaStreamSynchronize(stream_));
  prof_drain();
  stats_.last_d2h_bytes = static_cast<double>(out_floats_ * 4);
  int status = 0;
  std::memcpy(&status, h_out_, 4);
  if (status != 0) {
    throw TeiError(ERR_TIMEOUT, "a kernel's bounded wait ran out (device status " + std::to_string(status) + ")");
  }
  float ms = 0.f;
  if (cudaEventElapsedTime(&ms, ev_start_, ev_stop_) == cudaSuccess) {
    stats_.last_gpu_ms = ms;
    stats_.total_gpu_ms += ms;
  }
  stats_.total_tokens += static_cast<double>(T_);
  stats_.calls += 1.0;
  const size_t D = static_cast<size_t>(output_dim());
  const size_t Dpad = pooled_ld_;
  const float* hp = h_out_ + (d_pooled_ - d_out_);
  if (n_pooled_ && pooled_out) {
    if (D == Dpad) {
      std::memcpy(pooled_out, hp, n_pooled_ * D * 4);
    } else {
      for (size_t i = 0; i < n_pooled_; ++i) std::memcpy(pooled_out + i * D, hp + i * Dpad, D * 4);
    }
  }
  if (n_raw_rows_ && raw_out) {
    std::memcpy(raw_out, h_out_ + (d_raw_ - d_out_), n_raw_rows_ * static_cast<size_t>(raw_dim()) * 4);
  }
  if (predict_ && scores_out) {
    std::memcpy(scores_out, h_out_ + (d_scores_ - d_out_), B_ * static_cast<size_t>(spec_.n_classes) * 4);
  }
}

}  // namespace tei
