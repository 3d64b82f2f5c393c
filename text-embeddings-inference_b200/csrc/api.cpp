// extern "C" backend entry points (include/tei_b200.h): handle lifetime, error mapping, and the
// split of one packed batch over several GPU replicas.
#include "../../include/tei_b200.h"

#include "model.h"
#include "plan.h"

#include <algorithm>
#include <atomic>
#include <cstring>
#include <fstream>
#include <memory>
#include <mutex>
#include <sstream>
#include <thread>

using namespace tei;

namespace {

// A sub-batch for one replica plus where its rows go in the caller's buffers.
struct Shard {
  std::vector<uint32_t> ids, types, pos, cu, pooled_idx, raw_idx;
  uint32_t max_length = 0;
  std::vector<size_t> seqs;             // original batch positions, in shard order
  std::vector<size_t> pooled_dst_row;   // caller's pooled row of each pooled entry of the shard
  std::vector<size_t> raw_dst_row;      // caller's first raw row of each raw entry
  std::vector<size_t> raw_len;
  std::vector<float> pooled, raw, scores;
  int err_kind = 0;
  std::string err_msg;
};

void set_err(char* err, size_t cap, const std::string& msg) {
  if (!err || cap == 0) return;
  const size_t n = std::min(cap - 1, msg.size());
  std::memcpy(err, msg.data(), n);
  err[n] = '\0';
}

std::string read_file(const std::string& path) {
  std::ifstream in(path, std::ios::binary);
  if (!in) throw TeiError(ERR_START, "cannot read " + path);
  std::stringstream ss;
  ss << in.rdbuf();
  return ss.str();
}

}  // namespace

struct tei_b200 {
  ModelSpec spec;
  std::string model_dir;
  std::vector<std::unique_ptr<Replica>> replicas;
  // One lock per replica: the per-replica entry points (one caller thread per replica) take it,
  // so two threads that were given the same index by mistake queue up instead of corrupting the
  // replica's staging buffers.
  std::vector<std::unique_ptr<std::mutex>> replica_locks;
  std::atomic<bool> healthy{true};
  // state of the staged batch (stage / run / sync / fetch)
  bool staged = false;
  bool staged_predict = false;
  std::vector<Shard> shards;   // empty when a single replica took the whole batch
  size_t staged_n_pooled = 0, staged_raw_rows = 0, staged_n_seqs = 0;
  double linear_cost = 1.0, quadratic_cost = 0.0;
};

namespace {

template <class F>
int guarded(tei_b200* h, char* err, size_t cap, F&& fn) {
  try {
    fn();
    if (h) h->healthy = true;
    return TEI_B200_OK;
  } catch (const TeiError& e) {
    set_err(err, cap, e.what());
    if (h && e.kind != ERR_START && e.kind != ERR_WEIGHTS_NOT_FOUND) h->healthy = false;
    return e.kind;
  } catch (const std::exception& e) {
    set_err(err, cap, e.what());
    if (h) h->healthy = false;
    return TEI_B200_ERR_INFERENCE;
  } catch (...) {
    set_err(err, cap, "unknown error");
    if (h) h->healthy = false;
    return TEI_B200_ERR_INFERENCE;
  }
}

HostBatch make_batch(const uint32_t* ids, const uint32_t* types, const uint32_t* pos, size_t n_tokens,
                     const uint32_t* cu, size_t n_seqs, uint32_t max_length, const uint32_t* pooled,
                     size_t n_pooled, const uint32_t* raw, size_t n_raw) {
  HostBatch b;
  b.input_ids = ids;
  b.token_type_ids = types;
  b.position_ids = pos;
  b.n_tokens = n_tokens;
  b.cu_seqlens = cu;
  b.n_seqs = n_seqs;
  b.max_length = max_length;
  b.pooled_indices = pooled;
  b.n_pooled = n_pooled;
  b.raw_indices = raw;
  b.n_raw = n_raw;
  return b;
}

// Cheap structural checks needed before the batch can be split (the replicas validate the rest).
void precheck(const HostBatch& b) {
  if (b.n_seqs == 0 || b.n_tokens == 0) throw TeiError(ERR_INFERENCE, "empty batch");
  if (!b.input_ids || !b.cu_seqlens || !b.position_ids) throw TeiError(ERR_INFERENCE, "null batch pointer");
  if (b.cu_seqlens[0] != 0 || b.cu_seqlens[b.n_seqs] != b.n_tokens) {
    throw TeiError(ERR_INFERENCE, "cumulative_seq_lengths must start at 0 and end at the token count");
  }
  for (size_t i = 0; i < b.n_seqs; ++i) {
    if (b.cu_seqlens[i + 1] <= b.cu_seqlens[i]) {
      throw TeiError(ERR_INFERENCE, "cumulative_seq_lengths must be strictly increasing");
    }
  }
  for (size_t i = 0; i < b.n_pooled; ++i) {
    if (b.pooled_indices[i] >= b.n_seqs) throw TeiError(ERR_INFERENCE, "pooled index out of range");
  }
  for (size_t i = 0; i < b.n_raw; ++i) {
    if (b.raw_indices[i] >= b.n_seqs) throw TeiError(ERR_INFERENCE, "raw index out of range");
  }
}

void build_shards(tei_b200* h, const HostBatch& b, bool predict) {
  const int n = static_cast<int>(h->replicas.size());
  std::vector<int> shard_of(b.n_seqs, 0);
  plan_shards(b.cu_seqlens, static_cast<int>(b.n_seqs), n, h->linear_cost, h->quadratic_cost,
              shard_of.data());
  h->shards.assign(n, Shard());
  std::vector<size_t> local_index(b.n_seqs, 0);
  for (size_t s = 0; s < b.n_seqs; ++s) {
    Shard& sh = h->shards[shard_of[s]];
    if (sh.cu.empty()) sh.cu.push_back(0);
    const uint32_t a = b.cu_seqlens[s], e = b.cu_seqlens[s + 1];
    sh.ids.insert(sh.ids.end(), b.input_ids + a, b.input_ids + e);
    if (b.token_type_ids) sh.types.insert(sh.types.end(), b.token_type_ids + a, b.token_type_ids + e);
    else sh.types.insert(sh.types.end(), e - a, 0u);
    sh.pos.insert(sh.pos.end(), b.position_ids + a, b.position_ids + e);
    sh.cu.push_back(sh.cu.back() + (e - a));
    sh.max_length = std::max(sh.max_length, e - a);
    local_index[s] = sh.seqs.size();
    sh.seqs.push_back(s);
  }
  if (!predict) {
    for (size_t i = 0; i < b.n_pooled; ++i) {
      const uint32_t s = b.pooled_indices[i];
      Shard& sh = h->shards[shard_of[s]];
      sh.pooled_idx.push_back(static_cast<uint32_t>(local_index[s]));
      sh.pooled_dst_row.push_back(i);
    }
    size_t row = 0;
    for (size_t i = 0; i < b.n_raw; ++i) {
      const uint32_t s = b.raw_indices[i];
      Shard& sh = h->shards[shard_of[s]];
      const size_t len = b.cu_seqlens[s + 1] - b.cu_seqlens[s];
      sh.raw_idx.push_back(static_cast<uint32_t>(local_index[s]));
      sh.raw_dst_row.push_back(row);
      sh.raw_len.push_back(len);
      row += len;
    }
  }
}

template <class F>
void for_each_shard_parallel(tei_b200* h, F&& fn) {
  std::vector<std::thread> threads;
  for (size_t d = 0; d < h->shards.size(); ++d) {
    if (h->shards[d].seqs.empty()) continue;
    threads.emplace_back([h, d, &fn]() {
      Shard& sh = h->shards[d];
      try {
        fn(*h->replicas[d], sh);
      } catch (const TeiError& e) {
        sh.err_kind = e.kind;
        sh.err_msg = e.what();
      } catch (const std::exception& e) {
        sh.err_kind = ERR_INFERENCE;
        sh.err_msg = e.what();
      }
    });
  }
  for (auto& t : threads) t.join();
  for (auto& sh : h->shards) {
    if (sh.err_kind) {
      const int k = sh.err_kind;
      std::string m = sh.err_msg;
      sh.err_kind = 0;
      throw TeiError(k, m);
    }
  }
}

void do_stage(tei_b200* h, const HostBatch& b, bool predict, bool normalize) {
  precheck(b);
  h->staged = false;
  h->staged_predict = predict;
  h->staged_n_pooled = predict ? 0 : b.n_pooled;
  h->staged_n_seqs = b.n_seqs;
  size_t raw_rows = 0;
  if (!predict) {
    for (size_t i = 0; i < b.n_raw; ++i) raw_rows += b.cu_seqlens[b.raw_indices[i] + 1] - b.cu_seqlens[b.raw_indices[i]];
  }
  h->staged_raw_rows = raw_rows;
  if (h->replicas.size() == 1 || b.n_seqs == 1) {
    h->shards.clear();
    h->replicas[0]->stage(b, predict, normalize);
  } else {
    build_shards(h, b, predict);
    for_each_shard_parallel(h, [&](Replica& r, Shard& sh) {
      HostBatch sb = make_batch(sh.ids.data(), sh.types.data(), sh.pos.data(), sh.ids.size(), sh.cu.data(),
                                sh.seqs.size(), sh.max_length, sh.pooled_idx.data(), sh.pooled_idx.size(),
                                sh.raw_idx.data(), sh.raw_idx.size());
      r.stage(sb, predict, normalize);
    });
  }
  h->staged = true;
}

void do_run(tei_b200* h) {
  if (!h->staged) throw TeiError(ERR_INFERENCE, "no staged batch");
  if (h->shards.empty()) {
    h->replicas[0]->run();
  } else {
    for_each_shard_parallel(h, [](Replica& r, Shard&) { r.run(); });
  }
}

void do_sync(tei_b200* h) {
  if (!h->staged) throw TeiError(ERR_INFERENCE, "no staged batch");
  if (h->shards.empty()) {
    h->replicas[0]->sync_and_check();
  } else {
    for_each_shard_parallel(h, [](Replica& r, Shard&) { r.sync_and_check(); });
  }
}

void do_fetch(tei_b200* h, float* pooled_out, float* raw_out, float* scores_out) {
  if (!h->staged) throw TeiError(ERR_INFERENCE, "no staged batch");
  if (h->shards.empty()) {
    h->replicas[0]->fetch(pooled_out, raw_out, scores_out);
    return;
  }
  const size_t D = static_cast<size_t>(h->replicas[0]->output_dim());
  const size_t DR = static_cast<size_t>(h->replicas[0]->raw_dim());
  const size_t C = static_cast<size_t>(std::max(h->spec.n_classes, 1));
  const bool predict = h->staged_predict;
  for_each_shard_parallel(h, [&](Replica& r, Shard& sh) {
    size_t raw_rows = 0;
    for (size_t l : sh.raw_len) raw_rows += l;
    sh.pooled.resize(sh.pooled_idx.size() * D);
    sh.raw.resize(raw_rows * DR);
    sh.scores.resize(predict ? sh.seqs.size() * C : 0);
    r.fetch(sh.pooled.data(), sh.raw.data(), sh.scores.data());
  });
  // Host-side gather: every shard's rows go back to their original batch positions.
  for (auto& sh : h->shards) {
    if (sh.seqs.empty()) continue;
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
    if (predict && scores_out) {
      for (size_t i = 0; i < sh.seqs.size(); ++i) {
        std::memcpy(scores_out + sh.seqs[i] * C, sh.scores.data() + i * C, C * 4);
      }
    }
  }
}

}  // namespace

extern "C" {

int tei_b200_create(const char* model_dir, const char* dtype, int model_type, int pool,
                    const int* devices, int n_devices, tei_b200_t** out, char* err,
                    size_t err_cap) {
  if (!out) return TEI_B200_ERR_START;
  *out = nullptr;
  std::unique_ptr<tei_b200> h(new tei_b200());
  const int rc = guarded(nullptr, err, err_cap, [&]() {
    if (!model_dir || !dtype) throw TeiError(ERR_START, "model_dir and dtype are required");
    int dt;
    const std::string d = dtype;
    if (d == "float16") dt = 0;
    else if (d == "bfloat16") dt = 1;
    else throw TeiError(ERR_START, "DType " + d + " is not supported (float16 or bfloat16)");
    if (model_type != TEI_B200_CLASSIFIER && model_type != TEI_B200_EMBEDDING) {
      throw TeiError(ERR_START, "unknown model_type");
    }
    if (pool < 0 || pool > 3) throw TeiError(ERR_START, "unknown pool");
    const std::string dir = model_dir;
    h->model_dir = dir;
    Json config;
    try {
      config = Json::parse(read_file(dir + "/config.json"));
    } catch (const TeiError&) {
      throw;
    } catch (const std::exception& e) {
      throw TeiError(ERR_START, std::string("config.json: ") + e.what());
    }
    h->spec = parse_model_spec(config, model_type, pool, dt);
    SafeTensors st;
    try {
      st.open_dir(dir);
    } catch (const std::exception& e) {
      const std::string m = e.what();
      throw TeiError(m.rfind("weights not found", 0) == 0 ? ERR_WEIGHTS_NOT_FOUND : ERR_START, m);
    }
    std::vector<int> devs;
    if (devices && n_devices > 0) devs.assign(devices, devices + n_devices);
    else devs.push_back(0);
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
      throw TeiError(ERR_START, "no CUDA device is visible; this backend has no CPU fallback");
    }
    for (int dv : devs) {
      if (dv < 0 || dv >= count) throw TeiError(ERR_START, "CUDA device index out of range");
      h->replicas.emplace_back(new Replica(dv, h->spec, st));
      h->replica_locks.emplace_back(new std::mutex());
    }
    // Cost model of the sharding: FLOPs per token of the dense layers, FLOPs per token^2 of
    // attention (half of it when causal).
    const ModelSpec& s = h->spec;
    const double m = s.gated ? 3.0 : 2.0;
    h->linear_cost = 2.0 * (static_cast<double>(s.hidden) * s.q_width() + 2.0 * s.hidden * s.kv_width() +
                            static_cast<double>(s.q_width()) * s.hidden + m * s.hidden * s.inter);
    h->quadratic_cost = (s.causal ? 2.0 : 4.0) * s.q_width();
  });
  if (rc == TEI_B200_OK) *out = h.release();
  return rc;
}

int tei_b200_add_dense(tei_b200_t* h, const char* dense_path, char* err, size_t err_cap) {
  if (!h) return TEI_B200_ERR_START;
  int rc = guarded(nullptr, err, err_cap, [&]() {
    if (!dense_path) throw TeiError(ERR_START, "dense_path is required");
    const std::string dir = h->model_dir + "/" + dense_path;
    auto exists = [](const std::string& p) {
      std::ifstream f(p, std::ios::binary);
      return static_cast<bool>(f);
    };
    if (!exists(dir + "/model.safetensors")) {
      if (exists(dir + "/pytorch_model.bin")) {
        throw TeiError(ERR_START, "Dense module `" + std::string(dense_path) + "` has only pytorch_model.bin; safetensors is required");
      }
      // backends/candle/src/lib.rs:624-626: a path without weight files is skipped with a warning.
      set_err(err, err_cap, "Dense module files not found for path: " + std::string(dense_path));
      return;
    }
    for (auto& r : h->replicas) r->add_dense(dir);
    h->staged = false;
  });
  return rc;
}

void tei_b200_destroy(tei_b200_t* h) { delete h; }

int tei_b200_health(tei_b200_t* h) {
  if (!h) return TEI_B200_ERR_UNHEALTHY;
  if (h->healthy) return TEI_B200_OK;
  // One-token probe, like backends/src/lib.rs:393-409.
  const uint32_t ids[1] = {0}, types[1] = {0}, pos[1] = {0}, cu[2] = {0, 1}, idx[1] = {0};
  const ModelSpec& s = h->spec;
  int rc;
  if (s.classifier) {
    std::vector<float> scores(std::max(s.n_classes, 1));
    rc = tei_b200_predict(h, ids, types, pos, 1, cu, 1, 1, scores.data(), nullptr, 0);
  } else {
    std::vector<float> outv(static_cast<size_t>(h->replicas[0]->output_dim()));
    rc = tei_b200_embed(h, ids, types, pos, 1, cu, 1, 1, idx, 1, nullptr, 0, 0, outv.data(), nullptr, nullptr, 0);
  }
  return rc == TEI_B200_OK ? TEI_B200_OK : TEI_B200_ERR_UNHEALTHY;
}

int tei_b200_is_padded(const tei_b200_t*) { return 0; }
int tei_b200_max_batch_size(const tei_b200_t*) { return -1; }
int tei_b200_output_dim(const tei_b200_t* h) { return h ? h->replicas[0]->output_dim() : 0; }
int tei_b200_hidden_size(const tei_b200_t* h) {
  if (!h) return 0;
  return h->spec.pool == POOL_SPLADE ? h->spec.hidden : h->replicas[0]->raw_dim();
}
int tei_b200_num_classes(const tei_b200_t* h) { return h ? h->spec.n_classes : 0; }
int tei_b200_position_offset(const tei_b200_t* h) { return h ? h->spec.position_offset : 0; }

int tei_b200_embed(tei_b200_t* h, const uint32_t* input_ids, const uint32_t* token_type_ids,
                   const uint32_t* position_ids, size_t n_tokens,
                   const uint32_t* cumulative_seq_lengths, size_t n_seqs, uint32_t max_length,
                   const uint32_t* pooled_idx, size_t n_pooled, const uint32_t* raw_idx,
                   size_t n_raw, int normalize, float* pooled_out, float* raw_out, char* err,
                   size_t err_cap) {
  if (!h) return TEI_B200_ERR_UNHEALTHY;
  return guarded(h, err, err_cap, [&]() {
    if (h->spec.classifier) throw TeiError(ERR_INFERENCE, "`embed` is not implemented for classifier models");
    if ((n_pooled && !pooled_out) || (n_raw && !raw_out)) throw TeiError(ERR_INFERENCE, "null output buffer");
    HostBatch b = make_batch(input_ids, token_type_ids, position_ids, n_tokens, cumulative_seq_lengths,
                             n_seqs, max_length, pooled_idx, n_pooled, raw_idx, n_raw);
    do_stage(h, b, false, normalize != 0);
    do_run(h);
    do_fetch(h, pooled_out, raw_out, nullptr);
  });
}

int tei_b200_predict(tei_b200_t* h, const uint32_t* input_ids, const uint32_t* token_type_ids,
                     const uint32_t* position_ids, size_t n_tokens,
                     const uint32_t* cumulative_seq_lengths, size_t n_seqs, uint32_t max_length,
                     float* scores_out, char* err, size_t err_cap) {
  if (!h) return TEI_B200_ERR_UNHEALTHY;
  return guarded(h, err, err_cap, [&]() {
    if (!h->spec.classifier) throw TeiError(ERR_INFERENCE, "`predict` is not implemented for this model");
    if (!scores_out) throw TeiError(ERR_INFERENCE, "null output buffer");
    HostBatch b = make_batch(input_ids, token_type_ids, position_ids, n_tokens, cumulative_seq_lengths,
                             n_seqs, max_length, nullptr, 0, nullptr, 0);
    do_stage(h, b, true, false);
    do_run(h);
    do_fetch(h, nullptr, nullptr, scores_out);
  });
}

int tei_b200_num_replicas(const tei_b200_t* h) { return h ? static_cast<int>(h->replicas.size()) : 0; }

// The whole batch on one replica.  Nothing of the handle's own staged-batch state is touched, so
// calls with different replica indices may run at the same time from different threads.
int tei_b200_embed_on(tei_b200_t* h, int replica, const uint32_t* input_ids,
                      const uint32_t* token_type_ids, const uint32_t* position_ids, size_t n_tokens,
                      const uint32_t* cumulative_seq_lengths, size_t n_seqs, uint32_t max_length,
                      const uint32_t* pooled_idx, size_t n_pooled, const uint32_t* raw_idx,
                      size_t n_raw, int normalize, float* pooled_out, float* raw_out, char* err,
                      size_t err_cap) {
  if (!h) return TEI_B200_ERR_UNHEALTHY;
  return guarded(h, err, err_cap, [&]() {
    if (replica < 0 || replica >= static_cast<int>(h->replicas.size())) throw TeiError(ERR_INFERENCE, "replica index out of range");
    if (h->spec.classifier) throw TeiError(ERR_INFERENCE, "`embed` is not implemented for classifier models");
    if ((n_pooled && !pooled_out) || (n_raw && !raw_out)) throw TeiError(ERR_INFERENCE, "null output buffer");
    HostBatch b = make_batch(input_ids, token_type_ids, position_ids, n_tokens, cumulative_seq_lengths,
                             n_seqs, max_length, pooled_idx, n_pooled, raw_idx, n_raw);
    precheck(b);
    std::lock_guard<std::mutex> lock(*h->replica_locks[replica]);
    Replica& r = *h->replicas[replica];
    r.stage(b, false, normalize != 0);
    r.run();
    r.fetch(pooled_out, raw_out, nullptr);
  });
}

int tei_b200_predict_on(tei_b200_t* h, int replica, const uint32_t* input_ids,
                        const uint32_t* token_type_ids, const uint32_t* position_ids, size_t n_tokens,
                        const uint32_t* cumulative_seq_lengths, size_t n_seqs, uint32_t max_length,
                        float* scores_out, char* err, size_t err_cap) {
  if (!h) return TEI_B200_ERR_UNHEALTHY;
  return guarded(h, err, err_cap, [&]() {
    if (replica < 0 || replica >= static_cast<int>(h->replicas.size())) throw TeiError(ERR_INFERENCE, "replica index out of range");
    if (!h->spec.classifier) throw TeiError(ERR_INFERENCE, "`predict` is not implemented for this model");
    if (!scores_out) throw TeiError(ERR_INFERENCE, "null output buffer");
    HostBatch b = make_batch(input_ids, token_type_ids, position_ids, n_tokens, cumulative_seq_lengths,
                             n_seqs, max_length, nullptr, 0, nullptr, 0);
    precheck(b);
    std::lock_guard<std::mutex> lock(*h->replica_locks[replica]);
    Replica& r = *h->replicas[replica];
    r.stage(b, true, false);
    r.run();
    r.fetch(nullptr, nullptr, scores_out);
  });
}

int tei_b200_stage(tei_b200_t* h, const uint32_t* input_ids, const uint32_t* token_type_ids,
                   const uint32_t* position_ids, size_t n_tokens,
                   const uint32_t* cumulative_seq_lengths, size_t n_seqs, uint32_t max_length,
                   const uint32_t* pooled_idx, size_t n_pooled, const uint32_t* raw_idx,
                   size_t n_raw, int normalize, int predict, char* err, size_t err_cap) {
  if (!h) return TEI_B200_ERR_UNHEALTHY;
  return guarded(h, err, err_cap, [&]() {
    HostBatch b = make_batch(input_ids, token_type_ids, position_ids, n_tokens, cumulative_seq_lengths,
                             n_seqs, max_length, pooled_idx, n_pooled, raw_idx, n_raw);
    if (predict && !h->spec.classifier) throw TeiError(ERR_INFERENCE, "`predict` is not implemented for this model");
    if (!predict && h->spec.classifier) throw TeiError(ERR_INFERENCE, "`embed` is not implemented for classifier models");
    do_stage(h, b, predict != 0, normalize != 0);
  });
}

int tei_b200_run_staged(tei_b200_t* h, char* err, size_t err_cap) {
  if (!h) return TEI_B200_ERR_UNHEALTHY;
  return guarded(h, err, err_cap, [&]() { do_run(h); });
}

int tei_b200_sync(tei_b200_t* h, char* err, size_t err_cap) {
  if (!h) return TEI_B200_ERR_UNHEALTHY;
  return guarded(h, err, err_cap, [&]() { do_sync(h); });
}

int tei_b200_fetch(tei_b200_t* h, float* pooled_out, float* raw_out, float* scores_out, char* err,
                   size_t err_cap) {
  if (!h) return TEI_B200_ERR_UNHEALTHY;
  return guarded(h, err, err_cap, [&]() { do_fetch(h, pooled_out, raw_out, scores_out); });
}

int tei_b200_run_staged_timed(tei_b200_t* h, int steps, double* device_ms, char* err, size_t err_cap) {
  if (!h) return TEI_B200_ERR_UNHEALTHY;
  return guarded(h, err, err_cap, [&]() {
    if (!h->staged) throw TeiError(ERR_INFERENCE, "no staged batch");
    if (steps <= 0) throw TeiError(ERR_INFERENCE, "steps must be positive");
    double worst = 0.0;
    if (h->shards.empty()) {
      worst = h->replicas[0]->timed_runs(steps);
    } else {
      std::vector<double> ms(h->shards.size(), 0.0);
      for_each_shard_parallel(h, [&](Replica& r, Shard& sh) { ms[&sh - h->shards.data()] = r.timed_runs(steps); });
      for (double v : ms) worst = std::max(worst, v);
    }
    if (device_ms) *device_ms = worst;
  });
}

int tei_b200_set_profiling(tei_b200_t* h, int on) {
  if (!h) return TEI_B200_ERR_UNHEALTHY;
  return guarded(h, nullptr, 0, [&]() {
    for (auto& r : h->replicas) r->set_profiling(on != 0);
  });
}

int tei_b200_kernel_times(const tei_b200_t* h, double* ms_out, double* launches_out, int n) {
  if (!h || !ms_out || !launches_out || n <= 0) return 0;
  const int m = std::min(n, static_cast<int>(KC_COUNT));
  for (int i = 0; i < m; ++i) {
    ms_out[i] = 0.0;
    launches_out[i] = 0.0;
  }
  for (const auto& r : h->replicas) {
    double ms[KC_COUNT], ln[KC_COUNT];
    r->kernel_times(ms, ln, KC_COUNT);
    for (int i = 0; i < m; ++i) {
      ms_out[i] = std::max(ms_out[i], ms[i]);
      launches_out[i] += ln[i];
    }
  }
  return m;
}

int tei_b200_stats(const tei_b200_t* h, double* out, int n) {
  if (!h || !out || n <= 0) return 0;
  double v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (const auto& r : h->replicas) {
    const ReplicaStats& s = r->stats();
    v[0] = std::max(v[0], s.last_gpu_ms);
    v[1] += s.last_h2d_bytes;
    v[2] += s.last_d2h_bytes;
    v[3] += s.last_launches;
    v[4] += s.last_tokens;
    v[5] = std::max(v[5], s.calls);
    v[6] = std::max(v[6], s.total_gpu_ms);
    v[7] += s.total_tokens;
  }
  const int m = std::min(n, 8);
  for (int i = 0; i < m; ++i) out[i] = v[i];
  return m;
}

int tei_b200_plan_shards(const uint32_t* cumulative_seq_lengths, size_t n_seqs, int n_shards,
                         double linear_cost, double quadratic_cost, int* shard_of_seq) {
  if (!cumulative_seq_lengths || !shard_of_seq || n_shards <= 0) return TEI_B200_ERR_INFERENCE;
  plan_shards(cumulative_seq_lengths, static_cast<int>(n_seqs), n_shards, linear_cost, quadratic_cost,
              shard_of_seq);
  return TEI_B200_OK;
}

}  // extern "C"
