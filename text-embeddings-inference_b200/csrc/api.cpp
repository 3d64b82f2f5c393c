// extern "C" backend entry points (include/tei_b200.h): handle lifetime, error mapping, and the
// split of one packed batch over several GPU replicas.
#include "../../include/tei_b200.h"

#include "model.h"
#include "plan.h"
#include "split.h"

#include <algorithm>
#include <atomic>
#include <condition_variable>
#include <cstring>
#include <fstream>
#include <functional>
#include <memory>
#include <mutex>
#include <sstream>
#include <thread>

using namespace tei;

namespace {

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

// The thread that drives one replica of a multi-replica handle.  It lives as long as the handle
// and sleeps on a condition variable between calls, so a split embed / predict costs one wake-up
// per replica instead of thread creations.  Jobs never throw (the posting code wraps them).
class Worker {
 public:
  Worker() : thread_([this]() { loop(); }) {}
  ~Worker() {
    {
      std::lock_guard<std::mutex> g(m_);
      stop_ = true;
    }
    cv_.notify_all();
    thread_.join();
  }
  Worker(const Worker&) = delete;
  Worker& operator=(const Worker&) = delete;
  void post(std::function<void()> job) {
    {
      std::lock_guard<std::mutex> g(m_);
      job_ = std::move(job);
      pending_ = true;
      done_ = false;
    }
    cv_.notify_all();
  }
  void wait() {
    std::unique_lock<std::mutex> g(m_);
    cv_.wait(g, [this]() { return done_; });
  }

 private:
  void loop() {
    std::unique_lock<std::mutex> g(m_);
    for (;;) {
      cv_.wait(g, [this]() { return pending_ || stop_; });
      if (stop_) return;
      std::function<void()> job = std::move(job_);
      pending_ = false;
      g.unlock();
      job();
      g.lock();
      done_ = true;
      cv_.notify_all();
    }
  }
  std::mutex m_;
  std::condition_variable cv_;
  std::function<void()> job_;
  bool pending_ = false, done_ = true, stop_ = false;
  std::thread thread_;  // last member: the loop reads the others
};

}  // namespace

struct tei_b200 {
  ModelSpec spec;
  std::string model_dir;
  std::vector<std::unique_ptr<Replica>> replicas;
  // One lock per replica.  The per-replica entry points (one caller thread per replica) take
  // their replica's; the whole-handle entry points take all of them, in index order.  Two
  // threads that were given the same index by mistake, or a health probe next to per-replica
  // callers, queue up instead of corrupting a replica's staging buffers.
  std::vector<std::unique_ptr<std::mutex>> replica_locks;
  std::vector<std::unique_ptr<Worker>> workers;  // one per replica when there are several
  std::atomic<bool> healthy{true};
  // state of the staged batch (stage / run / sync / fetch)
  bool staged = false;
  bool staged_predict = false;
  std::vector<Shard> shards;   // all empty when a single replica took the whole batch
  bool split = false;          // the staged batch is spread over `shards`
  size_t staged_n_pooled = 0, staged_raw_rows = 0, staged_n_seqs = 0;
  double linear_cost = 1.0, quadratic_cost = 0.0;
};

namespace {

// Every replica lock of the handle, taken in index order.
struct AllReplicas {
  std::vector<std::unique_lock<std::mutex>> held;
  explicit AllReplicas(tei_b200* h) {
    held.reserve(h->replica_locks.size());
    for (auto& m : h->replica_locks) held.emplace_back(*m);
  }
};

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

// Runs fn(replica, shard) for every shard that holds sequences, each on its replica's own
// thread, and waits for all of them.  The first error of a shard is rethrown here.
template <class F>
void for_each_shard_parallel(tei_b200* h, F&& fn) {
  std::vector<size_t> posted;
  for (size_t d = 0; d < h->shards.size(); ++d) {
    if (h->shards[d].seqs.empty()) continue;
    Shard* sh = &h->shards[d];
    Replica* r = h->replicas[d].get();
    sh->err_kind = 0;
    h->workers[d]->post([sh, r, &fn]() {
      try {
        fn(*r, *sh);
      } catch (const TeiError& e) {
        sh->err_kind = e.kind;
        sh->err_msg = e.what();
      } catch (const std::exception& e) {
        sh->err_kind = ERR_INFERENCE;
        sh->err_msg = e.what();
      } catch (...) {
        sh->err_kind = ERR_INFERENCE;
        sh->err_msg = "unknown error";
      }
    });
    posted.push_back(d);
  }
  for (size_t d : posted) h->workers[d]->wait();
  for (auto& sh : h->shards) {
    if (sh.err_kind) {
      const int k = sh.err_kind;
      std::string m = sh.err_msg;
      sh.err_kind = 0;
      throw TeiError(k, m);
    }
  }
}

bool wants_split(const tei_b200* h, const HostBatch& b) { return h->replicas.size() > 1 && b.n_seqs > 1; }

void note_staged(tei_b200* h, const HostBatch& b, bool predict) {
  h->staged_predict = predict;
  h->staged_n_pooled = predict ? 0 : b.n_pooled;
  h->staged_n_seqs = b.n_seqs;
  size_t raw_rows = 0;
  if (!predict) {
    for (size_t i = 0; i < b.n_raw; ++i) raw_rows += b.cu_seqlens[b.raw_indices[i] + 1] - b.cu_seqlens[b.raw_indices[i]];
  }
  h->staged_raw_rows = raw_rows;
}

void do_stage(tei_b200* h, const HostBatch& b, bool predict, bool normalize) {
  precheck(b);
  h->staged = false;
  note_staged(h, b, predict);
  h->split = wants_split(h, b);
  if (!h->split) {
    h->replicas[0]->stage(b, predict, normalize);
  } else {
    assign_shards(b, predict, static_cast<int>(h->replicas.size()), h->linear_cost, h->quadratic_cost, h->shards);
    for_each_shard_parallel(h, [&](Replica& r, Shard& sh) {
      gather_shard_tokens(b, sh);
      r.stage(sh.view(), predict, normalize);
    });
  }
  h->staged = true;
}

void do_run(tei_b200* h) {
  if (!h->staged) throw TeiError(ERR_INFERENCE, "no staged batch");
  if (!h->split) {
    h->replicas[0]->run();
  } else {
    for_each_shard_parallel(h, [](Replica& r, Shard&) { r.run(); });
  }
}

void do_sync(tei_b200* h) {
  if (!h->staged) throw TeiError(ERR_INFERENCE, "no staged batch");
  if (!h->split) {
    h->replicas[0]->sync_and_check();
  } else {
    for_each_shard_parallel(h, [](Replica& r, Shard&) { r.sync_and_check(); });
  }
}

struct RowWidths {
  size_t D, DR, C;
};
RowWidths row_widths(const tei_b200* h) {
  return {static_cast<size_t>(h->replicas[0]->output_dim()), static_cast<size_t>(h->replicas[0]->raw_dim()),
          static_cast<size_t>(std::max(h->spec.n_classes, 1))};
}

void do_fetch(tei_b200* h, float* pooled_out, float* raw_out, float* scores_out) {
  if (!h->staged) throw TeiError(ERR_INFERENCE, "no staged batch");
  if (!h->split) {
    h->replicas[0]->fetch(pooled_out, raw_out, scores_out);
    return;
  }
  const RowWidths w = row_widths(h);
  const bool predict = h->staged_predict;
  for_each_shard_parallel(h, [&](Replica& r, Shard& sh) {
    size_shard_results(sh, predict, w.D, w.DR, w.C);
    r.fetch(sh.pooled.data(), sh.raw.data(), sh.scores.data());
    // every shard's rows go back to their original batch positions
    scatter_shard(sh, predict, w.D, w.DR, w.C, pooled_out, raw_out, scores_out);
  });
}

// embed / predict in one pass: with several replicas each replica's thread gathers its tokens,
// stages, runs, waits once, copies back and scatters its rows; the calling thread only plans the
// split and sleeps.
void do_all(tei_b200* h, const HostBatch& b, bool predict, bool normalize, float* pooled_out,
            float* raw_out, float* scores_out) {
  precheck(b);
  h->staged = false;
  note_staged(h, b, predict);
  h->split = wants_split(h, b);
  if (!h->split) {
    Replica& r = *h->replicas[0];
    r.stage(b, predict, normalize);
    h->staged = true;
    r.run();
    r.fetch(pooled_out, raw_out, scores_out);
    return;
  }
  assign_shards(b, predict, static_cast<int>(h->replicas.size()), h->linear_cost, h->quadratic_cost, h->shards);
  const RowWidths w = row_widths(h);
  for_each_shard_parallel(h, [&](Replica& r, Shard& sh) {
    gather_shard_tokens(b, sh);
    r.stage(sh.view(), predict, normalize);
    r.run();
    size_shard_results(sh, predict, w.D, w.DR, w.C);
    r.fetch(sh.pooled.data(), sh.raw.data(), sh.scores.data());
    scatter_shard(sh, predict, w.D, w.DR, w.C, pooled_out, raw_out, scores_out);
  });
  h->staged = true;
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
    if (h->replicas.size() > 1) {
      for (size_t i = 0; i < h->replicas.size(); ++i) h->workers.emplace_back(new Worker());
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
    AllReplicas all(h);
    for (auto& r : h->replicas) r->add_dense(dir);
    h->staged = false;
  });
  return rc;
}

void tei_b200_destroy(tei_b200_t* h) { delete h; }

int tei_b200_health(tei_b200_t* h) {
  if (!h) return TEI_B200_ERR_UNHEALTHY;
  if (h->healthy) return TEI_B200_OK;
  // One-token probe, like backends/src/lib.rs:393-409.  It runs on replica 0 under that
  // replica's lock and leaves the handle's staged-batch state alone, so it may be called while
  // other threads are inside the per-replica entry points.
  const uint32_t ids[1] = {0}, types[1] = {0}, pos[1] = {0}, cu[2] = {0, 1}, idx[1] = {0};
  const ModelSpec& s = h->spec;
  int rc;
  if (s.classifier) {
    std::vector<float> scores(std::max(s.n_classes, 1));
    rc = tei_b200_predict_on(h, 0, ids, types, pos, 1, cu, 1, 1, scores.data(), nullptr, 0);
  } else {
    std::vector<float> outv(static_cast<size_t>(h->replicas[0]->output_dim()));
    rc = tei_b200_embed_on(h, 0, ids, types, pos, 1, cu, 1, 1, idx, 1, nullptr, 0, 0, outv.data(), nullptr, nullptr, 0);
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
    AllReplicas all(h);
    do_all(h, b, false, normalize != 0, pooled_out, raw_out, nullptr);
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
    AllReplicas all(h);
    do_all(h, b, true, false, nullptr, nullptr, scores_out);
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
    AllReplicas all(h);
    do_stage(h, b, predict != 0, normalize != 0);
  });
}

int tei_b200_run_staged(tei_b200_t* h, char* err, size_t err_cap) {
  if (!h) return TEI_B200_ERR_UNHEALTHY;
  return guarded(h, err, err_cap, [&]() {
    AllReplicas all(h);
    do_run(h);
  });
}

int tei_b200_sync(tei_b200_t* h, char* err, size_t err_cap) {
  if (!h) return TEI_B200_ERR_UNHEALTHY;
  return guarded(h, err, err_cap, [&]() {
    AllReplicas all(h);
    do_sync(h);
  });
}

int tei_b200_fetch(tei_b200_t* h, float* pooled_out, float* raw_out, float* scores_out, char* err,
                   size_t err_cap) {
  if (!h) return TEI_B200_ERR_UNHEALTHY;
  return guarded(h, err, err_cap, [&]() {
    AllReplicas all(h);
    do_fetch(h, pooled_out, raw_out, scores_out);
  });
}

int tei_b200_run_staged_timed(tei_b200_t* h, int steps, double* device_ms, char* err, size_t err_cap) {
  if (!h) return TEI_B200_ERR_UNHEALTHY;
  return guarded(h, err, err_cap, [&]() {
    if (!h->staged) throw TeiError(ERR_INFERENCE, "no staged batch");
    if (steps <= 0) throw TeiError(ERR_INFERENCE, "steps must be positive");
    AllReplicas all(h);
    double worst = 0.0;
    if (!h->split) {
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
    AllReplicas all(h);
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

int tei_b200_set_last_layer_shortcut(tei_b200_t* h, int on) {
  if (!h) return TEI_B200_ERR_UNHEALTHY;
  return guarded(nullptr, nullptr, 0, [&]() {
    AllReplicas all(h);
    for (auto& r : h->replicas) r->set_last_layer_shortcut(on != 0);
  });
}

int tei_b200_set_fused_rope(tei_b200_t* h, int on) {
  if (!h) return TEI_B200_ERR_UNHEALTHY;
  return guarded(nullptr, nullptr, 0, [&]() {
    AllReplicas all(h);
    for (auto& r : h->replicas) r->set_fused_rope(on < 0 ? -1 : (on != 0 ? 1 : 0));
  });
}

int tei_b200_set_fused_residual(tei_b200_t* h, int on) {
  if (!h) return TEI_B200_ERR_UNHEALTHY;
  return guarded(nullptr, nullptr, 0, [&]() {
    AllReplicas all(h);
    for (auto& r : h->replicas) r->set_fused_residual(on != 0);
  });
}

int tei_b200_selftest_report_timeout(tei_b200_t* h, int replica, int device_code) {
  if (!h || replica < 0 || replica >= static_cast<int>(h->replicas.size()) || device_code <= 0) {
    return TEI_B200_ERR_INFERENCE;
  }
  return guarded(nullptr, nullptr, 0, [&]() {
    std::lock_guard<std::mutex> lock(*h->replica_locks[replica]);
    h->replicas[replica]->report_status_once(device_code);
  });
}

int tei_b200_split_echo(const uint32_t* input_ids, const uint32_t* token_type_ids, const uint32_t* position_ids,
                        size_t n_tokens, const uint32_t* cumulative_seq_lengths, size_t n_seqs,
                        const uint32_t* pooled_idx, size_t n_pooled, const uint32_t* raw_idx, size_t n_raw,
                        int predict, int n_shards, double linear_cost, double quadratic_cost, int width,
                        float* pooled_out, float* raw_out, float* scores_out, int* shard_tokens_out) {
  if (n_shards <= 0 || width <= 0) return TEI_B200_ERR_INFERENCE;
  try {
    HostBatch b = make_batch(input_ids, token_type_ids, position_ids, n_tokens, cumulative_seq_lengths, n_seqs, 0,
                             pooled_idx, n_pooled, raw_idx, n_raw);
    precheck(b);
    std::vector<Shard> shards;
    assign_shards(b, predict != 0, n_shards, linear_cost, quadratic_cost, shards);
    const size_t W = static_cast<size_t>(width);
    for (size_t d = 0; d < shards.size(); ++d) {
      Shard& sh = shards[d];
      if (shard_tokens_out) shard_tokens_out[d] = 0;
      if (sh.seqs.empty()) continue;
      gather_shard_tokens(b, sh);
      const HostBatch v = sh.view();
      precheck(v);  // the sub-batch is a well-formed batch of its own
      if (shard_tokens_out) shard_tokens_out[d] = static_cast<int>(v.n_tokens);
      size_shard_results(sh, predict != 0, W, W, W);
      // Stand-in for the forward, computed from the SUB-batch alone: a pooled or score row is
      // (sum of the sequence's ids mod 65521) + column, a raw row id + 7 type + 13 position + column.
      auto seq_value = [&](uint32_t local) {
        uint64_t acc = 0;
        for (uint32_t t = v.cu_seqlens[local]; t < v.cu_seqlens[local + 1]; ++t) acc += v.input_ids[t];
        return static_cast<float>(acc % 65521u);
      };
      for (size_t i = 0; i < v.n_pooled; ++i) {
        for (size_t j = 0; j < W; ++j) sh.pooled[i * W + j] = seq_value(v.pooled_indices[i]) + static_cast<float>(j);
      }
      size_t row = 0;
      for (size_t i = 0; i < v.n_raw; ++i) {
        const uint32_t l = v.raw_indices[i];
        for (uint32_t t = v.cu_seqlens[l]; t < v.cu_seqlens[l + 1]; ++t, ++row) {
          const float base = static_cast<float>(v.input_ids[t] % 4096u + 7u * v.token_type_ids[t] + 13u * (v.position_ids[t] % 4096u));
          for (size_t j = 0; j < W; ++j) sh.raw[row * W + j] = base + static_cast<float>(j);
        }
      }
      if (predict) {
        for (size_t i = 0; i < v.n_seqs; ++i) {
          for (size_t j = 0; j < W; ++j) sh.scores[i * W + j] = seq_value(static_cast<uint32_t>(i)) + static_cast<float>(j);
        }
      }
      scatter_shard(sh, predict != 0, W, W, W, pooled_out, raw_out, scores_out);
    }
    return TEI_B200_OK;
  } catch (...) {
    return TEI_B200_ERR_INFERENCE;
  }
}

int tei_b200_compile_compute_cap(void) { return tei::kCompileComputeCap; }

int tei_b200_compute_cap_matching(int runtime_cap, int compile_cap) {
  return tei::compute_cap_matching(runtime_cap, compile_cap) ? 1 : 0;
}

int tei_b200_plan_shards(const uint32_t* cumulative_seq_lengths, size_t n_seqs, int n_shards,
                         double linear_cost, double quadratic_cost, int* shard_of_seq) {
  if (!cumulative_seq_lengths || !shard_of_seq || n_shards <= 0) return TEI_B200_ERR_INFERENCE;
  plan_shards(cumulative_seq_lengths, static_cast<int>(n_seqs), n_shards, linear_cost, quadratic_cost,
              shard_of_seq);
  return TEI_B200_OK;
}

}  // extern "C"
