/* N backend threads over one handle, in plain C over the C ABI.
 *
 * The reference's router starts ONE backend thread that takes one batch at a time
 * (backends/src/lib.rs:612-647) while the batching task keeps one more batch ready
 * (core/src/infer.rs:547-625).  This program is the N-thread form of that loop, the way a router
 * with one backend thread per replica would run it: the main thread plays the batching side
 * (tokenised requests appended to the queue, core/src/queue.rs:67-75), every backend thread i
 * repeats NextBatch (queue.rs:118-195) -> tei_b200_embed_on(handle, i, batch) and files the
 * pooled rows under the requests' tags.  Afterwards every request is embedded again alone and
 * must give the same row.
 *
 * usage: router_threads <model_dir> <n_replicas> <n_requests> <vocab> <max_batch_tokens>
 * prints "ok batches=<n> per_thread=<a,b,..> max_abs_diff=<x>" and exits 0, or a message and
 * a non-zero code. */
#include <math.h>
#include <pthread.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "tei_b200.h"
#include "tei_b200_queue.h"

#define MAX_REPLICAS 16

typedef struct {
  tei_b200_t* h;
  tei_b200_queue_t* q;
  int replica;
  size_t max_tokens, max_seqs;
  int dim;
  float* rows;          /* [n_requests, dim], filled by tag */
  unsigned char* seen;  /* [n_requests] */
  volatile int* producer_done;
  int batches;
  int rc;
  char err[256];
} worker_t;

static void* backend_thread(void* arg) {
  worker_t* w = (worker_t*)arg;
  uint32_t* ids = malloc(w->max_tokens * 4);
  uint32_t* types = malloc(w->max_tokens * 4);
  uint32_t* pos = malloc(w->max_tokens * 4);
  uint32_t* cu = malloc((w->max_seqs + 1) * 4);
  uint32_t* pooled = malloc(w->max_seqs * 4);
  uint32_t* raw = malloc(w->max_seqs * 4);
  uint64_t* tags = malloc(w->max_seqs * 8);
  float* out = malloc(w->max_seqs * (size_t)w->dim * 4);
  for (;;) {
    size_t nt = 0, ns = 0, np = 0, nr = 0;
    uint32_t max_len = 0;
    const int done_before = *w->producer_done;
    int rc = tei_b200_queue_next_batch(w->q, ids, types, pos, w->max_tokens, cu, pooled, raw, tags, w->max_seqs,
                                       &nt, &ns, &np, &nr, &max_len);
    if (rc != TEI_B200_OK) {
      w->rc = rc;
      snprintf(w->err, sizeof w->err, "next_batch failed");
      break;
    }
    if (ns == 0) {
      if (done_before) break; /* queue empty and nothing more will come */
      continue;
    }
    rc = tei_b200_embed_on(w->h, w->replica, ids, types, pos, nt, cu, ns, max_len, pooled, np, raw, nr, 0, out,
                           NULL, w->err, sizeof w->err);
    if (rc != TEI_B200_OK) {
      w->rc = rc;
      break;
    }
    for (size_t i = 0; i < np; ++i) { /* pooled row i belongs to batch position pooled[i] */
      const uint64_t tag = tags[pooled[i]];
      memcpy(w->rows + tag * (size_t)w->dim, out + i * (size_t)w->dim, (size_t)w->dim * 4);
      w->seen[tag] += 1;
    }
    w->batches += 1;
  }
  free(ids); free(types); free(pos); free(cu); free(pooled); free(raw); free(tags); free(out);
  return NULL;
}

static uint32_t lcg(uint32_t* s) {
  *s = *s * 1664525u + 1013904223u;
  return *s >> 8;
}

int main(int argc, char** argv) {
  if (argc != 6) {
    fprintf(stderr, "usage: %s model_dir n_replicas n_requests vocab max_batch_tokens\n", argv[0]);
    return 64;
  }
  const int n_rep = atoi(argv[2]);
  const int n_req = atoi(argv[3]);
  const uint32_t vocab = (uint32_t)atoi(argv[4]);
  const size_t max_tokens = (size_t)atoi(argv[5]);
  if (n_rep < 1 || n_rep > MAX_REPLICAS || n_req < 1 || max_tokens < 300) return 64;
  int devices[MAX_REPLICAS];
  for (int i = 0; i < n_rep; ++i) devices[i] = 0; /* replicas of one GPU: own stream, workspace, pinned block each */
  char err[512];
  tei_b200_t* h = NULL;
  int rc = tei_b200_create(argv[1], "float16", TEI_B200_EMBEDDING, TEI_B200_POOL_MEAN, devices, n_rep, &h, err, sizeof err);
  if (rc != TEI_B200_OK) {
    fprintf(stderr, "create: %d %s\n", rc, err);
    return 2;
  }
  if (tei_b200_num_replicas(h) != n_rep) return 3;
  const int dim = tei_b200_output_dim(h);
  tei_b200_queue_t* q = NULL;
  if (tei_b200_queue_create(0, max_tokens, 0, &q) != TEI_B200_OK) return 4;

  /* the requests: lengths 1..300, ids below the vocabulary */
  uint32_t seed = 12345u;
  uint32_t** req_ids = malloc((size_t)n_req * sizeof *req_ids);
  size_t* req_len = malloc((size_t)n_req * sizeof *req_len);
  for (int r = 0; r < n_req; ++r) {
    req_len[r] = 1 + lcg(&seed) % 300;
    req_ids[r] = malloc(req_len[r] * 4);
    for (size_t t = 0; t < req_len[r]; ++t) req_ids[r][t] = lcg(&seed) % vocab;
  }
  float* rows = calloc((size_t)n_req * (size_t)dim, 4);
  unsigned char* seen = calloc((size_t)n_req, 1);
  volatile int producer_done = 0;
  worker_t w[MAX_REPLICAS];
  pthread_t th[MAX_REPLICAS];
  for (int i = 0; i < n_rep; ++i) {
    memset(&w[i], 0, sizeof w[i]);
    w[i].h = h; w[i].q = q; w[i].replica = i; w[i].max_tokens = max_tokens; w[i].max_seqs = max_tokens;
    w[i].dim = dim; w[i].rows = rows; w[i].seen = seen; w[i].producer_done = &producer_done;
    if (pthread_create(&th[i], NULL, backend_thread, &w[i]) != 0) return 5;
  }
  /* the batching side: requests arrive while the backend threads are already pulling */
  for (int r = 0; r < n_req; ++r) {
    if (tei_b200_queue_append(q, req_ids[r], NULL, NULL, req_len[r], 0, 1, (uint64_t)r) != TEI_B200_OK) return 6;
  }
  producer_done = 1;
  int batches = 0;
  for (int i = 0; i < n_rep; ++i) {
    pthread_join(th[i], NULL);
    if (w[i].rc != TEI_B200_OK) {
      fprintf(stderr, "backend thread %d: %d %s\n", i, w[i].rc, w[i].err);
      return 7;
    }
    batches += w[i].batches;
  }
  if (tei_b200_queue_len(q) != 0) return 8;
  for (int r = 0; r < n_req; ++r) {
    if (seen[r] != 1) {
      fprintf(stderr, "request %d answered %d times\n", r, (int)seen[r]);
      return 9;
    }
  }
  /* every request again, alone, through the whole-handle call */
  float* one = malloc((size_t)dim * 4);
  uint32_t* pos = malloc(300 * 4);
  uint32_t* zeros = calloc(300, 4); /* token type ids: the queue fills zeros in, here they are explicit */
  for (uint32_t t = 0; t < 300; ++t) pos[t] = t;
  double worst = 0.0;
  for (int r = 0; r < n_req; ++r) {
    const uint32_t cu[2] = {0, (uint32_t)req_len[r]};
    const uint32_t idx[1] = {0};
    rc = tei_b200_embed(h, req_ids[r], zeros, pos, req_len[r], cu, 1, (uint32_t)req_len[r], idx, 1, NULL, 0, 0, one,
                        NULL, err, sizeof err);
    if (rc != TEI_B200_OK) {
      fprintf(stderr, "single embed: %d %s\n", rc, err);
      return 10;
    }
    for (int j = 0; j < dim; ++j) {
      const double d = fabs((double)one[j] - (double)rows[(size_t)r * (size_t)dim + (size_t)j]);
      if (!(d <= worst)) worst = d; /* NaN ends up in worst too */
    }
  }
  if (!(worst <= 4e-3)) {
    fprintf(stderr, "rows differ: max abs diff %g\n", worst);
    return 11;
  }
  if (tei_b200_health(h) != TEI_B200_OK) return 12;
  printf("ok batches=%d per_thread=", batches);
  for (int i = 0; i < n_rep; ++i) printf("%d%s", w[i].batches, i + 1 < n_rep ? "," : "");
  printf(" max_abs_diff=%g\n", worst);
  tei_b200_queue_destroy(q);
  tei_b200_destroy(h);
  return 0;
}
