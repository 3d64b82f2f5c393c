// Variable-length (unpadded) attention on tcgen05 tensor cores.
//
// Replaces the reference's flash_attn_varlen call (backends/candle/src/flash_attn.rs:23-120;
// call sites models/flash_bert.rs:95-108, flash_nomic.rs:83-96, flash_qwen3.rs:155-169):
// for every sequence s of the packed batch and head h,
//     out = softmax(scale * Q_s K_s^T  [- slope_h * |i - j|]  [window / causal mask]) V_s
// with q-head h reading kv-head h / (n_heads / n_kv_heads); key j counts for query i when
// i - window_left <= j <= i + window_right (causal: right window 0).  Q, K and V are strided
// views of the projection output (token-major rows), exactly as the reference passes them.
//
// Persistent CTAs (two per SM) walk the (sequence, 128-row query
// tile, head) work units, sorted by cost and handed out in alternating direction, in steps of
// 64 keys.  Everything a step needs is multi-buffered (AttnCfg), so the three roles of a CTA
// run decoupled:
//   warp 5 (one lane)  TMA producer: Q tile per unit, K and V tiles per step into two rings,
//                      128-byte swizzle, plain per-CTA loads (no cluster multicast); runs ahead
//                      of the MMAs by the free stages and, with two Q buffers, by one unit.
//   warp 4 (one lane)  MMA issuer, polling two streams: S = Q K^T of a step into one of S_BUFS
//                      64-column score tiles in TMEM, up to S_BUFS - 1 steps ahead of the
//                      softmax and across unit boundaries; O += P V of a step into an output
//                      tile in TMEM behind the score tiles, with P read from TMEM (A operand)
//                      and V from shared memory (MN-major operand).
//   warps 0-3          one query row per thread: the 64 scores of the step are read from TMEM
//                      into registers once; exp2 against the row's running maximum in one pass
//                      (a row maximum pass first only at a unit's first step and when a
//                      maximum has to be raised), P written back as fp16/bf16
//                      over the row's own scores in TMEM, so P never touches shared memory (the
//                      kernel is bound by shared-memory bandwidth otherwise: every MMA operand
//                      read and every TMA write goes through it).  O stays in TMEM across the
//                      key steps; the running maximum is raised lazily (only when a step's sum
//                      of probabilities against the old maximum exceeds 2^8), in which case
//                      the rows rescale their partial output in TMEM.  A finished unit's rows
//                      are read, normalised and staged in shared memory (128-byte swizzle,
//                      conflict-free both ways); a warp whose 32 rows all belong to
//                      the sequence hands them to one TMA store, a ragged one writes them back
//                      itself as whole 128-byte lines.
// Every mbarrier wait is bounded and reports through *status instead of spinning forever.
#include "kernels.h"
#include "ptx.cuh"
#include "tmap.h"

#include <atomic>

namespace tei {
namespace {

constexpr int BQ = 128;  // query rows per CTA
constexpr int BKV = 64;  // keys per step
constexpr int ATTN_THREADS = 192;

// Depth of the pipeline per head size.  A softmax warp needs about 1,800 cycles for the 64 keys
// of a step (512 of them on the exp2 unit alone), the tensor pipe 320 (D = 64) to 640 (D = 128):
// what bounds the kernel is how many softmax warps an SM keeps busy, so both head sizes run two
// CTAs per SM (eight softmax warps, two per scheduler), each with half of the TMEM columns and
// of the shared memory.  D = 64 (and 32): two score tiles, two output tiles, two Q buffers, four
// K/V stages (a K/V tile takes about 1,750 cycles from the load's issue to the barrier, more
// than a step: with three stages the ring, not the softmax, set the pace).  D = 128: two score tiles, one output tile, one Q buffer and only two K and two V
// stages (112 KB per CTA), which is enough because the K ring is released early (see K_EARLY).
template <int D>
struct AttnCfg {
  static constexpr int S_BUFS = 2;                     // score / P tiles of 64 columns
  static constexpr int O_BUFS = (D <= 64) ? 2 : 1;     // output tiles of D columns
  static constexpr int Q_BUFS = (D <= 64) ? 2 : 1;
  // K and V tiles live in two rings of their own: a K tile is free again as soon as the S MMA
  // that read it is done, long before the P V of the same step releases the V tile, so with
  // separate rings two stages each already let the next K arrive a whole step early.
  static constexpr int K_STAGES = (D <= 64) ? 4 : 2;
  static constexpr int V_STAGES = (D <= 64) ? 4 : 2;
  // With more stages than score tiles (D = 64) the early release buys nothing: there a K tile is
  // released together with the V tile of its step and both are loaded in the same turn.
  static constexpr bool K_EARLY = K_STAGES <= S_BUFS;
  static constexpr int K_LEAD = K_EARLY ? 1 : 0;       // steps K is loaded ahead of V
  static_assert(K_EARLY || K_STAGES == V_STAGES, "shared release needs rings of one length");
  static constexpr int CTAS_PER_SM = 2;
  static constexpr uint32_t TMEM_COLS = 256;
  static_assert(S_BUFS * BKV + O_BUFS * D <= TMEM_COLS, "TMEM budget");
};

// Head sizes of 64 and more are held as 64-element atoms (128-byte rows, 128-byte swizzle), one
// after the other; head_dim 32 is one atom of 64-byte rows with the 64-byte swizzle.
template <int D>
struct AttnSmem {
  using C = AttnCfg<D>;
  static constexpr int ATOM = D < 64 ? D : 64;   // elements per swizzle row
  static constexpr int ROW_BYTES = ATOM * 2;
  static constexpr int D_ATOMS = D / ATOM;
  static constexpr int Q_BYTES = BQ * D * 2;
  static constexpr int KV_BYTES = BKV * D * 2;   // one K or one V tile
  static constexpr int STAGE_BYTES = BQ * 128;   // output rows, 64 columns at a time
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + C::Q_BUFS * Q_BYTES;
  static constexpr int OFF_V = OFF_K + C::K_STAGES * KV_BYTES;
  static constexpr int OFF_STAGE = OFF_V + C::V_STAGES * KV_BYTES;
  static constexpr int OFF_BAR = OFF_STAGE + STAGE_BYTES;
  // No alignment slack: two CTAs of the D = 64 variant must fit in one SM's shared memory.  The
  // kernel checks that the dynamic window is 1024-byte aligned and reports an error otherwise.
  static constexpr int TOTAL = OFF_BAR + 320;  // 32 mbarrier slots + the TMEM address slot
  static_assert(C::CTAS_PER_SM * (TOTAL + 1024) <= 228 * 1024, "shared memory budget");
};

struct AttnParams {
  void* out;
  const int* work;  // [n_work][4] = {seq_start, seq_len, q0, first key of the unit (multiple of 64)}
  int n_work;
  int n_heads, n_kv_heads;
  int ld_o;
  int win_left, win_right;  // keys j of query i count when i - win_left <= j <= i + win_right; -1: no limit
  float scale_log2;         // scale * log2(e)
  const float* alibi_slopes;
  int* status;
};

template <class T>
__device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// One thread owns one query row of the 64-key score tile; the row is read from TMEM into
// registers once per step (one wait) and both passes work from there.
// Only the first n_chunks * 32 columns are touched.  MASKED: only keys [lo, lim) count.
// ALIBI: subtract slope * |rel - key| (rel = query position - first key position of the tile).
//
// Pass 1: row maximum in the scaled log2 domain (-inf when the row sees no key).
template <bool MASKED, bool ALIBI>
__device__ __forceinline__ float row_max(const uint32_t (&sc)[BKV / 32][32], int lo, int lim, int n_chunks, float sl2,
                                         float slope, int rel) {
  const unsigned span = static_cast<unsigned>(max(0, lim - lo));  // visible keys: [lo, lim)
  float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // four independent chains
#pragma unroll
  for (int c = 0; c < BKV / 32; ++c) {
    if (c >= n_chunks) break;
    const uint32_t (&s)[32] = sc[c];
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      float x0 = __uint_as_float(s[i]), x1 = __uint_as_float(s[i + 1]);
      const int kk = c * 32 + i;
      if (ALIBI) {
        x0 = x0 * sl2 - slope * fabsf(static_cast<float>(rel - kk));
        x1 = x1 * sl2 - slope * fabsf(static_cast<float>(rel - kk - 1));
      }
      if (MASKED) {
        x0 = static_cast<unsigned>(kk - lo) < span ? x0 : -INFINITY;
        x1 = static_cast<unsigned>(kk + 1 - lo) < span ? x1 : -INFINITY;
      }
      mx[(i >> 1) & 3] = ptx::max3(mx[(i >> 1) & 3], x0, x1);
    }
  }
  const float mx_all = fmaxf(ptx::max3(mx[0], mx[1], mx[2]), mx[3]);
  return ALIBI ? mx_all : mx_all * sl2;  // the scale is positive, so the maximum commutes with it
}

// Pass 2: p = 2^(score - m_use), written as T back into TMEM over the row's own scores (two
// values per 32-bit column from column `t_p` on: the A operand of the P V MMA); returns the row
// sum.
template <class T, bool MASKED, bool ALIBI>
__device__ __forceinline__ float write_probs(const uint32_t (&sc)[BKV / 32][32], uint32_t t_p, int lo, int lim,
                                             int n_chunks, float sl2, float slope, int rel, float m_use) {
  const unsigned span = static_cast<unsigned>(max(0, lim - lo));  // visible keys: [lo, lim)
  // Packed pairs: one FMA scales and shifts two scores, one add accumulates two probabilities.
  const uint64_t sl2_2 = ptx::pack_f32x2(sl2, sl2), neg_m2 = ptx::pack_f32x2(-m_use, -m_use);
  uint64_t acc[2] = {0ull, 0ull};  // two independent accumulator pairs
#pragma unroll
  for (int c = 0; c < BKV / 32; ++c) {
    if (c >= n_chunks) break;
    const uint32_t (&s)[32] = sc[c];
    uint32_t pk[16];
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      const int kk = c * 32 + i;
      float e0, e1;
      if (ALIBI) {
        e0 = ex2_fast(__uint_as_float(s[i]) * sl2 - slope * fabsf(static_cast<float>(rel - kk)) - m_use);
        e1 = ex2_fast(__uint_as_float(s[i + 1]) * sl2 - slope * fabsf(static_cast<float>(rel - kk - 1)) - m_use);
      } else {
        float a0, a1;
        ptx::unpack_f32x2(ptx::fma_f32x2(ptx::pack_f32x2(__uint_as_float(s[i]), __uint_as_float(s[i + 1])), sl2_2, neg_m2), a0, a1);
        e0 = ex2_fast(a0);
        e1 = ex2_fast(a1);
      }
      if (MASKED) {
        e0 = static_cast<unsigned>(kk - lo) < span ? e0 : 0.f;
        e1 = static_cast<unsigned>(kk + 1 - lo) < span ? e1 : 0.f;
      }
      acc[(i >> 1) & 1] = ptx::add_f32x2(acc[(i >> 1) & 1], ptx::pack_f32x2(e0, e1));
      pk[i / 2] = pack2<T>(e0, e1);
    }
    ptx::tmem_st16(t_p + c * 16, pk);  // 32 keys = 16 columns of packed pairs
  }
  float s0, s1, s2, s3;
  ptx::unpack_f32x2(acc[0], s0, s1);
  ptx::unpack_f32x2(acc[1], s2, s3);
  return (s0 + s1) + (s2 + s3);
}

// After a unit's first step the probabilities of a step are first taken relative to the maximum
// the row already has (one pass, no dependency on a maximum of this step).  The result stands
// as long as the step's sum stays below this bound: then no probability exceeded it either (far
// inside fp16 / bf16 range), and the accumulator in TMEM needs no rescaling.  A larger sum (inf
// and NaN included) means some exponent was above log2(bound / 64) = 2: the row takes the true
// maximum of the step and its warp redoes the step with the two passes.
constexpr float kLazySumBound = 256.0f;


// ALIBI is a compile-time switch: the softmax code of the models without a positional bias
// (all but JinaBERT with ALiBi) then holds two variants of each pass instead of three.
// LWIN (a left window is set) is one too: only then can a row pass a key tile without seeing a
// key, and the softmax loop of every other model is spared the test for it.
template <class T, int D, bool ALIBI, bool LWIN>
__global__ void __launch_bounds__(ATTN_THREADS, AttnCfg<D>::CTAS_PER_SM)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_q,
                         const __grid_constant__ CUtensorMap tm_k,
                         const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                         const AttnParams p) {
  using L = AttnSmem<D>;
  constexpr int D_ATOMS = L::D_ATOMS;  // swizzle atoms per head
  constexpr int ATOM = L::ATOM, ROW_BYTES = L::ROW_BYTES;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if (ptx::smem_u32(smem) & 1023u) {  // swizzled operand tiles need 1024-byte alignment
    ptx::grid_dependency_sync();
    if (threadIdx.x == 0) atomicExch(p.status, DEV_SMEM_ALIGN);
    return;
  }
  using C = AttnCfg<D>;
  constexpr int S_BUFS = C::S_BUFS, O_BUFS = C::O_BUFS, Q_BUFS = C::Q_BUFS;
  constexpr int K_STAGES = C::K_STAGES, V_STAGES = C::V_STAGES;
  static_assert(Q_BUFS <= 2 && K_STAGES <= 4 && V_STAGES <= 4 && S_BUFS <= 4, "barrier slots");
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  // Every tcgen05.commit costs the issuing thread 100 to 180 cycles, and that thread is the
  // busiest of the CTA, so each MMA group signals ONE barrier and everybody who depends on it
  // waits there: bar_s (S of a step done) tells the softmax warps that the scores are in TMEM
  // and, with the early K release, the producer that the K stage is free (K_STAGES == S_BUFS, so
  // stage and score tile share their index); bar_done (P V of a step done) serves the output
  // read-out, the rescale, the V stage and, without the early release, the K stage.  bar_done
  // is a ring of DONE_RING barriers indexed by the step: the producer, which waits for the step
  // K_STAGES back before it loads the tiles of the next one, is the last to look at a step, and
  // no P V can run more than one step beyond what the producer has loaded, so a phase is
  // always looked at before its barrier comes round (DONE_RING > K_STAGES + 1).
  uint64_t* bar_q = bars;             // [Q_BUFS] Q buffer landed
  uint64_t* bar_qfree = bars + 2;     // [Q_BUFS] last S of the unit that used the Q buffer is done
  uint64_t* bar_k = bars + 4;         // [K_STAGES] K tile landed
  uint64_t* bar_v = bars + 8;         // [V_STAGES] V tile landed
  uint64_t* bar_s = bars + 12;        // [S_BUFS] score tile holds the scores of its step
  uint64_t* bar_p = bars + 16;        // [S_BUFS] P written over the scores of the step (one arrival per warp)
  uint64_t* bar_done = bars + 20;     // [DONE_RING] the P V of step g is done: slot g % DONE_RING
  constexpr uint32_t DONE_RING = 6;
  static_assert(DONE_RING > K_STAGES + 1 && DONE_RING > V_STAGES + 1, "done ring");
  static_assert(!C::K_EARLY || K_STAGES == S_BUFS, "the early K release shares bar_s with the score tile");
  auto done_bar = [&](uint32_t step) { return &bar_done[step % DONE_RING]; };
  auto done_parity = [](uint32_t step) { return (step / DONE_RING) & 1u; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 32);
  constexpr uint32_t TMEM_COLS = C::TMEM_COLS;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int total = p.n_work * p.n_heads;  // work units: (sequence, query tile) x head

  if (threadIdx.x == 0) {
    for (int i = 0; i < Q_BUFS; ++i) {
      ptx::mbar_init(&bar_q[i], 1);
      ptx::mbar_init(&bar_qfree[i], 1);
    }
    for (int i = 0; i < S_BUFS; ++i) {
      ptx::mbar_init(&bar_s[i], 1);
      ptx::mbar_init(&bar_p[i], 4);
    }
    for (int i = 0; i < K_STAGES; ++i) ptx::mbar_init(&bar_k[i], 1);
    for (int i = 0; i < V_STAGES; ++i) ptx::mbar_init(&bar_v[i], 1);
    for (uint32_t i = 0; i < DONE_RING; ++i) ptx::mbar_init(&bar_done[i], 1);
    ptx::fence_mbar_init();
  }
  if (warp == 4) {
    ptx::tmem_alloc(tmem_slot, TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  // Barriers and TMEM are set up; from here on the kernel touches what its predecessor wrote.
  ptx::grid_dependency_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  // Score tiles: S_BUFS x 64 columns from column 0; output tiles behind them.  With two output
  // tiles (D = 64) units alternate, so that a finished unit's rows can be read out while the
  // next unit is already running.
  const uint32_t tmem_o0 = tmem_base + S_BUFS * BKV;
  const int group = p.n_heads / p.n_kv_heads;

  // A work item {seq_start, seq_len, q0, first key} is read from global memory once per unit, as
  // one 16-byte load, and the NEXT unit's item is already on its way while the current one runs:
  // the issuing threads are the busiest of the CTA and should not wait for a load per step.
  auto item_at = [&](int w) { return __ldg(reinterpret_cast<const int4*>(p.work) + w / p.n_heads); };
  // One past the last key any row of the query tile can see (causal = win_right 0).
  auto unit_kv_end = [&](const int4& it) {
    return p.win_right >= 0 ? min(it.y, it.z + BQ + p.win_right) : it.y;
  };
  // The CTA's n-th work unit.  Units are sorted by cost; handing them out in alternating
  // direction (0..G-1, then G-1..0, ...) keeps the sums per CTA close when the costs fall
  // steadily, as they do for causal batches.
  auto unit_at = [&](uint32_t n) {
    const int G = static_cast<int>(gridDim.x), b = static_cast<int>(blockIdx.x);
    return static_cast<int>(n) * G + ((n & 1u) ? G - 1 - b : b);
  };

  // A cursor walks the CTA's key steps in order, across unit boundaries.  Each role keeps its
  // own: steps are handed from role to role through the barriers only.
  struct Cursor {
    int w, j, n_kv;
    uint32_t n;
    int kv_end;   // one past the last key any row of the unit can see
    int4 it;      // the unit's work item
    int4 next;    // the item of the CTA's next unit, loaded a unit ahead
    // Steps of the unit: 64-key tiles from its first key (it.w; 0 unless a left window cuts the
    // early keys off) up to kv_end.  Keys of step j that any row can see (CTA-uniform):
    __device__ __forceinline__ int keys_in_tile(int step) const { return min(BKV, kv_end - it.w - step * BKV); }
  };
  auto enter_unit = [&](Cursor& c) {  // c.it holds the item of unit c.w
    if (c.w < total) {
      c.kv_end = unit_kv_end(c.it);
      c.n_kv = (c.kv_end - c.it.w + BKV - 1) / BKV;
      const int w_next = unit_at(c.n + 1);
      if (w_next < total) c.next = item_at(w_next);
    }
  };
  auto start_cursor = [&](Cursor& c) {
    c.w = static_cast<int>(blockIdx.x);
    c.j = 0;
    c.n_kv = 0;
    c.n = 0u;
    c.kv_end = 0;
    c.it = c.next = make_int4(0, 0, 0, 0);
    if (c.w < total) c.it = item_at(c.w);
    enter_unit(c);
  };
  auto advance = [&](Cursor& c) {
    if (++c.j == c.n_kv) {
      ++c.n;
      c.w = unit_at(c.n);
      c.j = 0;
      c.it = c.next;
      enter_unit(c);
    }
  };

  // The CTA is persistent: it walks the work units unit_at(0), unit_at(1), ...
  // `g` counts key steps over the CTA's whole life, `n` counts units; they drive every buffer
  // index and barrier parity in all three roles.
  if (warp == 5) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      ptx::prefetch_tmap(&tm_q);
      ptx::prefetch_tmap(&tm_k);
      ptx::prefetch_tmap(&tm_v);
      // K runs one step ahead of V: K of step t (and Q, at the first step of a unit), then V of
      // step t - 1.  K(t) only waits for the S MMA of step t - K_STAGES, V(t) for the P V of
      // step t - V_STAGES, which finishes a whole softmax later.
      Cursor ck, cv;
      start_cursor(ck);
      cv = ck;
      uint32_t gk = 0, gv = 0;
      int k_col = 0, v_col = 0;  // first column of the unit's K / V head (divisions once per unit)
      bool ok = true;
      while (cv.w < total && ok) {
        // The cursors move on only after both loads of the turn are out: at a unit boundary
        // that reads the next work item from global memory.
        const bool do_k = ck.w < total && gk <= gv + C::K_LEAD;
        if (do_k) {
          if (ck.j == 0) {
            const int head = ck.w % p.n_heads;
            k_col = (head / group) * D;
            // Q of this unit into buffer n % Q_BUFS, once the unit that used it before is past
            // its last S.
            const int qb = ck.n % Q_BUFS;
            if (ck.n >= Q_BUFS) {
              ok = ptx::mbar_wait(&bar_qfree[qb], ((ck.n / Q_BUFS) - 1) & 1);
              if (!ok) break;
            }
            ptx::mbar_expect_tx(&bar_q[qb], L::Q_BYTES);
#pragma unroll
            for (int a = 0; a < D_ATOMS; ++a) {
              ptx::tma_load_2d(smem + L::OFF_Q + qb * L::Q_BYTES + a * (BQ * ROW_BYTES), &tm_q, &bar_q[qb],
                               head * D + a * ATOM, ck.it.x + ck.it.z);
            }
          }
          const int st = gk % K_STAGES;
          if (gk >= K_STAGES) {
            // the stage held the K tile of step gk - K_STAGES: free after that step's S (early
            // release) or after its P V
            ok = C::K_EARLY ? ptx::mbar_wait(&bar_s[st], ((gk / K_STAGES) - 1) & 1)
                            : ptx::mbar_wait(done_bar(gk - K_STAGES), done_parity(gk - K_STAGES));
            if (!ok) break;
          }
          // shared release: the V tile of the step follows in the same turn on the same barrier
          ptx::mbar_expect_tx(&bar_k[st], C::K_EARLY ? L::KV_BYTES : 2 * L::KV_BYTES);
#pragma unroll
          for (int a = 0; a < D_ATOMS; ++a) {
            ptx::tma_load_2d(smem + L::OFF_K + st * L::KV_BYTES + a * (BKV * ROW_BYTES), &tm_k, &bar_k[st],
                             k_col + a * ATOM, ck.it.x + ck.it.w + ck.j * BKV);
          }
          ++gk;
        }
        const bool do_v = gv < gk && (gk > gv + C::K_LEAD || !do_k);
        if (do_v) {
          if (C::K_LEAD == 0) v_col = k_col;  // same step, same head
          else if (cv.j == 0) v_col = ((cv.w % p.n_heads) / group) * D;
          const int st = gv % V_STAGES;
          if (gv >= V_STAGES) {
            ok = ptx::mbar_wait(done_bar(gv - V_STAGES), done_parity(gv - V_STAGES));
            if (!ok) break;
          }
          uint64_t* landed = C::K_EARLY ? &bar_v[st] : &bar_k[st];
          if (C::K_EARLY) ptx::mbar_expect_tx(landed, L::KV_BYTES);
#pragma unroll
          for (int a = 0; a < D_ATOMS; ++a) {
            ptx::tma_load_2d(smem + L::OFF_V + st * L::KV_BYTES + a * (BKV * ROW_BYTES), &tm_v, landed,
                             v_col + a * ATOM, cv.it.x + cv.it.w + cv.j * BKV);
          }
          ++gv;
        }
        if (do_k) advance(ck);
        if (do_v) advance(cv);
      }
      if (!ok) atomicExch(p.status, DEV_TIMEOUT_ATTN);
    }
  } else if (warp == 4) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // P V: A = P from TMEM (row = lane, two keys per 32-bit column), B = V tile [keys][D] =
      // MN-major (D contiguous).
      constexpr uint32_t idesc_o = ptx::make_idesc_f16(ptx::DTypeFmt<T>::value, BQ, D, 0, 1);
      // Operand descriptors are built once; each MMA adds a constant to the address field
      // (units of 16 bytes; every operand sits below 256 KB, so the 14-bit field cannot carry).
      // The swizzle pattern repeats every 8 rows (sbo); for V, lbo is the distance between the
      // atoms of one key row group.
      constexpr uint64_t SWZ = D < 64 ? 4 : 2;  // SWIZZLE_64B : SWIZZLE_128B
      const uint64_t dq = ptx::make_smem_desc(ptx::smem_u32(smem + L::OFF_Q), 16, 8 * ROW_BYTES, SWZ);
      const uint64_t dk = ptx::make_smem_desc(ptx::smem_u32(smem + L::OFF_K), 16, 8 * ROW_BYTES, SWZ);
      const uint64_t dv = ptx::make_smem_desc(ptx::smem_u32(smem + L::OFF_V), BKV * ROW_BYTES, 8 * ROW_BYTES, SWZ);
      Cursor cs, cp;
      start_cursor(cs);
      cp = cs;
      uint32_t gs = 0, g = 0;  // steps whose S / P V has been issued
      uint32_t gvr = 0;        // steps whose V tile is known to have landed (own barrier only)
      uint32_t idle = 0;
      bool ok = true;
      while (cp.w < total) {
        bool progress = false;
        // S of step gs into score tile gs % S_BUFS.  The tile holds P of step gs - S_BUFS, whose
        // P V must have been issued (MMAs run in issue order): gs - S_BUFS < g.
        if (cs.w < total && gs < g + S_BUFS) {
          const int qb = cs.n % Q_BUFS;
          const bool ready = (cs.j != 0 || ptx::mbar_test_wait(&bar_q[qb], (cs.n / Q_BUFS) & 1)) &&
                             ptx::mbar_test_wait(&bar_k[gs % K_STAGES], (gs / K_STAGES) & 1);
          if (ready) {
            ptx::tc_fence_after();
            const int keys = cs.keys_in_tile(cs.j);
            // only ceil(keys / 16) * 16 columns are computed
            const uint32_t idesc_s = ptx::make_idesc_f16(ptx::DTypeFmt<T>::value, BQ, ((keys + 15) / 16) * 16, 0, 0);
            const uint64_t dqs = dq + static_cast<uint64_t>((qb * L::Q_BYTES) >> 4);
            const uint64_t dks = dk + static_cast<uint64_t>(((gs % K_STAGES) * L::KV_BYTES) >> 4);
            const uint32_t d_s = tmem_base + (gs % S_BUFS) * BKV;
#pragma unroll
            for (int k = 0; k < D / 16; ++k) {
              const uint64_t qoff = static_cast<uint64_t>(((k / 4) * (BQ * ROW_BYTES) + (k % 4) * 32) >> 4);
              const uint64_t koff = static_cast<uint64_t>(((k / 4) * (BKV * ROW_BYTES) + (k % 4) * 32) >> 4);
              ptx::umma_ss(d_s, dqs + qoff, dks + koff, idesc_s, k != 0 ? 1u : 0u);
            }
            ptx::umma_commit(&bar_s[gs % S_BUFS]);
            if (cs.j + 1 == cs.n_kv) ptx::umma_commit(&bar_qfree[qb]);  // last S of the unit
            ++gs;
            advance(cs);
            progress = true;
          }
        }
        // O (+)= P V of step g, once its P is written.
        // V's own barrier is looked at while P is still being written, not after it.
        if (C::K_EARLY && gvr == g && g < gs &&
            ptx::mbar_test_wait(&bar_v[g % V_STAGES], (g / V_STAGES) & 1)) {
          ++gvr;
        }
        if (g < gs && (!C::K_EARLY || g < gvr) &&
            ptx::mbar_test_wait(&bar_p[g % S_BUFS], (g / S_BUFS) & 1)) {
          ptx::tc_fence_after();
          const int k_steps = (cp.keys_in_tile(cp.j) + 15) / 16;
          const uint32_t tmem_o = tmem_o0 + (cp.n % O_BUFS) * D;
          const uint32_t t_p = tmem_base + (g % S_BUFS) * BKV;  // P lies over the scores of the step
          const uint64_t dvs = dv + static_cast<uint64_t>(((g % V_STAGES) * L::KV_BYTES) >> 4);
#pragma unroll
          for (int k = 0; k < BKV / 16; ++k) {
            if (k < k_steps) {
              ptx::umma_ts(tmem_o, t_p + k * 8, dvs + static_cast<uint64_t>((k * 16 * ROW_BYTES) >> 4), idesc_o,
                           (cp.j | k) != 0 ? 1u : 0u);
            }
          }
          ptx::umma_commit(done_bar(g));
          ++g;
          advance(cp);
          progress = true;
        }
        if (progress) {
          idle = 0;
        } else if (++idle > ptx::kSpinLimit) {  // bounded: nothing became ready for too long
          ok = false;
          break;
        }
      }
      // Nothing may be in flight when the CTA frees its TMEM.
      if (ok && g > 0) ok = ptx::mbar_wait(done_bar(g - 1), done_parity(g - 1));
      if (!ok) atomicExch(p.status, DEV_TIMEOUT_ATTN);
    }
  } else {
    // ------------------------------------------------------------ softmax warps
    const int r = warp * 32 + lane;           // row inside the query tile = TMEM lane
    const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
    uint32_t g = 0, n = 0;
    bool ok = true;
    // A finished unit whose output rows still sit in TMEM (deferred read-out, D = 64).
    bool pend = false;
    uint32_t pend_g = 0, pend_o = 0;
    int pend_rows = 0;
    float pend_inv = 0.f;
    T* pend_dst = nullptr;
    // Reads a finished unit's 32 output rows of this warp from TMEM, normalises them and stores
    // them.  g_last: the unit's last step (its P V must be complete).  Each thread holds one
    // row, but a store instruction should cover whole 128-byte lines: the rows are transposed
    // through this warp's own 4 KB slice of the staging tile, 64 columns at a time, and
    // written back with 8 lanes per row, or, when all 32 rows belong to the sequence, by one TMA
    // store of the slice (the tensor map knows nothing of sequence ends, so a ragged warp cannot
    // use it).  warp_dst: row 0 of the warp; rows_valid: how many of
    // the 32 rows belong to the sequence.
    auto flush = [&](uint32_t g_last, uint32_t t_o, float inv, T* warp_dst, int rows_valid) -> bool {
      if (!ptx::mbar_wait(done_bar(g_last), done_parity(g_last))) return false;
      ptx::tc_fence_after();
      uint8_t* stage = smem + L::OFF_STAGE + warp * (32 * 128);
      if constexpr (D == 32) {
        // 64-byte rows: four 16-byte chunks per row, chunk index XORed with bits 1-2 of the row;
        // written back with 4 lanes per row.
        uint32_t t[32];
        ptx::tmem_ld32(t_o, t);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int q8 = 0; q8 < 4; ++q8) {
          uint4 v;
          v.x = pack2<T>(__uint_as_float(t[q8 * 8 + 0]) * inv, __uint_as_float(t[q8 * 8 + 1]) * inv);
          v.y = pack2<T>(__uint_as_float(t[q8 * 8 + 2]) * inv, __uint_as_float(t[q8 * 8 + 3]) * inv);
          v.z = pack2<T>(__uint_as_float(t[q8 * 8 + 4]) * inv, __uint_as_float(t[q8 * 8 + 5]) * inv);
          v.w = pack2<T>(__uint_as_float(t[q8 * 8 + 6]) * inv, __uint_as_float(t[q8 * 8 + 7]) * inv);
          *reinterpret_cast<uint4*>(stage + lane * 64 + ((q8 ^ ((lane >> 1) & 3)) * 16)) = v;
        }
        __syncwarp();
        const int sub = lane >> 2, ch = lane & 3;
#pragma unroll
        for (int i8 = 0; i8 < 4; ++i8) {
          const int row = i8 * 8 + sub;
          const uint4 v = *reinterpret_cast<const uint4*>(stage + row * 64 + ((ch ^ ((row >> 1) & 3)) * 16));
          if (row < rows_valid) {
            *reinterpret_cast<uint4*>(warp_dst + static_cast<size_t>(row) * p.ld_o + ch * 8) = v;
          }
        }
        __syncwarp();
      } else {
        // A warp whose 32 rows all belong to the sequence hands its staged rows to one TMA store.
        const bool use_tma = rows_valid == 32;
        const size_t off = static_cast<size_t>(warp_dst - reinterpret_cast<T*>(p.out));
        const int row0 = static_cast<int>(off / p.ld_o), col0 = static_cast<int>(off % p.ld_o);
#pragma unroll
        for (int c2 = 0; c2 < D / 64; ++c2) {
          // the staging slice may still be read by the store of the piece (or unit) before
          if (lane == 0) ptx::tma_store_wait_read<0>();
          __syncwarp();
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t t[32];
            ptx::tmem_ld32(t_o + c2 * 64 + h * 32, t);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int q8 = 0; q8 < 4; ++q8) {
              uint4 v;
              v.x = pack2<T>(__uint_as_float(t[q8 * 8 + 0]) * inv, __uint_as_float(t[q8 * 8 + 1]) * inv);
              v.y = pack2<T>(__uint_as_float(t[q8 * 8 + 2]) * inv, __uint_as_float(t[q8 * 8 + 3]) * inv);
              v.z = pack2<T>(__uint_as_float(t[q8 * 8 + 4]) * inv, __uint_as_float(t[q8 * 8 + 5]) * inv);
              v.w = pack2<T>(__uint_as_float(t[q8 * 8 + 6]) * inv, __uint_as_float(t[q8 * 8 + 7]) * inv);
              // 16-byte chunk index XORed with (row & 7): conflict-free both ways
              *reinterpret_cast<uint4*>(stage + lane * 128 + (((h * 4 + q8) ^ (lane & 7)) * 16)) = v;
            }
          }
          if (use_tma) {
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              ptx::tma_store_2d(&tm_o, stage, col0 + c2 * 64, row0);
              ptx::tma_store_commit();
            }
          } else {
            __syncwarp();
            const int sub = lane >> 3, ch = lane & 7;
#pragma unroll
            for (int i4 = 0; i4 < 8; ++i4) {
              const int row = i4 * 4 + sub;
              const uint4 v = *reinterpret_cast<const uint4*>(stage + row * 128 + ((ch ^ (row & 7)) * 16));
              if (row < rows_valid) {
                *reinterpret_cast<uint4*>(warp_dst + static_cast<size_t>(row) * p.ld_o + c2 * 64 + ch * 8) = v;
              }
            }
          }
          __syncwarp();
        }
      }
      ptx::tc_fence_before();
      return true;
    };
    for (int w = unit_at(n); w < total && ok; w = unit_at(++n)) {
      const int4 it = item_at(w);
      const int head = w % p.n_heads;
      const uint32_t tmem_o = tmem_o0 + (n % O_BUFS) * D;
      const int seq_start = it.x, seq_len = it.y, q0 = it.z;
      const int kv_begin = it.w;
      const int kv_end = unit_kv_end(it);
      const int n_kv = (kv_end - kv_begin + BKV - 1) / BKV;
      const int qi = q0 + r;                  // position inside the sequence
      const float slope = ALIBI ? p.alibi_slopes[head] * 1.4426950408889634f : 0.f;
      float m = -INFINITY, l = 0.f;           // running maximum (scaled log2 domain) and sum
      for (int j = 0; j < n_kv; ++j, ++g) {
        const int b = g % S_BUFS;
        if (!ptx::mbar_wait(&bar_s[b], (g / S_BUFS) & 1)) {
          ok = false;
          break;
        }
        ptx::tc_fence_after();
        const int k_base = kv_begin + j * BKV;
        // Keys this row may attend to within the tile: [lo, lim).
        int lim = seq_len - k_base;
        if (p.win_right >= 0) lim = min(lim, qi - k_base + p.win_right + 1);
        lim = max(0, min(lim, BKV));
        const int lo = p.win_left >= 0 ? max(0, qi - p.win_left - k_base) : 0;
        // Columns beyond the tile's last key are neither computed by the S MMA nor read by
        // the P V MMA: only ceil(keys / 32) chunks of 32 columns are processed.
        const int n_chunks = (min(BKV, kv_end - k_base) + 31) / 32;
        // Uniform per (CTA, step): interior tiles need no per-element mask.
        const bool tile_full = (k_base + BKV <= seq_len) &&
                               (p.win_right < 0 || k_base + BKV <= q0 + p.win_right + 1) &&
                               (p.win_left < 0 || q0 + BQ - 1 - p.win_left <= k_base);
        const uint32_t t_s = tmem_base + b * BKV + lane_off;
        const int rel = qi - k_base;
        // The score row of this step: one TMEM read, one wait.
        uint32_t sc[BKV / 32][32];
#pragma unroll
        for (int c = 0; c < BKV / 32; ++c) {
          if (c < n_chunks) ptx::tmem_ld32(t_s + c * 32, sc[c]);
        }
        ptx::tmem_ld_wait();
        auto true_max = [&]() {
          if constexpr (ALIBI) {
            return row_max<true, true>(sc, lo, lim, n_chunks, p.scale_log2, slope, rel);
          } else {
            if (tile_full) return row_max<false, false>(sc, lo, lim, n_chunks, p.scale_log2, 0.f, 0);
            return row_max<true, false>(sc, lo, lim, n_chunks, p.scale_log2, 0.f, 0);
          }
        };
        auto probs = [&](float m_use) {
          if constexpr (ALIBI) {
            return write_probs<T, true, true>(sc, t_s, lo, lim, n_chunks, p.scale_log2, slope, rel, m_use);
          } else {
            if (tile_full) return write_probs<T, false, false>(sc, t_s, lo, lim, n_chunks, p.scale_log2, 0.f, 0, m_use);
            return write_probs<T, true, false>(sc, t_s, lo, lim, n_chunks, p.scale_log2, 0.f, 0, m_use);
          }
        };
        // P goes over this step's scores.  Their columns were last read by the P V of step
        // g-2, which ran before the S MMA of this step wrote them (MMAs run in issue order).
        // The two-pass form has ONE call site (warp-uniform flag): the unrolled passes are long,
        // and the instruction footprint of the step is what the warps wait for most.
        float sum = 0.f;
        bool two_pass = j == 0;
        if (j == 0) {
          // P V of the first step overwrites the output tile: nothing to rescale
          m = true_max();
        } else {
          // Later steps first try the maximum the row already has: one pass, no dependency of
          // the exponentials on a maximum of this step.
          // A row that has not seen a key yet (left window: its keys start in a later tile) has
          // no maximum to be lazy about: its warp goes straight to the true maxima.  Without a
          // left window every row sees a key in the unit's first tile.
          bool unseen = false;
          if constexpr (LWIN) unseen = __any_sync(0xffffffffu, m == -INFINITY);
          bool grow = false;
          if (!unseen) {
            sum = probs(m);
            grow = !(sum <= kLazySumBound);  // also true for inf and NaN
          }
          if (unseen || __any_sync(0xffffffffu, grow)) {
            // Raise the maximum of the rows that need it and rescale their partial outputs in
            // TMEM (warp-wide tcgen05.ld / st; rows that keep their maximum scale by 1).  Every
            // P V issued so far must be complete; the next one is only issued after this
            // warp's arrival on bar_p below.
            if (!ptx::mbar_wait(done_bar(g - 1), done_parity(g - 1))) {
              ok = false;
              break;
            }
            ptx::tc_fence_after();
            const float mx = true_max();  // from the scores still in registers; above m + 2 where grow is set
            // without the lazy pass: raise where the maximum grew by more than 2^8 (always, for a
            // row that sees its first key)
            if (unseen) grow = mx > m + 8.0f;
            const float alpha = grow ? ex2_fast(m - mx) : 1.0f;
            if (grow) {
              l *= alpha;
              m = mx;
            }
#pragma unroll 1
            for (int c = 0; c < D / 16; ++c) {  // small pieces: the score row is live in registers
              uint32_t t[16];
              ptx::tmem_ld16(tmem_o + lane_off + c * 16, t);
              ptx::tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 16; ++i) t[i] = __float_as_uint(__uint_as_float(t[i]) * alpha);
              ptx::tmem_st16(tmem_o + lane_off + c * 16, t);
            }
            // The probabilities again, now relative to the raised maxima (the scores are still
            // in registers; rows that kept their maximum write the same values once more).
            two_pass = true;
          }
        }
        if (two_pass) sum = probs(m == -INFINITY ? 0.f : m);
        l += sum;
        // P and the rescaled O written, S read: hand over to the MMA thread.
        ptx::tmem_st_wait();
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&bar_p[b]);
        if (pend) {
          // The previous unit's rows leave TMEM now, behind this unit's first step: its last
          // P V has long finished, so nothing waits.
          pend = false;
          if (!flush(pend_g, pend_o, pend_inv, pend_dst, pend_rows)) {
            ok = false;
            break;
          }
        }
      }
      if (!ok) break;
      // Unit finished.  With two output tiles the read-out is deferred behind the next unit's
      // first step; with one it happens now (after the unit's last P V).
      {
        const float inv = l > 0.f ? 1.0f / l : 0.f;
        T* warp_dst = reinterpret_cast<T*>(p.out) +
                      static_cast<size_t>(seq_start + q0 + warp * 32) * p.ld_o + head * D;
        const int rows_valid = max(0, min(32, seq_len - q0 - warp * 32));
        if (O_BUFS == 2) {
          pend = true;
          pend_g = g - 1;
          pend_o = tmem_o + lane_off;
          pend_inv = inv;
          pend_dst = warp_dst;
          pend_rows = rows_valid;
        } else if (!flush(g - 1, tmem_o + lane_off, inv, warp_dst, rows_valid)) {
          ok = false;
          break;
        }
      }
    }
    if (ok && pend) ok = flush(pend_g, pend_o, pend_inv, pend_dst, pend_rows);
    if (lane == 0) ptx::tma_store_wait<0>();  // the stores' global writes before the CTA exits
    if (!ok && lane == 0) atomicExch(p.status, DEV_TIMEOUT_ATTN);
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <class T, int D, bool ALIBI, bool LWIN>
int launch_variant(const AttnArgs& a, cudaStream_t stream) {
  using L = AttnSmem<D>;
  const CUtensorMapDataType dt =
      a.dtype == DT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tm_q, tm_k, tm_v, tm_o;
  int rc = make_tmap_2d(&tm_q, a.q, dt, 2, static_cast<uint64_t>(a.n_heads) * D, a.total_tokens,
                        static_cast<uint64_t>(a.ld_q) * 2, L::ATOM, BQ);
  if (rc) return rc;
  rc = make_tmap_2d(&tm_k, a.k, dt, 2, static_cast<uint64_t>(a.n_kv_heads) * D, a.total_tokens,
                    static_cast<uint64_t>(a.ld_k) * 2, L::ATOM, BKV);
  if (rc) return rc;
  rc = make_tmap_2d(&tm_v, a.v, dt, 2, static_cast<uint64_t>(a.n_kv_heads) * D, a.total_tokens,
                    static_cast<uint64_t>(a.ld_v) * 2, L::ATOM, BKV);
  if (rc) return rc;
  // output rows: boxes of 32 rows x 64 columns (the D = 32 variant stores by hand and never uses it)
  rc = make_tmap_2d(&tm_o, a.out, dt, 2, static_cast<uint64_t>(a.n_heads) * D, a.total_tokens,
                    static_cast<uint64_t>(a.ld_o) * 2, 64 <= D ? 64 : D, 32);
  if (rc) return rc;
  // The opt-in shared-memory size is a per-device function attribute; setting it twice is
  // harmless, so replicas on several threads may race to set it, but not on the flag itself.
  static std::atomic<bool> attr_set[64];
  auto kern = attention_tcgen05_kernel<T, D, ALIBI, LWIN>;
  const int dev = current_device() & 63;
  if (!attr_set[dev].load(std::memory_order_acquire)) {
    cudaError_t e =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set[dev].store(true, std::memory_order_release);
  }
  AttnParams p;
  p.out = a.out;
  p.work = a.work_items;
  p.n_work = a.n_work;
  p.n_heads = a.n_heads;
  p.n_kv_heads = a.n_kv_heads;
  p.ld_o = a.ld_o;
  // causal is a right window of 0 (backends/candle/src/flash_attn.rs:72-78)
  p.win_left = a.window_left;
  p.win_right = a.causal ? 0 : a.window_right;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.alibi_slopes = a.alibi_slopes;
  p.status = a.status;
  const long long total = static_cast<long long>(a.n_work) * a.n_heads;
  if (total > 0x7fffffffLL) return static_cast<int>(cudaErrorInvalidValue);
  const long long resident = static_cast<long long>(num_sms()) * AttnCfg<D>::CTAS_PER_SM;
  const long long grid = total < resident ? total : resident;
  return static_cast<int>(launch_dependent(kern, dim3(static_cast<unsigned>(grid)), dim3(ATTN_THREADS), L::TOTAL, stream,
                                           tm_q, tm_k, tm_v, tm_o, p));
}

template <class T, int D>
int launch_typed(const AttnArgs& a, cudaStream_t stream) {
  if (a.window_left >= 0) {
    return a.alibi_slopes ? launch_variant<T, D, true, true>(a, stream) : launch_variant<T, D, false, true>(a, stream);
  }
  return a.alibi_slopes ? launch_variant<T, D, true, false>(a, stream) : launch_variant<T, D, false, false>(a, stream);
}

}  // namespace

int launch_attention(const AttnArgs& a, cudaStream_t stream) {
  // The kernel reports a wait that ran out through *status: without it there is nowhere to write.
  if (a.status == nullptr) return static_cast<int>(cudaErrorInvalidValue);
  if (a.n_work <= 0 || a.total_tokens <= 0) return 0;
  if (a.n_kv_heads <= 0 || a.n_heads % a.n_kv_heads != 0) {
    return static_cast<int>(cudaErrorInvalidValue);
  }
  if (a.ld_q % 8 || a.ld_k % 8 || a.ld_v % 8 || a.ld_o % 8) {
    return static_cast<int>(cudaErrorInvalidValue);
  }
  if (a.head_dim == 32) {
    return a.dtype == DT_F16 ? launch_typed<__half, 32>(a, stream)
                             : launch_typed<__nv_bfloat16, 32>(a, stream);
  }
  if (a.head_dim == 64) {
    return a.dtype == DT_F16 ? launch_typed<__half, 64>(a, stream)
                             : launch_typed<__nv_bfloat16, 64>(a, stream);
  }
  if (a.head_dim == 128) {
    return a.dtype == DT_F16 ? launch_typed<__half, 128>(a, stream)
                             : launch_typed<__nv_bfloat16, 128>(a, stream);
  }
  return static_cast<int>(cudaErrorInvalidValue);
}

}  // namespace tei
