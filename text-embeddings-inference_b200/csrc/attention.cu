// Variable-length (unpadded) attention on tcgen05 tensor cores.
//
// Replaces the reference's flash_attn_varlen call (backends/candle/src/flash_attn.rs:23-120;
// call sites models/flash_bert.rs:95-108, flash_nomic.rs:83-96, flash_qwen3.rs:155-169):
// for every sequence s of the packed batch and head h,
//     out = softmax(scale * Q_s K_s^T  [- slope_h * |i - j|]  [causal mask]) V_s
// with q-head h reading kv-head h / (n_heads / n_kv_heads).  Q, K and V are strided views of
// the projection output (token-major rows), exactly as the reference passes them.
//
// Persistent CTAs (two per SM for D = 64) walk the (sequence, 128-row query tile, head) work
// units, most expensive first; the next unit's Q and first K/V tile are fetched while the
// current one finishes.  Within a CTA:
//   warp 4 (one elected lane)  TMA loads (Q once, K/V double-buffered, 128-byte swizzle, no
//                              cluster multicast) and tcgen05.mma issue:
//                              S = Q K^T into TMEM columns [0,128), P V into columns [128,128+D).
//   warps 0-3 (one row each)   read S from TMEM, online softmax in fp32 registers, write P as
//                              fp16/bf16 into shared memory in the K-major swizzled operand
//                              layout.  P V accumulates in TMEM across the key tiles; the
//                              running maximum is raised lazily (only when it grows by more
//                              than 2^8), in which case the rows rescale their partial output
//                              in TMEM.  At the end the row is read, normalised and stored.
// Two CTAs fit on an SM (D = 64), so one CTA's softmax overlaps the other's MMAs.
// Every mbarrier wait is bounded and reports through *status instead of spinning forever.
#include "kernels.h"
#include "ptx.cuh"
#include "tmap.h"


namespace tei {
namespace {

constexpr int BQ = 128;   // query rows per CTA
constexpr int BKV = 128;  // keys per inner step
constexpr int ATTN_THREADS = 160;

template <int D>
struct AttnSmem {
  static constexpr int Q_BYTES = BQ * D * 2;
  static constexpr int KV_BYTES = BKV * D * 2;
  static constexpr int P_BYTES = BQ * BKV * 2;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + Q_BYTES;          // 2 stages
  static constexpr int OFF_V = OFF_K + 2 * KV_BYTES;     // 2 stages
  static constexpr int OFF_P = OFF_V + 2 * KV_BYTES;
  static constexpr int OFF_BAR = OFF_P + P_BYTES;
  // No alignment slack: two CTAs of the D = 64 variant must fit in one SM's shared memory.  The
  // kernel checks that the dynamic window is 1024-byte aligned and reports an error otherwise.
  static constexpr int TOTAL = OFF_BAR + 128;
};

struct AttnParams {
  void* out;
  const int* work;  // [n_work][4] = {seq_start, seq_len, q0, unused}
  int n_work;
  int n_heads, n_kv_heads;
  int ld_o;
  int causal;
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

template <class T>
__device__ __forceinline__ float2 unpack2(uint32_t v);
template <>
__device__ __forceinline__ float2 unpack2<__half>(uint32_t v) {
  return __half22float2(*reinterpret_cast<const __half2*>(&v));
}
template <>
__device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t v) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v));
}

__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// One thread owns one query row of the 128-key score tile that sits in TMEM at `tmem_row`.
// Only the first n_chunks * 32 columns are touched.  MASKED: only keys [0, lim) count.
// ALIBI: subtract slope * |rel - key| (rel = query position - first key position of the tile).
// Two passes over TMEM keep the register footprint at one 32-column chunk (keeping the whole
// row in registers was measured slower: it costs occupancy-critical registers).
//
// Pass 1: row maximum in the scaled log2 domain (-inf when the row sees no key).
template <bool MASKED, bool ALIBI>
__device__ __forceinline__ float row_max(uint32_t tmem_row, int lim, int n_chunks, float sl2, float slope,
                                         int rel) {
  float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll 1
  for (int c = 0; c < n_chunks; ++c) {
    uint32_t s[32];
    ptx::tmem_ld32(tmem_row + c * 32, s);
    ptx::tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
      float x0 = __uint_as_float(s[i]), x1 = __uint_as_float(s[i + 1]);
      float x2 = __uint_as_float(s[i + 2]), x3 = __uint_as_float(s[i + 3]);
      const int kk = c * 32 + i;
      if (ALIBI) {
        x0 = x0 * sl2 - slope * fabsf(static_cast<float>(rel - kk));
        x1 = x1 * sl2 - slope * fabsf(static_cast<float>(rel - kk - 1));
        x2 = x2 * sl2 - slope * fabsf(static_cast<float>(rel - kk - 2));
        x3 = x3 * sl2 - slope * fabsf(static_cast<float>(rel - kk - 3));
      }
      if (MASKED) {
        x0 = kk < lim ? x0 : -INFINITY;
        x1 = kk + 1 < lim ? x1 : -INFINITY;
        x2 = kk + 2 < lim ? x2 : -INFINITY;
        x3 = kk + 3 < lim ? x3 : -INFINITY;
      }
      mx0 = fmaxf(mx0, x0);
      mx1 = fmaxf(mx1, x1);
      mx2 = fmaxf(mx2, x2);
      mx3 = fmaxf(mx3, x3);
    }
  }
  const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
  return ALIBI ? mx : mx * sl2;  // the scale is positive, so the maximum commutes with it
}

// Pass 2: p = 2^(score - m_use), written as T into the K-major 128-byte-swizzled operand tile
// `sp` ([k atom of 64][row][64], 16-byte chunk index XORed with (row & 7)); returns the row sum.
template <class T, bool MASKED, bool ALIBI>
__device__ __forceinline__ float write_probs(uint32_t tmem_row, uint8_t* sp, int r, int lim, int n_chunks,
                                             float sl2, float slope, int rel, float m_use) {
  float sum0 = 0.f, sum1 = 0.f;
#pragma unroll 1
  for (int c = 0; c < n_chunks; ++c) {
    uint32_t s[32];
    ptx::tmem_ld32(tmem_row + c * 32, s);
    ptx::tmem_ld_wait();
    uint32_t pk[16];
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      const int kk = c * 32 + i;
      float e0, e1;
      if (ALIBI) {
        e0 = ex2_fast(__uint_as_float(s[i]) * sl2 - slope * fabsf(static_cast<float>(rel - kk)) - m_use);
        e1 = ex2_fast(__uint_as_float(s[i + 1]) * sl2 - slope * fabsf(static_cast<float>(rel - kk - 1)) - m_use);
      } else {
        e0 = ex2_fast(fmaf(__uint_as_float(s[i]), sl2, -m_use));
        e1 = ex2_fast(fmaf(__uint_as_float(s[i + 1]), sl2, -m_use));
      }
      if (MASKED) {
        e0 = kk < lim ? e0 : 0.f;
        e1 = kk + 1 < lim ? e1 : 0.f;
      }
      sum0 += e0;
      sum1 += e1;
      pk[i / 2] = pack2<T>(e0, e1);
    }
    uint8_t* rowp = sp + (c >> 1) * (BQ * 128) + r * 128;
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) {
      const int chunk = ((c & 1) * 4 + q4) ^ (r & 7);
      *reinterpret_cast<uint4*>(rowp + chunk * 16) =
          make_uint4(pk[q4 * 4 + 0], pk[q4 * 4 + 1], pk[q4 * 4 + 2], pk[q4 * 4 + 3]);
    }
  }
  return sum0 + sum1;
}

// The running maximum is only raised when it grows by more than this many powers of two; until
// then probabilities are taken relative to the stale maximum (they stay below 2^8, far inside
// fp16 / bf16 range) and the accumulator in TMEM needs no rescaling.
constexpr float kRescaleThreshold = 8.0f;

template <class T, int D>
__global__ void __launch_bounds__(ATTN_THREADS, (D == 64 ? 2 : 1))
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_q,
                         const __grid_constant__ CUtensorMap tm_k,
                         const __grid_constant__ CUtensorMap tm_v, const AttnParams p) {
  using L = AttnSmem<D>;
  constexpr int D_ATOMS = D / 64;  // 64-element (128-byte) swizzle atoms per head
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if (ptx::smem_u32(smem) & 1023u) {  // swizzled operand tiles need 1024-byte alignment
    if (threadIdx.x == 0) atomicExch(p.status, DEV_SMEM_ALIGN);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* bar_q = bars;          // Q tile landed
  uint64_t* bar_kv = bars + 1;     // [2] K/V stage landed
  uint64_t* bar_s = bars + 3;      // S = Q K^T finished
  uint64_t* bar_p = bars + 4;      // P written (one arrival per softmax warp)
  uint64_t* bar_o = bars + 5;      // P V finished
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6);
  constexpr uint32_t TMEM_COLS = 256;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int total = p.n_work * p.n_heads;  // work units: (sequence, query tile) x head

  if (threadIdx.x == 0) {
    ptx::mbar_init(bar_q, 1);
    ptx::mbar_init(&bar_kv[0], 1);
    ptx::mbar_init(&bar_kv[1], 1);
    ptx::mbar_init(bar_s, 1);
    ptx::mbar_init(bar_p, 4);  // one arrival per softmax warp
    ptx::mbar_init(bar_o, 1);
    ptx::fence_mbar_init();
  }
  if (warp == 4) {
    ptx::tmem_alloc(tmem_slot, TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  const uint32_t tmem_s = tmem_base;
  const uint32_t tmem_o = tmem_base + 128;
  const int group = p.n_heads / p.n_kv_heads;

  // The CTA is persistent: it walks the work units blockIdx.x, blockIdx.x + gridDim.x, ...
  // `g` counts key/value steps over the CTA's whole life and drives every barrier parity.
  if (warp == 4) {
    if (lane == 0) {
      ptx::prefetch_tmap(&tm_q);
      ptx::prefetch_tmap(&tm_k);
      ptx::prefetch_tmap(&tm_v);
      // P V: A = P (K-major), B = V tile [keys][D] = MN-major (D contiguous).
      constexpr uint32_t idesc_o = ptx::make_idesc_f16(ptx::DTypeFmt<T>::value, BQ, D, 0, 1);
      auto load_q = [&](int w) {
        const int* it = p.work + (w / p.n_heads) * 4;
        const int head = w % p.n_heads;
        ptx::mbar_expect_tx(bar_q, L::Q_BYTES);
#pragma unroll
        for (int a = 0; a < D_ATOMS; ++a) {
          ptx::tma_load_2d(smem + L::OFF_Q + a * (BQ * 128), &tm_q, bar_q, head * D + a * 64, it[0] + it[2]);
        }
      };
      auto load_kv = [&](int w, int j, uint32_t step) {
        const int* it = p.work + (w / p.n_heads) * 4;
        const int kv_head = (w % p.n_heads) / group;
        const int st = step & 1;
        ptx::mbar_expect_tx(&bar_kv[st], 2 * L::KV_BYTES);
#pragma unroll
        for (int a = 0; a < D_ATOMS; ++a) {
          ptx::tma_load_2d(smem + L::OFF_K + st * L::KV_BYTES + a * (BKV * 128), &tm_k, &bar_kv[st],
                           kv_head * D + a * 64, it[0] + j * BKV);
          ptx::tma_load_2d(smem + L::OFF_V + st * L::KV_BYTES + a * (BKV * 128), &tm_v, &bar_kv[st],
                           kv_head * D + a * 64, it[0] + j * BKV);
        }
      };
      // Number of keys of step j of a unit that any row can see (CTA-uniform).
      auto keys_in_tile = [&](const int* it, int j) {
        const int kv_end = p.causal ? min(it[1], it[2] + BQ) : it[1];
        return min(BKV, kv_end - j * BKV);
      };
      // Operand descriptors are built once; each MMA adds a constant to the address field
      // (units of 16 bytes; every operand sits below 256 KB, so the 14-bit field cannot carry).
      const uint64_t dq = ptx::make_smem_desc_sw128(ptx::smem_u32(smem + L::OFF_Q), 16, 1024);
      const uint64_t dk = ptx::make_smem_desc_sw128(ptx::smem_u32(smem + L::OFF_K), 16, 1024);
      const uint64_t dp = ptx::make_smem_desc_sw128(ptx::smem_u32(smem + L::OFF_P), 16, 1024);
      const uint64_t dv = ptx::make_smem_desc_sw128(ptx::smem_u32(smem + L::OFF_V), BKV * 128, 1024);
      // S = Q K^T for the K tile in stage `st`; only the first ceil(keys/32)*32 columns are
      // computed (the softmax reads no more than that).
      auto issue_s = [&](int st, int keys) {
        const uint32_t idesc_s = ptx::make_idesc_f16(ptx::DTypeFmt<T>::value, BQ, ((keys + 31) / 32) * 32, 0, 0);
        const uint64_t dks = dk + static_cast<uint64_t>((st * L::KV_BYTES) >> 4);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          constexpr int kAtom = BQ * 128;
          const uint64_t off = static_cast<uint64_t>(((k / 4) * kAtom + (k % 4) * 32) >> 4);
          ptx::umma_ss(tmem_s, dq + off, dks + off, idesc_s, k != 0 ? 1u : 0u);
        }
        ptx::umma_commit(bar_s);
      };
      // O (+)= P V over the first k_steps * 16 keys of the tile in stage `st`.
      auto issue_pv = [&](int st, int k_steps, bool accumulate) {
        const uint64_t dvs = dv + static_cast<uint64_t>((st * L::KV_BYTES) >> 4);
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k) {
          if (k < k_steps) {
            constexpr int kAtom = BQ * 128;
            const uint64_t aoff = static_cast<uint64_t>(((k / 4) * kAtom + (k % 4) * 32) >> 4);
            ptx::umma_ss(tmem_o, dp + aoff, dvs + static_cast<uint64_t>((k * 2048) >> 4), idesc_o,
                         (accumulate || k != 0) ? 1u : 0u);
          }
        }
        ptx::umma_commit(bar_o);
      };
      uint32_t g = 0, n_item = 0;
      bool ok = true;
      if (static_cast<int>(blockIdx.x) < total) {
        load_q(blockIdx.x);
        load_kv(blockIdx.x, 0, 0);
        ok = ptx::mbar_wait(bar_q, 0) && ptx::mbar_wait(&bar_kv[0], 0);
        if (ok) {
          ptx::tc_fence_after();
          issue_s(0, keys_in_tile(p.work + (blockIdx.x / p.n_heads) * 4, 0));
        }
      }
      // Invariant at the top of every step g: S of step g has been issued.  Each step then
      // (1) waits for the previous step's P V (its K/V stage becomes free) and starts the loads
      // of the next step, (2) waits for P, (3) issues the NEXT step's S and, behind it, this
      // step's P V, which accumulates into the output tile in TMEM.
      for (int w = blockIdx.x; w < total && ok; w += gridDim.x, ++n_item) {
        const int* it = p.work + (w / p.n_heads) * 4;
        const int seq_len = it[1], q0 = it[2];
        const int kv_end = p.causal ? min(seq_len, q0 + BQ) : seq_len;
        const int n_kv = (kv_end + BKV - 1) / BKV;
        const int w_next = w + static_cast<int>(gridDim.x);
        for (int j = 0; j < n_kv && ok; ++j, ++g) {
          const int st = g & 1;
          const bool last = (j + 1 == n_kv);
          if (g > 0) {
            ok = ptx::mbar_wait_spin(bar_o, (g - 1) & 1);
            if (!ok) break;
          }
          if (!last) {
            load_kv(w, j + 1, g + 1);
          } else if (w_next < total) {
            // Last step of this unit: once its S is done nothing reads the Q tile any more.
            ok = ptx::mbar_wait(bar_s, g & 1);
            if (!ok) break;
            load_q(w_next);
            load_kv(w_next, 0, g + 1);
          }
          ok = ptx::mbar_wait_spin(bar_p, g & 1);
          if (!ok) break;
          ptx::tc_fence_after();
          // Next step's S first: the softmax warps can start on it while P V runs.
          if (!last) {
            ok = ptx::mbar_wait(&bar_kv[(g + 1) & 1], ((g + 1) >> 1) & 1);
            if (!ok) break;
            ptx::tc_fence_after();
            issue_s((g + 1) & 1, keys_in_tile(it, j + 1));
          } else if (w_next < total) {
            ok = ptx::mbar_wait(bar_q, (n_item + 1) & 1);
            ok = ok && ptx::mbar_wait(&bar_kv[(g + 1) & 1], ((g + 1) >> 1) & 1);
            if (!ok) break;
            ptx::tc_fence_after();
            issue_s((g + 1) & 1, keys_in_tile(p.work + (w_next / p.n_heads) * 4, 0));
          }
          // O (+)= P_j V_j over the keys of this tile (rounded up to the MMA's K step of 16).
          issue_pv(st, (keys_in_tile(it, j) + 15) / 16, j != 0);
        }
      }
      if (ok && g > 0) ok = ptx::mbar_wait_spin(bar_o, (g - 1) & 1);
      if (!ok) atomicExch(p.status, DEV_TIMEOUT_ATTN);
    }
  } else {
    // ------------------------------------------------------------ softmax warps
    const int r = warp * 32 + lane;           // row inside the query tile = TMEM lane
    const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
    uint8_t* sp = smem + L::OFF_P;
    uint32_t g = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
      const int* it = p.work + (w / p.n_heads) * 4;
      const int head = w % p.n_heads;
      const int seq_start = it[0], seq_len = it[1], q0 = it[2];
      const int kv_end = p.causal ? min(seq_len, q0 + BQ) : seq_len;
      const int n_kv = (kv_end + BKV - 1) / BKV;
      const int qi = q0 + r;                  // position inside the sequence
      const float slope = p.alibi_slopes ? p.alibi_slopes[head] * 1.4426950408889634f : 0.f;
      float m = -INFINITY, l = 0.f;           // running maximum (scaled log2 domain) and sum
      for (int j = 0; j < n_kv; ++j, ++g) {
        if (!ptx::mbar_wait(bar_s, g & 1)) {
          ok = false;
          break;
        }
        ptx::tc_fence_after();
        const int k_base = j * BKV;
        // Keys this row may attend to within the tile: [0, lim).
        int lim = seq_len - k_base;
        if (p.causal) lim = min(lim, qi - k_base + 1);
        lim = max(0, min(lim, BKV));
        // Columns beyond the tile's last key are neither computed by the S MMA nor read by
        // the P V MMA: only ceil(keys / 32) chunks of 32 columns are processed.
        const int n_chunks = (min(BKV, kv_end - k_base) + 31) / 32;
        // Uniform per (CTA, step): interior tiles need no per-element mask.
        const bool tile_full = (k_base + BKV <= seq_len) && (!p.causal || k_base + BKV <= q0 + 1);
        const uint32_t t_s = tmem_s + lane_off;
        const int rel = qi - k_base;
        float mx;
        if (p.alibi_slopes) mx = row_max<true, true>(t_s, lim, n_chunks, p.scale_log2, slope, rel);
        else if (tile_full) mx = row_max<false, false>(t_s, lim, n_chunks, p.scale_log2, 0.f, 0);
        else mx = row_max<true, false>(t_s, lim, n_chunks, p.scale_log2, 0.f, 0);
        // The previous step's P V must be complete before P is overwritten or O is touched.
        if (g > 0) {
          if (!ptx::mbar_wait(bar_o, (g - 1) & 1)) {
            ok = false;
            break;
          }
          ptx::tc_fence_after();
        }
        if (j == 0) {
          m = mx;  // P V of the first step overwrites the output tile: nothing to rescale
        } else {
          const bool grow = mx > m + kRescaleThreshold;
          if (__any_sync(0xffffffffu, grow)) {
            // Raise the maximum of the rows that need it and rescale their partial outputs in
            // TMEM (warp-wide tcgen05.ld / st; rows that keep their maximum scale by 1).
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
            ptx::tmem_st_wait();
          }
        }
        const float m_use = (m == -INFINITY) ? 0.f : m;
        float sum;
        if (p.alibi_slopes) sum = write_probs<T, true, true>(t_s, sp, r, lim, n_chunks, p.scale_log2, slope, rel, m_use);
        else if (tile_full) sum = write_probs<T, false, false>(t_s, sp, r, lim, n_chunks, p.scale_log2, 0.f, 0, m_use);
        else sum = write_probs<T, true, false>(t_s, sp, r, lim, n_chunks, p.scale_log2, 0.f, 0, m_use);
        l += sum;
        // P visible to the tensor core (async proxy), S reads and O writes finished: hand over.
        ptx::fence_proxy_async_smem();
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(bar_p);
      }
      if (!ok) break;
      // Unit finished: wait for its last P V, read the output row, normalise, store.
      if (!ptx::mbar_wait(bar_o, (g - 1) & 1)) {
        ok = false;
        break;
      }
      ptx::tc_fence_after();
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      T* dst = reinterpret_cast<T*>(p.out) + static_cast<size_t>(seq_start + qi) * p.ld_o + head * D;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t t[32];
        ptx::tmem_ld32(tmem_o + lane_off + c * 32, t);
        ptx::tmem_ld_wait();
        if (qi < seq_len) {
#pragma unroll
          for (int q8 = 0; q8 < 4; ++q8) {
            uint4 v;
            v.x = pack2<T>(__uint_as_float(t[q8 * 8 + 0]) * inv, __uint_as_float(t[q8 * 8 + 1]) * inv);
            v.y = pack2<T>(__uint_as_float(t[q8 * 8 + 2]) * inv, __uint_as_float(t[q8 * 8 + 3]) * inv);
            v.z = pack2<T>(__uint_as_float(t[q8 * 8 + 4]) * inv, __uint_as_float(t[q8 * 8 + 5]) * inv);
            v.w = pack2<T>(__uint_as_float(t[q8 * 8 + 6]) * inv, __uint_as_float(t[q8 * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + c * 32 + q8 * 8) = v;
          }
        }
      }
      ptx::tc_fence_before();
    }
    if (!ok && lane == 0) atomicExch(p.status, DEV_TIMEOUT_ATTN);
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <class T, int D>
int launch_typed(const AttnArgs& a, cudaStream_t stream) {
  using L = AttnSmem<D>;
  const CUtensorMapDataType dt =
      a.dtype == DT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tm_q, tm_k, tm_v;
  int rc = make_tmap_2d(&tm_q, a.q, dt, 2, static_cast<uint64_t>(a.n_heads) * D, a.total_tokens,
                        static_cast<uint64_t>(a.ld_q) * 2, 64, BQ);
  if (rc) return rc;
  rc = make_tmap_2d(&tm_k, a.k, dt, 2, static_cast<uint64_t>(a.n_kv_heads) * D, a.total_tokens,
                    static_cast<uint64_t>(a.ld_k) * 2, 64, BKV);
  if (rc) return rc;
  rc = make_tmap_2d(&tm_v, a.v, dt, 2, static_cast<uint64_t>(a.n_kv_heads) * D, a.total_tokens,
                    static_cast<uint64_t>(a.ld_v) * 2, 64, BKV);
  if (rc) return rc;
  static bool attr_set[64] = {};
  auto kern = attention_tcgen05_kernel<T, D>;
  const int dev = current_device() & 63;
  if (!attr_set[dev]) {
    cudaError_t e =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set[dev] = true;
  }
  AttnParams p;
  p.out = a.out;
  p.work = a.work_items;
  p.n_work = a.n_work;
  p.n_heads = a.n_heads;
  p.n_kv_heads = a.n_kv_heads;
  p.ld_o = a.ld_o;
  p.causal = a.causal;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.alibi_slopes = a.alibi_slopes;
  p.status = a.status;
  const long long total = static_cast<long long>(a.n_work) * a.n_heads;
  if (total > 0x7fffffffLL) return static_cast<int>(cudaErrorInvalidValue);
  const long long resident = static_cast<long long>(num_sms()) * (D == 64 ? 2 : 1);
  const long long grid = total < resident ? total : resident;
  kern<<<static_cast<unsigned>(grid), ATTN_THREADS, L::TOTAL, stream>>>(tm_q, tm_k, tm_v, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

int launch_attention(const AttnArgs& a, cudaStream_t stream) {
  if (a.n_work <= 0 || a.total_tokens <= 0) return 0;
  if (a.n_kv_heads <= 0 || a.n_heads % a.n_kv_heads != 0) {
    return static_cast<int>(cudaErrorInvalidValue);
  }
  if (a.ld_q % 8 || a.ld_k % 8 || a.ld_v % 8 || a.ld_o % 8) {
    return static_cast<int>(cudaErrorInvalidValue);
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
