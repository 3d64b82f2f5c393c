// Dense layer on the 5th-generation tensor cores: out = act(a @ w^T + bias) (+ residual).
//
// Replaces the cuBLASLt call behind the reference's Linear::forward
// (backends/candle/src/layers/linear.rs:51-75, layers/cublaslt.rs:49-87): same operand layout
// (activations [M,K] row-major, weights [N,K] row-major exactly as stored in safetensors), same
// fused epilogues (bias, tanh-GELU, ReLU), plus SwiGLU, tanh, log1p(relu) and a residual add that
// the reference runs as separate kernels.
//
// Structure (one CTA per SM, persistent over 128x256 output tiles):
//   warp 0      TMA producer: 128x64 A tile + 256x64 W tile per stage, 128-byte swizzle,
//               4-stage mbarrier ring.  Plain per-CTA TMA loads, no cluster multicast.
//   warp 1      allocates 512 TMEM columns (two 128x256 fp32 accumulators) and issues
//               tcgen05.mma.cta_group::1.kind::f16 (M=128, N=256, K=16), four per stage.
//   warps 2-5   epilogue: tcgen05.ld the finished accumulator (one row per thread), bias /
//               activation in registers, rows packed into a 128-byte-swizzled staging tile in
//               shared memory and written out with TMA stores (full 128-byte lines; the tensor
//               map clips the M and N tails).  Runs while the MMA warp fills the other
//               accumulator.  Outputs whose row pitch is not a multiple of 16 bytes, and the
//               residual variant, use plain per-thread stores instead.
// Every mbarrier wait is bounded; a wait that runs out writes a code to *status and the CTA
// drains and exits.
#include "kernels.h"
#include "ptx.cuh"
#include "rope_math.cuh"
#include "tmap.h"

#include <atomic>

namespace tei {
namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;  // 64 x 2 B = one 128-byte swizzle row
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;
constexpr int B_BYTES = BN * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;
// Epilogue staging: per epilogue warp two buffers of 32 rows x 64 columns (128 B per row).
constexpr int EPI_BUF_BYTES = 32 * 128;
constexpr int EPI_BYTES = 4 * 2 * EPI_BUF_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
// The single-CTA kernel also comes with 128- and 64-column tiles, for problems whose 256-column
// tiles would leave most SMs idle (a 512-token batch is 4 x 3 tiles on the N = 768 layers).
// Narrow tiles take more stages: a stage is smaller.
template <int TN>
struct SingleCfg {
  static_assert(TN == 256 || TN == 128 || TN == 64, "tile widths");
  // (a stage is in flight for about 1,750 cycles; the MMAs of a 64-column k-block take 200)
  static constexpr int N_STAGES = TN == 256 ? STAGES : (TN == 128 ? 6 : 8);
  static constexpr int B_TILE_BYTES = TN * BK * 2;
  static constexpr int STAGE = A_BYTES + B_TILE_BYTES;
  static constexpr int TMEM = 2 * TN;  // two accumulators; a power of two >= 32
  static constexpr int SMEM = N_STAGES * STAGE + EPI_BYTES + 1024 + 256;
};

struct GemmParams {
  const void* bias;
  const void* residual;
  void* out;
  int M, N, K;
  int ldo, ldr;
  int tma_store;  // 1: outputs leave through the TMA store path
  int* status;
  const int* m_dev;  // optional device-side row count (see GemmArgs::m_dev)
  RopeFusion rope;   // used by the ROPE_D != 0 instantiations only
};

// Rows the kernel works on.
__device__ __forceinline__ int effective_rows(const GemmParams& p) {
  return p.m_dev ? min(p.M, *p.m_dev) : p.M;
}

__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float gelu_tanh(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float u = k0 * (x + k1 * x * x * x);
  return 0.5f * x * (1.0f + tanh_fast(u));
}
__device__ __forceinline__ float silu(float x) { return x / (1.0f + __expf(-x)); }

template <class T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) {
  return __half2float(v);
}
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <class T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) {
  return __float2half_rn(v);
}
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

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

// Internal epilogue variant, not part of the public activation list: no activation, and the
// residual rows are added on the TMA-store path (GemmArgs::act == ACT_NONE with a residual whose
// rows are 16-byte aligned and N a multiple of 64).  Meant for projections with a long K loop,
// where the tile's main loop hides the epilogue's wait for the residual rows: the post-LN
// models' feed-forward output, whose LayerNorm then reads one tensor instead of two.
constexpr int ACT_ADD_RES = 64;

template <class T>
__device__ __forceinline__ float2 widen2(uint32_t v);
template <>
__device__ __forceinline__ float2 widen2<__half>(uint32_t v) {
  return __half22float2(*reinterpret_cast<const __half2*>(&v));
}
template <>
__device__ __forceinline__ float2 widen2<__nv_bfloat16>(uint32_t v) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v));
}

// Gate activation of the gated feed-forwards.
template <int ACT>
__device__ __forceinline__ float glu_gate(float x) {
  if constexpr (ACT == ACT_GEGLU) return gelu_tanh(x);
  return silu(x);
}

template <int ACT>
__device__ __forceinline__ float apply_act(float x) {
  if constexpr (ACT == ACT_GELU) return gelu_tanh(x);
  if constexpr (ACT == ACT_RELU) return fmaxf(x, 0.0f);
  if constexpr (ACT == ACT_TANH) return tanhf(x);
  if constexpr (ACT == ACT_RELU_LOG1P) return log1pf(fmaxf(x, 0.0f));
  return x;
}

// Activation of a packed pair of fp32 values (one instruction per two values where the
// hardware has one), rounded to two T.
template <class T, int ACT>
__device__ __forceinline__ uint32_t act_pack2(uint64_t x) {
  if constexpr (ACT == ACT_GELU) {
    // 0.5 x (1 + tanh(k0 (x + k1 x^3))) = hx + hx tanh(x (k0 + k0 k1 x^2)), hx = x / 2
    const uint64_t kk = ptx::pack_f32x2(0.7978845608028654f * 0.044715f, 0.7978845608028654f * 0.044715f);
    const uint64_t k0 = ptx::pack_f32x2(0.7978845608028654f, 0.7978845608028654f);
    const uint64_t half = ptx::pack_f32x2(0.5f, 0.5f);
    const uint64_t u = ptx::mul_f32x2(x, ptx::fma_f32x2(ptx::mul_f32x2(x, x), kk, k0));
    float u0, u1;
    ptx::unpack_f32x2(u, u0, u1);
    const uint64_t hx = ptx::mul_f32x2(x, half);
    float r0, r1;
    ptx::unpack_f32x2(ptx::fma_f32x2(hx, ptx::pack_f32x2(tanh_fast(u0), tanh_fast(u1)), hx), r0, r1);
    return pack2<T>(r0, r1);
  } else {
    float x0, x1;
    ptx::unpack_f32x2(x, x0, x1);
    return pack2<T>(apply_act<ACT>(x0), apply_act<ACT>(x1));
  }
}

// Adds bias / applies the activation / adds the residual to 32 consecutive columns of one row
// and stores them.  `col` is the first output column, n_valid the number of columns in range.
template <class T, int ACT>
__device__ __forceinline__ void finish_and_store(float (&v)[32], const GemmParams& p, int row,
                                                 int col, int n_valid, bool vec_ok) {
  T* out = reinterpret_cast<T*>(p.out) + static_cast<size_t>(row) * p.ldo + col;
  const T* res = p.residual
                     ? reinterpret_cast<const T*>(p.residual) + static_cast<size_t>(row) * p.ldr + col
                     : nullptr;
  if (vec_ok && n_valid == 32) {
    if (res) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint4 r = *reinterpret_cast<const uint4*>(res + j * 8);
        const T* rr = reinterpret_cast<const T*>(&r);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[j * 8 + e] += to_f32<T>(rr[e]);
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint4 o;
      o.x = pack2<T>(v[j * 8 + 0], v[j * 8 + 1]);
      o.y = pack2<T>(v[j * 8 + 2], v[j * 8 + 3]);
      o.z = pack2<T>(v[j * 8 + 4], v[j * 8 + 5]);
      o.w = pack2<T>(v[j * 8 + 6], v[j * 8 + 7]);
      *reinterpret_cast<uint4*>(out + j * 8) = o;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if (j < n_valid) {
        float x = v[j];
        if (res) x += to_f32<T>(res[j]);
        out[j] = from_f32<T>(x);
      }
    }
  }
}

// Epilogue of one 128 x 256 accumulator for one warp (32 rows): bias / activation / optional
// residual, then either swizzled staging + TMA store (64 columns per step) or plain per-thread
// stores.  t_row: TMEM address of the warp's lane quadrant in the accumulator; m0 / n0: first
// row / column of the tile in the output.
template <class T, int ACT, int TN = BN, class Release>
__device__ __forceinline__ void epilogue_tile(const GemmParams& p, const CUtensorMap* tm_c, uint32_t t_row,
                                              int m0, int n0, int quad, int lane, const T* bias,
                                              bool bias_vec, bool vec_ok, uint8_t* stage_buf,
                                              uint32_t& store_count, int n_out, Release&& release, int part = 0,
                                              int n_parts = 1) {  // part: this warp's share of the columns
  const int row = m0 + quad * 32 + lane;
  const int m_rows = effective_rows(p);
  if (p.tma_store) {
    // 64 output columns per step: TMEM -> registers -> swizzled staging tile -> TMA store.  The
    // steps go two at a time: both are read from the accumulator (and converted) before the first
    // is staged, and after the warp's last read the accumulator goes back to the MMA thread, so
    // the staging writes and the stores of a tile no longer hold up the tile after next.
    static_assert(TN == BN || !(ACT == ACT_SWIGLU || ACT == ACT_GEGLU), "gated tiles are 256 wide");
    constexpr int STEPS = (ACT == ACT_SWIGLU || ACT == ACT_GEGLU) ? 2 : TN / 64;
    const int o0 = (ACT == ACT_SWIGLU || ACT == ACT_GEGLU) ? n0 / 2 : n0;
    auto load_step = [&](int c, uint32_t (&packed)[32]) {
      if constexpr (ACT == ACT_SWIGLU || ACT == ACT_GEGLU) {
        // Columns [0,128) of the tile are gate rows, [128,256) the matching up rows.
#pragma unroll
        for (int hlf = 0; hlf < 2; ++hlf) {
          uint32_t g[32], u[32];
          ptx::tmem_ld32(t_row + c * 64 + hlf * 32, g);
          ptx::tmem_ld32(t_row + 128 + c * 64 + hlf * 32, u);
          ptx::tmem_ld_wait();
          const int gcol = n0 + c * 64 + hlf * 32;
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            float gv0 = __uint_as_float(g[j]), gv1 = __uint_as_float(g[j + 1]);
            float uv0 = __uint_as_float(u[j]), uv1 = __uint_as_float(u[j + 1]);
            if (bias) {
              gv0 += to_f32<T>(bias[gcol + j]);
              gv1 += to_f32<T>(bias[gcol + j + 1]);
              uv0 += to_f32<T>(bias[gcol + 128 + j]);
              uv1 += to_f32<T>(bias[gcol + 128 + j + 1]);
            }
            packed[hlf * 16 + j / 2] = pack2<T>(glu_gate<ACT>(gv0) * uv0, glu_gate<ACT>(gv1) * uv1);
          }
        }
      } else if constexpr (ACT == ACT_ADD_RES) {
        // The thread's 64 residual values (one 128-byte line) are requested first and arrive
        // while the accumulator is read.  Same arithmetic as the plain-store path: accumulator
        // + bias, + residual, one rounding.
        uint32_t rq[32];
        {
          const T* rp = reinterpret_cast<const T*>(p.residual) + static_cast<size_t>(row) * p.ldr + n0 + c * 64;
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const uint4 v = row < m_rows ? *reinterpret_cast<const uint4*>(rp + q * 8) : make_uint4(0u, 0u, 0u, 0u);
            rq[q * 4 + 0] = v.x; rq[q * 4 + 1] = v.y; rq[q * 4 + 2] = v.z; rq[q * 4 + 3] = v.w;
          }
        }
#pragma unroll
        for (int hlf = 0; hlf < 2; ++hlf) {
          uint32_t r[32];
          ptx::tmem_ld32(t_row + c * 64 + hlf * 32, r);
          ptx::tmem_ld_wait();
          const int col = n0 + c * 64 + hlf * 32;
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            uint64_t x = ptx::pack_f32x2(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
            if (bias != nullptr) x = ptx::add_f32x2(x, ptx::pack_f32x2(to_f32<T>(bias[col + j]), to_f32<T>(bias[col + j + 1])));
            const float2 rf = widen2<T>(rq[hlf * 16 + j / 2]);
            float x0, x1;
            ptx::unpack_f32x2(ptx::add_f32x2(x, ptx::pack_f32x2(rf.x, rf.y)), x0, x1);
            packed[hlf * 16 + j / 2] = pack2<T>(x0, x1);
          }
        }
      } else {
        // both halves of the step in flight before the one wait
        uint32_t rr[2][32];
        ptx::tmem_ld32(t_row + c * 64, rr[0]);
        ptx::tmem_ld32(t_row + c * 64 + 32, rr[1]);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int hlf = 0; hlf < 2; ++hlf) {
          const uint32_t (&r)[32] = rr[hlf];
          const int col = n0 + c * 64 + hlf * 32;
          if (bias == nullptr) {
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              packed[hlf * 16 + j / 2] = act_pack2<T, ACT>(ptx::pack_f32x2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])));
            }
          } else {
            float bv[32];
            if (bias_vec && col + 32 <= p.N) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const uint4 b4 = *reinterpret_cast<const uint4*>(bias + col + j * 8);
                const T* bt = reinterpret_cast<const T*>(&b4);
#pragma unroll
                for (int e = 0; e < 8; ++e) bv[j * 8 + e] = to_f32<T>(bt[e]);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) bv[j] = (col + j < p.N) ? to_f32<T>(bias[col + j]) : 0.f;
            }
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              const uint64_t x = ptx::add_f32x2(ptx::pack_f32x2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])),
                                                ptx::pack_f32x2(bv[j], bv[j + 1]));
              packed[hlf * 16 + j / 2] = act_pack2<T, ACT>(x);
            }
          }
        }
      }
    };
    auto store_step = [&](int c, const uint32_t (&packed)[32]) {
      // The staging buffer used two stores ago must have been read out by its TMA store.
      uint8_t* buf = stage_buf + (store_count & 1) * EPI_BUF_BYTES;
      if (lane == 0) ptx::tma_store_wait_read<1>();
      __syncwarp();
      // Row `lane` of the 32 x 64 tile: eight 16-byte chunks, chunk index XORed with
      // (row & 7) as the 128-byte swizzle of the tensor map expects.
      uint8_t* rowp = buf + lane * 128;
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        *reinterpret_cast<uint4*>(rowp + ((q ^ (lane & 7)) * 16)) =
            make_uint4(packed[q * 4 + 0], packed[q * 4 + 1], packed[q * 4 + 2], packed[q * 4 + 3]);
      }
      ptx::fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        // A box that starts beyond the last row has nothing to write (the tensor map would clip
        // it anyway); the empty group keeps the wait_group accounting uniform.
        if (m0 + quad * 32 < m_rows) ptx::tma_store_2d(tm_c, buf, o0 + c * 64, m0 + quad * 32);
        ptx::tma_store_commit();
      }
      ++store_count;
    };
    const int c_end = (part + 1) * (STEPS / n_parts);
    bool released = false;
#pragma unroll 1
    for (int c = part * (STEPS / n_parts); c < c_end; c += (ACT == ACT_ADD_RES ? 1 : 2)) {
      if (o0 + c * 64 >= n_out) break;  // uniform across the CTA
      // (the residual variant goes one step at a time: its main loop is long, registers are not)
      const bool second = ACT != ACT_ADD_RES && c + 1 < c_end && o0 + (c + 1) * 64 < n_out;
      uint32_t pk0[32], pk1[32];
      load_step(c, pk0);
      if (second) load_step(c + 1, pk1);
      constexpr int kStride = ACT == ACT_ADD_RES ? 1 : 2;
      if (c + kStride >= c_end || o0 + (c + kStride) * 64 >= n_out) {  // the warp's last read of this accumulator
        release();
        released = true;
      }
      store_step(c, pk0);
      if (second) store_step(c + 1, pk1);
    }
    if (!released) release();
    return;
  } else if constexpr (ACT == ACT_SWIGLU || ACT == ACT_GEGLU) {
    // Columns [0,128) of the tile are gate rows, [128,256) the matching up rows.
#pragma unroll 1
    for (int c = part * (4 / n_parts); c < (part + 1) * (4 / n_parts); ++c) {
      uint32_t g[32], u[32];
      ptx::tmem_ld32(t_row + c * 32, g);
      ptx::tmem_ld32(t_row + 128 + c * 32, u);
      ptx::tmem_ld_wait();
      float v[32];
      const int gcol = n0 + c * 32;        // column in the interleaved weight
      const int ocol = n0 / 2 + c * 32;    // output column
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        float gv = __uint_as_float(g[j]);
        float uv = __uint_as_float(u[j]);
        if (bias) {
          if (gcol + j < p.N) gv += to_f32<T>(bias[gcol + j]);
          if (gcol + 128 + j < p.N) uv += to_f32<T>(bias[gcol + 128 + j]);
        }
        v[j] = glu_gate<ACT>(gv) * uv;
      }
      const int n_valid = min(32, p.N / 2 - ocol);
      if (row < m_rows && n_valid > 0) finish_and_store<T, ACT>(v, p, row, ocol, n_valid, vec_ok);
    }
  } else {
#pragma unroll 1
    for (int c = part * (TN / 32 / n_parts); c < (part + 1) * (TN / 32 / n_parts); ++c) {
      const int col = n0 + c * 32;
      if (col >= p.N) break;  // uniform across the CTA
      uint32_t r[32];
      ptx::tmem_ld32(t_row + c * 32, r);
      ptx::tmem_ld_wait();
      float v[32];
      const int n_valid = min(32, p.N - col);
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        float x = __uint_as_float(r[j]);
        if (bias && j < n_valid) x += to_f32<T>(bias[col + j]);
        v[j] = apply_act<ACT>(x);
      }
      if (row < m_rows) finish_and_store<T, ACT>(v, p, row, col, n_valid, vec_ok);
    }
  }
  release();
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

// 32 accumulator columns of one row plus bias, rounded to T: the values the plain projection
// would have stored and the standalone RoPE kernel would have read back, two per word.
template <class T>
__device__ __forceinline__ void round32(const uint32_t (&r)[32], const T* bias, int col, int N, uint32_t (&x)[16]) {
#pragma unroll
  for (int j = 0; j < 32; j += 2) {
    float v0 = __uint_as_float(r[j]), v1 = __uint_as_float(r[j + 1]);
    if (bias) {
      // the same packed add as the plain epilogue
      ptx::unpack_f32x2(ptx::add_f32x2(ptx::pack_f32x2(v0, v1),
                                       ptx::pack_f32x2(col + j < N ? to_f32<T>(bias[col + j]) : 0.f,
                                                       col + j + 1 < N ? to_f32<T>(bias[col + j + 1]) : 0.f)),
                        v0, v1);
    }
    x[j / 2] = pack2<T>(v0, v1);
  }
}
// Two chunks with both TMEM loads in flight before the one wait.
template <class T>
__device__ __forceinline__ void rounded_pair(uint32_t ta, uint32_t tb, const T* bias, int col_a, int col_b, int N,
                                             uint32_t (&a)[16], uint32_t (&b)[16]) {
  uint32_t ra[32], rb[32];
  ptx::tmem_ld32(ta, ra);
  ptx::tmem_ld32(tb, rb);
  ptx::tmem_ld_wait();
  round32<T>(ra, bias, col_a, N, a);
  round32<T>(rb, bias, col_b, N, b);
}

// Writes 32 values (16 words) of row `lane` into 16-byte chunks chunk0 .. chunk0 + 3 of a 32 x 64
// staging tile (128-byte rows, chunk index XORed with row & 7: the tensor map's 128-byte swizzle).
__device__ __forceinline__ void stage16(uint8_t* buf, int lane, int chunk0, const uint32_t (&w)[16]) {
  uint8_t* rowp = buf + lane * 128;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    *reinterpret_cast<uint4*>(rowp + (((chunk0 + q) ^ (lane & 7)) * 16)) =
        make_uint4(w[q * 4 + 0], w[q * 4 + 1], w[q * 4 + 2], w[q * 4 + 3]);
  }
}

// cos / sin of 8 consecutive pair indices of one table row.
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p));
  const float4 b = __ldg(reinterpret_cast<const float4*>(p + 4));
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
// 8 consecutive elements held as 4 words -> fp32.
template <class T>
__device__ __forceinline__ void widen8(const uint32_t* w, float (&v)[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = unpack2<T>(w[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}
// 8 consecutive norm weights (16-byte aligned) as fp32.
template <class T>
__device__ __forceinline__ void load_gamma8(const T* p, float (&v)[8]) {
  const uint4 u = __ldg(reinterpret_cast<const uint4*>(p));
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
  widen8<T>(w, v);
}

// ropemath::ss8 on 8 + 8 elements held as words, the products taken two at a time (the same IEEE
// operations in the same order: only the additions into ss are sequential).
template <class T>
__device__ __forceinline__ float ss8_words(const uint32_t* aw, const uint32_t* bw) {
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 fa = unpack2<T>(aw[i]), fb = unpack2<T>(bw[i]);
    const uint64_t a2 = ptx::pack_f32x2(fa.x, fa.y), b2 = ptx::pack_f32x2(fb.x, fb.y);
    float t0, t1;
    ptx::unpack_f32x2(ptx::fma_f32x2(a2, a2, ptx::mul_f32x2(b2, b2)), t0, t1);
    ss = __fadd_rn(ss, t0);
    ss = __fadd_rn(ss, t1);
  }
  return ss;
}

// NP pairs (a[i], b[i]) = (x[j0 + i], x[j0 + i + D/2]) of one head, held as NP/2 words each:
// optional RMSNorm scale r with the gammas of both halves, then the rotation with the table
// entries j0 .. j0 + NP - 1, rounded back to T in place.  Two pairs per instruction; operation
// for operation ropemath::normed / rot_lo / rot_hi (-(b s) and b (-s) are the same number).
template <class T, int NP>
__device__ __forceinline__ void norm_rotate(uint32_t* aw, uint32_t* bw, bool norm, float r, const T* gamma, int j0,
                                            int half, const float* cos_row, const float* sin_row) {
  const uint64_t r2 = ptx::pack_f32x2(r, r);
  // Every table load of the call is issued before the first use: the rows come from L2 (the L1
  // left beside 227 KB of shared memory holds next to nothing), and two warps per scheduler
  // cannot hide one round trip per 8 pairs.
  float c[NP], sn[NP];
#pragma unroll
  for (int s = 0; s < NP / 8; ++s) {
    load8(cos_row + j0 + s * 8, *reinterpret_cast<float(*)[8]>(c + s * 8));
    load8(sin_row + j0 + s * 8, *reinterpret_cast<float(*)[8]>(sn + s * 8));
  }
#pragma unroll
  for (int s = 0; s < NP / 8; ++s) {
    float ga[8], gb[8];
    if (norm) {
      load_gamma8<T>(gamma + j0 + s * 8, ga);
      load_gamma8<T>(gamma + half + j0 + s * 8, gb);
    }
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
      const int w = s * 4 + i / 2;
      const float2 fa = unpack2<T>(aw[w]), fb = unpack2<T>(bw[w]);
      uint64_t x = ptx::pack_f32x2(fa.x, fa.y);
      uint64_t y = ptx::pack_f32x2(fb.x, fb.y);
      if (norm) {
        x = ptx::mul_f32x2(ptx::mul_f32x2(x, r2), ptx::pack_f32x2(ga[i], ga[i + 1]));
        y = ptx::mul_f32x2(ptx::mul_f32x2(y, r2), ptx::pack_f32x2(gb[i], gb[i + 1]));
      }
      const uint64_t c2 = ptx::pack_f32x2(c[s * 8 + i], c[s * 8 + i + 1]);
      const uint64_t s2 = ptx::pack_f32x2(sn[s * 8 + i], sn[s * 8 + i + 1]);
      const uint64_t ns2 = ptx::pack_f32x2(-sn[s * 8 + i], -sn[s * 8 + i + 1]);
      float lo0, lo1, hi0, hi1;
      ptx::unpack_f32x2(ptx::fma_f32x2(x, c2, ptx::mul_f32x2(y, ns2)), lo0, lo1);
      ptx::unpack_f32x2(ptx::fma_f32x2(y, c2, ptx::mul_f32x2(x, s2)), hi0, hi1);
      aw[w] = pack2<T>(lo0, lo1);
      bw[w] = pack2<T>(hi0, hi1);
    }
  }
}

// Epilogue of a fused q/k/v projection (flash_qwen3.rs:119-153, flash_nomic.rs:60-81): bias, then
// on the q and k heads the per-head RMSNorm (Qwen3) and the rotary embedding, v as it is.  A
// thread owns one row; a head of D columns never straddles a 256-column tile, and in the CTA-pair
// kernel each warp's half of the tile (128 columns) holds whole heads.  The arithmetic is that of
// qk_norm_rope_vec_kernel on the rounded projection, operation for operation, so both paths give
// the same bits.  The rounded values stay packed two to a register between the passes; outputs
// leave through the same staging tiles and TMA stores as the plain path.
template <class T, int D, class Release>
__device__ __forceinline__ void epilogue_tile_rope(const GemmParams& p, const CUtensorMap* tm_c, uint32_t t_row,
                                                   int m0, int n0, int quad, int lane, const T* bias,
                                                   uint8_t* stage_buf, uint32_t& store_count, Release&& release,
                                                   int part, int n_parts) {
  constexpr int HALF = D / 2;
  const int row = m0 + quad * 32 + lane;
  const int m_rows = effective_rows(p);
  const RopeFusion& rp = p.rope;
  const int pos = row < m_rows ? rp.pos_ids[row] : 0;
  const float* cos_row = rp.cos_tab + static_cast<size_t>(pos) * HALF;
  const float* sin_row = rp.sin_tab + static_cast<size_t>(pos) * HALF;
  const int rope_end = rp.q_cols + rp.k_cols;
  const bool store_rows = m0 + quad * 32 < m_rows;
  auto store = [&](uint8_t* buf, int ocol) {
    // A box that starts beyond the last row has nothing to write; the empty group keeps the
    // wait_group accounting uniform.
    if (lane == 0) {
      if (store_rows) ptx::tma_store_2d(tm_c, buf, ocol, m0 + quad * 32);
      ptx::tma_store_commit();
    }
    ++store_count;
  };
  constexpr int STEPS = 4;  // 64 output columns each
  const int c_begin = part * (STEPS / n_parts), c_end = (part + 1) * (STEPS / n_parts);
  // The accumulator goes back to the MMA thread after the warp's last read of it: the table
  // loads, the arithmetic and the stores of a tile then run beside the next tiles' main loops.
  bool released = false;
  if constexpr (D == 128) {
    // One head = two steps: the first half of the head in one staging tile, the second half in
    // the other.
#pragma unroll 1
    for (int c = c_begin; c < c_end; c += 2) {
      const int col0 = n0 + c * 64;
      if (col0 >= p.N) break;  // uniform across the CTA
      const bool rotate = col0 < rope_end;
      const T* gamma = reinterpret_cast<const T*>(col0 < rp.q_cols ? rp.q_gamma : rp.k_gamma);
      const bool norm = rotate && gamma != nullptr;
      // the whole head in registers (64 words): one pass over TMEM
      uint32_t a0[16], b0[16], a1[16], b1[16];
      rounded_pair<T>(t_row + c * 64, t_row + c * 64 + 64, bias, col0, col0 + 64, p.N, a0, b0);
      rounded_pair<T>(t_row + c * 64 + 32, t_row + c * 64 + 96, bias, col0 + 32, col0 + 96, p.N, a1, b1);
      if (c + 2 >= c_end || n0 + (c + 2) * 64 >= p.N) {
        release();
        released = true;
      }
      float r = 1.f;
      if (norm) {
        float part_ss[8];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          part_ss[t] = ss8_words<T>(a0 + t * 4, b0 + t * 4);
          part_ss[4 + t] = ss8_words<T>(a1 + t * 4, b1 + t * 4);
        }
        r = ropemath::rms_scale(ropemath::combine<8>(part_ss), D, rp.eps);
      }
      if (rotate) {
        norm_rotate<T, 32>(a0, b0, norm, r, gamma, 0, HALF, cos_row, sin_row);
        norm_rotate<T, 32>(a1, b1, norm, r, gamma, 32, HALF, cos_row, sin_row);
      }
      // both staging tiles must have been read out by their TMA stores
      if (lane == 0) ptx::tma_store_wait_read<0>();
      __syncwarp();
      uint8_t* buf0 = stage_buf + (store_count & 1) * EPI_BUF_BYTES;
      uint8_t* buf1 = stage_buf + ((store_count + 1) & 1) * EPI_BUF_BYTES;
      stage16(buf0, lane, 0, a0);
      stage16(buf0, lane, 4, a1);
      stage16(buf1, lane, 0, b0);
      stage16(buf1, lane, 4, b1);
      ptx::fence_proxy_async_smem();
      __syncwarp();
      store(buf0, col0);
      store(buf1, col0 + 64);
    }
  } else {
#pragma unroll 1
    for (int c = c_begin; c < c_end; ++c) {
      const int col0 = n0 + c * 64;
      if (col0 >= p.N) break;  // uniform across the CTA
      uint32_t x0[16], x1[16];
      rounded_pair<T>(t_row + c * 64, t_row + c * 64 + 32, bias, col0, col0 + 32, p.N, x0, x1);
      if (c + 1 >= c_end || n0 + (c + 1) * 64 >= p.N) {
        release();
        released = true;
      }
      if constexpr (D == 64) {
        // the step is one head: x0 its first half, x1 the second
        if (col0 < rope_end) {
          const T* gamma = reinterpret_cast<const T*>(col0 < rp.q_cols ? rp.q_gamma : rp.k_gamma);
          float r = 1.f;
          if (gamma) {
            float part_ss[4];
#pragma unroll
            for (int t = 0; t < 4; ++t) part_ss[t] = ss8_words<T>(x0 + t * 4, x1 + t * 4);
            r = ropemath::rms_scale(ropemath::combine<4>(part_ss), D, rp.eps);
          }
          norm_rotate<T, 32>(x0, x1, gamma != nullptr, r, gamma, 0, HALF, cos_row, sin_row);
        }
      } else {
        // D == 32: each 32-column chunk is one head, elements [0, 16) pair with [16, 32)
#pragma unroll
        for (int hlf = 0; hlf < 2; ++hlf) {
          uint32_t* x = hlf ? x1 : x0;
          const int hcol = col0 + hlf * 32;
          if (hcol < rope_end) {
            const T* gamma = reinterpret_cast<const T*>(hcol < rp.q_cols ? rp.q_gamma : rp.k_gamma);
            float r = 1.f;
            if (gamma) {
              float part_ss[2];
#pragma unroll
              for (int t = 0; t < 2; ++t) part_ss[t] = ss8_words<T>(x + t * 4, x + 8 + t * 4);
              r = ropemath::rms_scale(ropemath::combine<2>(part_ss), D, rp.eps);
            }
            norm_rotate<T, 16>(x, x + 8, gamma != nullptr, r, gamma, 0, HALF, cos_row, sin_row);
          }
        }
      }
      // The staging buffer used two stores ago must have been read out by its TMA store.
      uint8_t* buf = stage_buf + (store_count & 1) * EPI_BUF_BYTES;
      if (lane == 0) ptx::tma_store_wait_read<1>();
      __syncwarp();
      stage16(buf, lane, 0, x0);
      stage16(buf, lane, 4, x1);
      ptx::fence_proxy_async_smem();
      __syncwarp();
      store(buf, col0);
    }
  }
  if (!released) release();
}

template <class T, int ACT, int ROPE_D, int TN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                    const __grid_constant__ CUtensorMap tm_c, const GemmParams p) {
  using Cfg = SingleCfg<TN>;
  static_assert(TN == BN || ROPE_D == 0, "the rotary epilogue works on 256-column tiles");
  constexpr int STAGES = Cfg::N_STAGES, STAGE_BYTES = Cfg::STAGE, TMEM_COLS = Cfg::TMEM;  // shadow the 256-column values
  extern __shared__ uint8_t smem_raw[];
  // 128-byte-swizzled operand tiles need 1024-byte alignment.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* epi_smem = smem + STAGES * STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + EPI_BYTES);
  uint64_t* full_bar = bars;                     // [STAGES] TMA -> MMA
  uint64_t* empty_bar = bars + STAGES;           // [STAGES] MMA -> TMA
  uint64_t* acc_full = bars + 2 * STAGES;        // [2] MMA -> epilogue
  uint64_t* acc_empty = bars + 2 * STAGES + 2;   // [2] epilogue -> MMA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    ptx::prefetch_tmap(&tm_a);
    ptx::prefetch_tmap(&tm_b);
    if (p.tma_store) ptx::prefetch_tmap(&tm_c);
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(&full_bar[s], 1);
      ptx::mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&acc_full[i], 1);
      ptx::mbar_init(&acc_empty[i], 4);  // one arrival per epilogue warp
    }
    ptx::fence_mbar_init();
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  // Set-up done; what follows reads what the previous kernel wrote (the row count included).
  ptx::grid_dependency_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  const int tiles_m = (effective_rows(p) + BM - 1) / BM;
  const int tiles_n = (p.N + TN - 1) / TN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (p.K + BK - 1) / BK;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile / tiles_n) * BM;
        const int n0 = (tile % tiles_n) * TN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!ptx::mbar_wait(&empty_bar[stage], phase ^ 1)) {
            atomicExch(p.status, DEV_TIMEOUT_PRODUCER);
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          ptx::mbar_expect_tx(&full_bar[stage], STAGE_BYTES);
          ptx::tma_load_2d(sa, &tm_a, &full_bar[stage], kb * BK, m0);
          ptx::tma_load_2d(sb, &tm_b, &full_bar[stage], kb * BK, n0);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = ptx::make_idesc_f16(ptx::DTypeFmt<T>::value, BM, TN, 0, 0);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!ptx::mbar_wait(&acc_empty[acc], acc_phase ^ 1)) {
          atomicExch(p.status, DEV_TIMEOUT_MMA);
          break;
        }
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * TN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!ptx::mbar_wait(&full_bar[stage], phase)) {
            atomicExch(p.status, DEV_TIMEOUT_MMA);
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          const uint32_t sa = ptx::smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t ad = ptx::make_smem_desc_sw128(sa + k * 32, 16, 1024);
            const uint64_t bd = ptx::make_smem_desc_sw128(sb + k * 32, 16, 1024);
            ptx::umma_ss(d_tmem, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          ptx::umma_commit(&empty_bar[stage]);  // stage reusable once these MMAs have read it
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) ptx::umma_commit(&acc_full[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    const T* bias = reinterpret_cast<const T*>(p.bias);
    const bool vec_ok = (p.ldo % 8 == 0) && (p.residual == nullptr || p.ldr % 8 == 0) &&
                        ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0) &&
                        ((reinterpret_cast<uintptr_t>(p.residual) & 15) == 0);
    const bool bias_vec = bias != nullptr && (reinterpret_cast<uintptr_t>(bias) & 15) == 0;
    uint8_t* stage_buf = epi_smem + (warp - 2) * (2 * EPI_BUF_BYTES);
    uint32_t store_count = 0;  // TMA stores issued by this warp (selects the staging buffer)
    const int n_out = (ACT == ACT_SWIGLU || ACT == ACT_GEGLU) ? p.N / 2 : p.N;
    int local = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      const int m0 = (tile / tiles_n) * BM;
      const int n0 = (tile % tiles_n) * TN;
      if (!ptx::mbar_wait(&acc_full[acc], acc_phase)) {
        if (lane == 0) atomicExch(p.status, DEV_TIMEOUT_EPILOGUE);
        break;
      }
      ptx::tc_fence_after();
      const uint32_t t_row = tmem_base + acc * TN + (static_cast<uint32_t>(quad * 32) << 16);
      // Hands the accumulator back to the MMA warp (once per tile and warp, after its last read).
      auto release = [&]() {
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&acc_empty[acc]);
      };
      if constexpr (ROPE_D != 0) {
        epilogue_tile_rope<T, ROPE_D>(p, &tm_c, t_row, m0, n0, quad, lane, bias, stage_buf, store_count, release, 0, 1);
      } else {
        epilogue_tile<T, ACT, TN>(p, &tm_c, t_row, m0, n0, quad, lane, bias, bias_vec, vec_ok, stage_buf,
                                  store_count, n_out, release);
      }
    }
    // Global writes of the TMA stores must have completed before the CTA exits.
    if (p.tma_store && lane == 0) ptx::tma_store_wait<0>();
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------------
// CTA-pair variant (cta_group::2): a cluster of two CTAs computes one 256 x 256 output tile.
// Each CTA loads its own 128 rows of A and HALF of the W tile (128 of the 256 rows) per stage -
// 32 KB instead of 48 KB for the same 128 x 256 x 64 of work - so the L2 -> shared-memory
// traffic, which bounds the single-CTA kernel on these shapes, drops by a third.  The freed
// shared memory pays for eight epilogue warps (two per TMEM lane quadrant, half of the columns
// each), which halves the time an accumulator stays busy.  The even CTA issues tcgen05.mma.cta_group::2 (M = 256), which reads both
// CTAs' shared memory and writes each CTA's 128 x 256 accumulator in its own TMEM; commits are
// multicast to the mbarriers of both CTAs.  TMA loads are plain per-CTA loads whose bytes are
// counted on the even CTA's "full" barrier.
constexpr int P_STAGES = 5;
constexpr int P_EPI_WARPS = 8;  // two warps per TMEM lane quadrant, each takes half of the columns
constexpr int P_THREADS = (2 + P_EPI_WARPS) * 32;
constexpr int P_EPI_BYTES = P_EPI_WARPS * 2 * EPI_BUF_BYTES;
constexpr int P_B_BYTES = 128 * BK * 2;
constexpr int P_STAGE_BYTES = A_BYTES + P_B_BYTES;
constexpr int P_SMEM_BYTES = P_STAGES * P_STAGE_BYTES + P_EPI_BYTES + 1024 + 256;

template <class T, int ACT, int ROPE_D>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(P_THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                         const __grid_constant__ CUtensorMap tm_c, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  // The same offset in both CTAs: shared-memory windows of a cluster's CTAs are congruent.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* epi_smem = smem + P_STAGES * P_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + P_EPI_BYTES);
  uint64_t* full_bar = bars;                       // [P_STAGES] used in the even CTA only
  uint64_t* empty_bar = bars + P_STAGES;           // [P_STAGES] one per CTA, signalled by commit
  uint64_t* acc_full = bars + 2 * P_STAGES;        // [2] one per CTA, signalled by commit
  uint64_t* acc_empty = bars + 2 * P_STAGES + 2;   // [2] used in the even CTA only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * P_STAGES + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    ptx::prefetch_tmap(&tm_a);
    ptx::prefetch_tmap(&tm_b);
    if (p.tma_store) ptx::prefetch_tmap(&tm_c);
    for (int s = 0; s < P_STAGES; ++s) {
      ptx::mbar_init(&full_bar[s], 1);
      ptx::mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&acc_full[i], 1);
      ptx::mbar_init(&acc_empty[i], 2 * P_EPI_WARPS);  // one arrival per epilogue warp of both CTAs
    }
    ptx::fence_mbar_init();
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(tmem_slot, TMEM_COLS);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync_all();  // the peer's barriers exist before anything is sent to them
  ptx::tc_fence_after();
  // Set-up done; what follows reads what the previous kernel wrote (the row count included).
  ptx::grid_dependency_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  const int tiles_m = (effective_rows(p) + 2 * BM - 1) / (2 * BM);
  const int tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (p.K + BK - 1) / BK;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        const int m0 = (tile / tiles_n) * (2 * BM) + static_cast<int>(rank) * BM;
        const int n0 = (tile % tiles_n) * BN + static_cast<int>(rank) * 128;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!ptx::mbar_wait(&empty_bar[stage], phase ^ 1)) {
            atomicExch(p.status, DEV_TIMEOUT_PRODUCER);
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * P_STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          // The even CTA arms its barrier for the bytes of both CTAs.
          if (rank == 0) ptx::mbar_expect_tx(&full_bar[stage], 2 * P_STAGE_BYTES);
          const uint32_t bar = ptx::smem_u32(&full_bar[stage]) & ptx::kPeerBitMask;
          ptx::tma_load_2d_pair(sa, &tm_a, bar, kb * BK, m0);
          ptx::tma_load_2d_pair(sb, &tm_b, bar, kb * BK, n0);
          if (++stage == P_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (even CTA only)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = ptx::make_idesc_f16(ptx::DTypeFmt<T>::value, 2 * BM, BN, 0, 0);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!ptx::mbar_wait(&acc_empty[acc], acc_phase ^ 1)) {
          atomicExch(p.status, DEV_TIMEOUT_MMA);
          break;
        }
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!ptx::mbar_wait(&full_bar[stage], phase)) {
            atomicExch(p.status, DEV_TIMEOUT_MMA);
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          const uint32_t sa = ptx::smem_u32(smem + stage * P_STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t ad = ptx::make_smem_desc_sw128(sa + k * 32, 16, 1024);
            const uint64_t bd = ptx::make_smem_desc_sw128(sb + k * 32, 16, 1024);
            ptx::umma_ss_pair(d_tmem, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          ptx::umma_commit_pair(&empty_bar[stage], 3);  // the stage is free in both CTAs
          if (++stage == P_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) ptx::umma_commit_pair(&acc_full[acc], 3);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..9, both CTAs)
    const int quad = warp & 3;           // TMEM lane quadrant this warp may read
    const int part = (warp - 2) >> 2;    // which half of the 256 columns it handles
    const T* bias = reinterpret_cast<const T*>(p.bias);
    const bool vec_ok = (p.ldo % 8 == 0) && (p.residual == nullptr || p.ldr % 8 == 0) &&
                        ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0) &&
                        ((reinterpret_cast<uintptr_t>(p.residual) & 15) == 0);
    const bool bias_vec = bias != nullptr && (reinterpret_cast<uintptr_t>(bias) & 15) == 0;
    uint8_t* stage_buf = epi_smem + (warp - 2) * (2 * EPI_BUF_BYTES);
    uint32_t store_count = 0;
    const int n_out = (ACT == ACT_SWIGLU || ACT == ACT_GEGLU) ? p.N / 2 : p.N;
    int local = 0;
    for (int tile = pair; tile < num_tiles; tile += num_pairs, ++local) {
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      const int m0 = (tile / tiles_n) * (2 * BM) + static_cast<int>(rank) * BM;
      const int n0 = (tile % tiles_n) * BN;
      if (!ptx::mbar_wait(&acc_full[acc], acc_phase)) {
        if (lane == 0) atomicExch(p.status, DEV_TIMEOUT_EPILOGUE);
        break;
      }
      ptx::tc_fence_after();
      const uint32_t t_row = tmem_base + acc * BN + (static_cast<uint32_t>(quad * 32) << 16);
      // Hands the accumulator back to the MMA thread of the even CTA (once per tile and warp,
      // after its last read).
      auto release = [&]() {
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive_cluster(ptx::smem_u32(&acc_empty[acc]) & ptx::kPeerBitMask);
      };
      if constexpr (ROPE_D != 0) {
        epilogue_tile_rope<T, ROPE_D>(p, &tm_c, t_row, m0, n0, quad, lane, bias, stage_buf, store_count, release, part,
                                      2);
      } else {
        epilogue_tile<T, ACT>(p, &tm_c, t_row, m0, n0, quad, lane, bias, bias_vec, vec_ok, stage_buf, store_count,
                              n_out, release, part, 2);
      }
    }
    if (p.tma_store && lane == 0) ptx::tma_store_wait<0>();
  }

  // Neither CTA may leave while the other can still read its shared memory or signal its
  // barriers.
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync_all();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

// One CTA per 128 x TN tile.
template <class T, int ACT, int ROPE_D, int TN>
int launch_single(const GemmArgs& g, const GemmParams& p, const CUtensorMap& tm_a, const CUtensorMap& tm_c,
                  CUtensorMapDataType dt, cudaStream_t stream) {
  using Cfg = SingleCfg<TN>;
  CUtensorMap tm_b;
  const int rc = make_tmap_2d(&tm_b, g.w, dt, 2, g.K, g.N, static_cast<uint64_t>(g.K) * 2, BK, TN);
  if (rc) return rc;
  // The opt-in shared-memory size is a per-device function attribute; setting it twice is
  // harmless, so replicas on several threads may race to set it, but not on the flag itself.
  static std::atomic<bool> attr_set[64];
  const int dev = current_device() & 63;
  auto kern = gemm_tcgen05_kernel<T, ACT, ROPE_D, TN>;
  if (!attr_set[dev].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set[dev].store(true, std::memory_order_release);
  }
  const long long tiles = static_cast<long long>((g.M + BM - 1) / BM) * ((g.N + TN - 1) / TN);
  const int grid = tiles < num_sms() ? static_cast<int>(tiles) : num_sms();
  return static_cast<int>(launch_dependent(kern, dim3(grid), dim3(NUM_THREADS), Cfg::SMEM, stream, tm_a, tm_b, tm_c, p));
}

// Which tiling finishes first, counted in waves of the CTA-pair kernel (one 256 x 256 tile per
// pair of SMs = one 128 x 256 tile per SM).  A narrow tile does a half or a quarter of the
// arithmetic but its wave is hardly shorter: every k-block still waits for a 16 KB A tile and a
// W tile from L2, and the main loop of these kernels is bound by those loads, not by the MMAs
// (measured at 8,572 and 34,288 rows: a wave of 128-column tiles takes 0.8 to 0.9 of a wave of
// pairs, a wave of 64-column tiles about 0.8).  So the narrow tiles only pay where the wide ones
// would leave most SMs without a tile: batches of up to about two thousand tokens.
// 0: CTA pairs, else the single-CTA tile width.
inline int pick_tiling(int M, int N, int sms, bool narrow_ok) {
  auto waves = [](long long tiles, int slots) { return static_cast<double>((tiles + slots - 1) / slots); };
  const long long tm = (M + BM - 1) / BM, tm2 = (M + 2 * BM - 1) / (2 * BM);
  int best = 256;
  double best_cost = 1.25 * waves(tm * ((N + 255) / 256), sms);
  if (M > BM && sms >= 2) {
    const double c = waves(tm2 * ((N + 255) / 256), sms / 2);
    if (c <= best_cost) best_cost = c, best = 0;
  }
  if (narrow_ok) {
    const double c128 = 0.88 * waves(tm * ((N + 127) / 128), sms);
    if (c128 < best_cost) best_cost = c128, best = 128;
    const double c64 = 0.80 * waves(tm * ((N + 63) / 64), sms);
    if (c64 < best_cost) best_cost = c64, best = 64;
  }
  return best;
}

template <class T, int ACT, int ROPE_D = 0>
int launch_typed(const GemmArgs& g, cudaStream_t stream) {
  CUtensorMap tm_a;
  const CUtensorMapDataType dt =
      g.dtype == DT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  int rc = make_tmap_2d(&tm_a, g.a, dt, 2, g.K, g.M, static_cast<uint64_t>(g.lda) * 2, BK, BM);
  if (rc) return rc;
  // Outputs leave through TMA stores when the output rows are 16-byte aligned and no residual
  // is fused; otherwise the epilogue falls back to per-thread stores.
  const int n_out = (ACT == ACT_SWIGLU || ACT == ACT_GEGLU) ? g.N / 2 : g.N;
  const bool tma_store = (g.residual == nullptr || ACT == ACT_ADD_RES) && g.ldo % 8 == 0 &&
                         (reinterpret_cast<uintptr_t>(g.out) & 15) == 0;
  CUtensorMap tm_c = tm_a;  // placeholder when unused (never dereferenced by the kernel)
  if (tma_store) {
    rc = make_tmap_2d(&tm_c, g.out, dt, 2, n_out, g.M, static_cast<uint64_t>(g.ldo) * 2, 64, 32);
    if (rc) return rc;
  }

  static std::atomic<bool> attr_set_pair[64];  // see launch_single
  const int dev = current_device() & 63;
  GemmParams p;
  p.bias = g.bias;
  p.residual = g.residual;
  p.out = g.out;
  p.M = g.M;
  p.m_dev = g.m_dev;
  p.N = g.N;
  p.K = g.K;
  p.ldo = g.ldo;
  p.ldr = g.ldr;
  p.tma_store = tma_store ? 1 : 0;
  p.status = g.status;
  p.rope = RopeFusion{};
  if (ROPE_D != 0) {
    if (!tma_store || g.rope == nullptr) return static_cast<int>(cudaErrorInvalidValue);
    p.rope = *g.rope;
  }
  // Narrow tiles exist for the plain epilogues only; a row count known only on the device (the
  // experts of a mixture) says nothing about the waves.
  constexpr bool kNarrow = ROPE_D == 0 && !(ACT == ACT_SWIGLU || ACT == ACT_GEGLU);
  const int tiling = pick_tiling(g.M, g.N, num_sms(), kNarrow && g.m_dev == nullptr);
  if (tiling == 0) {
    // CTA pairs: 256 x 256 tiles, W loaded in halves of 128 rows.
    CUtensorMap tm_b2;
    rc = make_tmap_2d(&tm_b2, g.w, dt, 2, g.K, g.N, static_cast<uint64_t>(g.K) * 2, BK, 128);
    if (rc) return rc;
    auto kern2 = gemm_tcgen05_pair_kernel<T, ACT, ROPE_D>;
    if (!attr_set_pair[dev].load(std::memory_order_acquire)) {
      cudaError_t e = cudaFuncSetAttribute(kern2, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM_BYTES);
      if (e != cudaSuccess) return static_cast<int>(e);
      attr_set_pair[dev].store(true, std::memory_order_release);
    }
    const int tiles2 = ((g.M + 2 * BM - 1) / (2 * BM)) * ((g.N + BN - 1) / BN);
    const int max_pairs = num_sms() / 2;
    const int pairs = tiles2 < max_pairs ? tiles2 : max_pairs;
    return static_cast<int>(launch_dependent(kern2, dim3(2 * pairs), dim3(P_THREADS), P_SMEM_BYTES, stream, tm_a, tm_b2,
                                             tm_c, p));
  }
  if constexpr (kNarrow) {
    if (tiling == 128) return launch_single<T, ACT, ROPE_D, 128>(g, p, tm_a, tm_c, dt, stream);
    if (tiling == 64) return launch_single<T, ACT, ROPE_D, 64>(g, p, tm_a, tm_c, dt, stream);
  }
  return launch_single<T, ACT, ROPE_D, 256>(g, p, tm_a, tm_c, dt, stream);
}

template <class T>
int launch_by_act(const GemmArgs& g, cudaStream_t stream) {
  if (g.rope) {
    const RopeFusion& r = *g.rope;
    if (g.act != ACT_NONE || g.residual || !r.pos_ids || !r.cos_tab || !r.sin_tab || r.q_cols < 0 || r.k_cols < 0 ||
        r.q_cols + r.k_cols > g.N || (r.head_dim != 32 && r.head_dim != 64 && r.head_dim != 128) ||
        r.q_cols % r.head_dim || r.k_cols % r.head_dim || g.N % r.head_dim || (g.bias && g.N % 2) ||
        (reinterpret_cast<uintptr_t>(r.q_gamma) & 15) || (reinterpret_cast<uintptr_t>(r.k_gamma) & 15) ||
        (reinterpret_cast<uintptr_t>(r.cos_tab) & 15) || (reinterpret_cast<uintptr_t>(r.sin_tab) & 15)) {
      return static_cast<int>(cudaErrorInvalidValue);
    }
    switch (r.head_dim) {
      case 32: return launch_typed<T, ACT_NONE, 32>(g, stream);
      case 64: return launch_typed<T, ACT_NONE, 64>(g, stream);
      default: return launch_typed<T, ACT_NONE, 128>(g, stream);
    }
  }
  if (g.act == ACT_NONE && g.residual != nullptr && g.N % 64 == 0 && g.ldr % 8 == 0 &&
      (reinterpret_cast<uintptr_t>(g.residual) & 15) == 0 && (g.bias == nullptr || g.N % 2 == 0)) {
    return launch_typed<T, ACT_ADD_RES>(g, stream);
  }
  switch (g.act) {
    case ACT_NONE: return launch_typed<T, ACT_NONE>(g, stream);
    case ACT_GELU: return launch_typed<T, ACT_GELU>(g, stream);
    case ACT_RELU: return launch_typed<T, ACT_RELU>(g, stream);
    case ACT_TANH: return launch_typed<T, ACT_TANH>(g, stream);
    case ACT_SWIGLU: return launch_typed<T, ACT_SWIGLU>(g, stream);
    case ACT_RELU_LOG1P: return launch_typed<T, ACT_RELU_LOG1P>(g, stream);
    case ACT_GEGLU: return launch_typed<T, ACT_GEGLU>(g, stream);
    default: return static_cast<int>(cudaErrorInvalidValue);
  }
}

}  // namespace

int gemm_smem_bytes() { return SMEM_BYTES; }

int gemm_tiling(int M, int N, int sms, bool narrow_ok) { return pick_tiling(M, N, sms, narrow_ok); }

int launch_gemm(const GemmArgs& g, cudaStream_t stream) {
  // The kernels report a wait that ran out through *status: without it there is nowhere to write.
  if (g.status == nullptr) return static_cast<int>(cudaErrorInvalidValue);
  if (g.M <= 0) return 0;
  if (g.N <= 0 || g.K <= 0 || g.K % 8 != 0 || g.lda % 8 != 0) {
    return static_cast<int>(cudaErrorInvalidValue);
  }
  if (act_is_glu(g.act) && g.N % 256 != 0) return static_cast<int>(cudaErrorInvalidValue);
  if ((reinterpret_cast<uintptr_t>(g.a) & 15) || (reinterpret_cast<uintptr_t>(g.w) & 15)) {
    return static_cast<int>(cudaErrorInvalidValue);
  }
  return g.dtype == DT_F16 ? launch_by_act<__half>(g, stream)
                           : launch_by_act<__nv_bfloat16>(g, stream);
}

}  // namespace tei
