// HBM-bound row kernels of the encoder forward: fused embedding gather + LayerNorm, fused
// residual add + LayerNorm / RMSNorm, per-head RMSNorm + rotary embedding, segmented pooling
// driven by cu_seqlens, row gather to fp32 and the small dense heads.
//
// All of them move each byte once with 16-byte accesses, keep the row in registers between the
// statistics pass and the normalisation pass, and do their arithmetic in fp32.
#include "kernels.h"
#include "ptx.cuh"
#include "rope_math.cuh"
#include "tmap.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace tei {
namespace {

template <class T>
__device__ __forceinline__ float ldf(const T& v);
template <>
__device__ __forceinline__ float ldf<__half>(const __half& v) {
  return __half2float(v);
}
template <>
__device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16& v) {
  return __bfloat162float(v);
}
template <class T>
__device__ __forceinline__ T stf(float v);
template <>
__device__ __forceinline__ __half stf<__half>(float v) {
  return __float2half_rn(v);
}
template <>
__device__ __forceinline__ __nv_bfloat16 stf<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// Takes the 16 bytes BY VALUE: a reference to a dereferenced global pointer would let the
// compiler read the eight elements with eight narrow loads instead of one 128-bit load.
template <class T>
__device__ __forceinline__ void unpack8(uint4 u, float* f);
template <>
__device__ __forceinline__ void unpack8<__half>(uint4 u, float* f) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    f[2 * i] = v.x;
    f[2 * i + 1] = v.y;
  }
}
template <>
__device__ __forceinline__ void unpack8<__nv_bfloat16>(uint4 u, float* f) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    // bf16 -> fp32 is a 16-bit shift
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
// 128-bit read-only load.
__device__ __forceinline__ uint4 ld16(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
template <class T>
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 u;
  T* t = reinterpret_cast<T*>(&u);
#pragma unroll
  for (int i = 0; i < 8; ++i) t[i] = stf<T>(f[i]);
  return u;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ------------------------------------------------------------------ row normalisation core
// One warp owns one row of H = 8 * n_chunks elements; lane l holds chunks l, l+32, ...
// (at most MAXC of them) in registers.  Returns with v[] normalised and scaled.
template <class T, int MAXC, bool RMS>
__device__ __forceinline__ void normalise_row(float (&v)[MAXC][8], int n_chunks, int lane, int H,
                                              float eps, const T* gamma, const T* beta) {
  float s = 0.f;
  if (!RMS) {
#pragma unroll
    for (int c = 0; c < MAXC; ++c) {
      if (lane + c * 32 < n_chunks) {
#pragma unroll
        for (int i = 0; i < 8; ++i) s += v[c][i];
      }
    }
    s = warp_sum(s);
  }
  const float mean = RMS ? 0.f : s / static_cast<float>(H);
  float q = 0.f;
#pragma unroll
  for (int c = 0; c < MAXC; ++c) {
    if (lane + c * 32 < n_chunks) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float d = v[c][i] - mean;
        q += d * d;
      }
    }
  }
  q = warp_sum(q);
  const float rstd = rsqrtf(q / static_cast<float>(H) + eps);
#pragma unroll
  for (int c = 0; c < MAXC; ++c) {
    const int ch = lane + c * 32;
    if (ch < n_chunks) {
      float g[8], b[8];
      unpack8<T>(ld16(gamma + ch * 8), g);
      if (!RMS && beta) {
        unpack8<T>(ld16(beta + ch * 8), b);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) b[i] = 0.f;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) v[c][i] = (v[c][i] - mean) * rstd * g[i] + b[i];
    }
  }
}

// ------------------------------------------------------------------ embedding (+ LayerNorm)
// word[ids] + type[type_ids] + pos[pos_ids] -> LayerNorm, as BertEmbeddings::forward
// (backends/candle/src/models/bert.rs:83-101) and NomicBertEmbeddings::forward
// (models/nomic.rs:84-95); with gamma == nullptr it is the plain gather of
// flash_qwen3.rs:409.
template <class T, int MAXC>
__global__ void __launch_bounds__(256)
embed_ln_kernel(const int* __restrict__ ids, const int* __restrict__ type_ids,
                const int* __restrict__ pos_ids, const T* __restrict__ word,
                const T* __restrict__ type_tab, const T* __restrict__ pos_tab,
                const T* __restrict__ gamma, const T* __restrict__ beta, T* __restrict__ out, int T_,
                int H, float eps) {
  ptx::grid_dependency_sync();
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= T_) return;
  const int n_chunks = H >> 3;
  const T* w = word + static_cast<size_t>(ids[row]) * H;
  const T* t = type_tab ? type_tab + static_cast<size_t>(type_ids[row]) * H : nullptr;
  const T* p = pos_tab ? pos_tab + static_cast<size_t>(pos_ids[row]) * H : nullptr;
  float v[MAXC][8];
#pragma unroll
  for (int c = 0; c < MAXC; ++c) {
    const int ch = lane + c * 32;
    if (ch < n_chunks) {
      unpack8<T>(ld16(w + ch * 8), v[c]);
      float a[8];
      if (t) {
        unpack8<T>(ld16(t + ch * 8), a);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[c][i] += a[i];
      }
      if (p) {
        unpack8<T>(ld16(p + ch * 8), a);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[c][i] += a[i];
      }
    }
  }
  if (gamma) normalise_row<T, MAXC, false>(v, n_chunks, lane, H, eps, gamma, beta);
  T* o = out + static_cast<size_t>(row) * H;
#pragma unroll
  for (int c = 0; c < MAXC; ++c) {
    const int ch = lane + c * 32;
    if (ch < n_chunks) *reinterpret_cast<uint4*>(o + ch * 8) = pack8<T>(v[c]);
  }
}

// ------------------------------------------------------------------ residual add + norm
// LayerNorm: out = LN(x + residual) (backends/candle/src/layers/layer_norm.rs:108-132).
// RMSNorm:   sum = x + residual, out = sum * rsqrt(mean(sum^2) + eps) * gamma
//            (layers/rms_norm.rs:30-57); the running sum is kept in fp32 so that rounding does
//            not pile up over the decoder's layers.
// F32RES: the residual is fp32 and the sum is written back in fp32 (the pre-norm models: RMSNorm
// decoders, and ModernBERT with LayerNorm).  gamma == nullptr: no normalisation, out = sum.
template <class T, int MAXC, bool RMS, bool F32RES>
__global__ void __launch_bounds__(256, (MAXC <= 3 ? 6 : (MAXC == 4 ? 4 : 1)))
add_norm_kernel(const T* __restrict__ x, const void* residual, const T* __restrict__ gamma,
                const T* __restrict__ beta, T* __restrict__ out, float* sum_out, int T_, int H,
                float eps) {
  ptx::grid_dependency_sync();  // residual and sum_out may be the same buffer: no __restrict__
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= T_) return;
  const int n_chunks = H >> 3;
  const T* xr = x + static_cast<size_t>(row) * H;
  float v[MAXC][8];
#pragma unroll
  for (int c = 0; c < MAXC; ++c) {
    const int ch = lane + c * 32;
    if (ch < n_chunks) {
      unpack8<T>(ld16(xr + ch * 8), v[c]);
      if (residual) {
        if (F32RES) {
          const float* rr = reinterpret_cast<const float*>(residual) + static_cast<size_t>(row) * H;
          const float4 r0 = *reinterpret_cast<const float4*>(rr + ch * 8);
          const float4 r1 = *reinterpret_cast<const float4*>(rr + ch * 8 + 4);
          v[c][0] += r0.x; v[c][1] += r0.y; v[c][2] += r0.z; v[c][3] += r0.w;
          v[c][4] += r1.x; v[c][5] += r1.y; v[c][6] += r1.z; v[c][7] += r1.w;
        } else {
          const T* rr = reinterpret_cast<const T*>(residual) + static_cast<size_t>(row) * H;
          float a[8];
          unpack8<T>(ld16(rr + ch * 8), a);
#pragma unroll
          for (int i = 0; i < 8; ++i) v[c][i] += a[i];
        }
      }
      if (F32RES && sum_out) {
        float* so = sum_out + static_cast<size_t>(row) * H + ch * 8;
        *reinterpret_cast<float4*>(so) = make_float4(v[c][0], v[c][1], v[c][2], v[c][3]);
        *reinterpret_cast<float4*>(so + 4) = make_float4(v[c][4], v[c][5], v[c][6], v[c][7]);
      }
    }
  }
  if (gamma) normalise_row<T, MAXC, RMS>(v, n_chunks, lane, H, eps, gamma, beta);
  T* o = out + static_cast<size_t>(row) * H;
#pragma unroll
  for (int c = 0; c < MAXC; ++c) {
    const int ch = lane + c * 32;
    if (ch < n_chunks) *reinterpret_cast<uint4*>(o + ch * 8) = pack8<T>(v[c]);
  }
}

// LayerNorm without bias over fp32 rows, in place (the classification head of ModernBERT,
// backends/candle/src/models/modernbert.rs:443-456, runs on the few pooled rows).
template <class T>
__global__ void __launch_bounds__(256) layernorm_rows_f32_kernel(float* __restrict__ x, const T* __restrict__ gamma,
                                                                 int rows, int H, float eps) {
  ptx::grid_dependency_sync();
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  float* r = x + static_cast<size_t>(row) * H;
  float s = 0.f;
  for (int j = lane; j < H; j += 32) s += r[j];
  const float mean = warp_sum(s) / static_cast<float>(H);
  float q = 0.f;
  for (int j = lane; j < H; j += 32) q += (r[j] - mean) * (r[j] - mean);
  const float rstd = rsqrtf(warp_sum(q) / static_cast<float>(H) + eps);
  for (int j = lane; j < H; j += 32) r[j] = (r[j] - mean) * rstd * ldf<T>(gamma[j]);
}

// LayerNorm over whole q rows and whole k rows (all heads together), in place, on strided views
// of the fused projection output: JinaCodeBert normalises q and k before attention
// (backends/candle/src/models/flash_jina_code.rs:112-120).  One warp per row; rows [0, T) are
// q, rows [T, 2T) are k.  Statistics in fp32 from the values as stored, like layer_norm.rs:108-132.
template <class T>
__global__ void __launch_bounds__(256)
layernorm_qk_kernel(T* q, T* k, int ld, const T* __restrict__ gq, const T* __restrict__ bq,
                    const T* __restrict__ gk, const T* __restrict__ bk, int T_, int H, float eps) {
  ptx::grid_dependency_sync();
  const int lane = threadIdx.x & 31;
  const int idx = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (idx >= 2 * T_) return;
  const bool is_k = idx >= T_;
  T* r = (is_k ? k : q) + static_cast<size_t>(is_k ? idx - T_ : idx) * ld;
  const T* g = is_k ? gk : gq;
  const T* b = is_k ? bk : bq;
  float s = 0.f;
  for (int j = lane; j < H; j += 32) s += ldf<T>(r[j]);
  const float mean = warp_sum(s) / static_cast<float>(H);
  float v = 0.f;
  for (int j = lane; j < H; j += 32) {
    const float d = ldf<T>(r[j]) - mean;
    v += d * d;
  }
  const float rstd = rsqrtf(warp_sum(v) / static_cast<float>(H) + eps);
  for (int j = lane; j < H; j += 32) {
    // cast back to the model dtype before the affine part (layer_norm.rs:127-131)
    const float n = ldf<T>(stf<T>((ldf<T>(r[j]) - mean) * rstd));
    r[j] = stf<T>(n * ldf<T>(g[j]) + ldf<T>(b[j]));
  }
}

// ------------------------------------------------------------------ per-head RMSNorm + RoPE
// One warp per (token, head).  Optional RMSNorm over the head (flash_qwen3.rs:150-151), then
// x*cos + rotate_half(x)*sin with the half-rotation pairing (j, j + head_dim/2)
// (layers/rotary.rs:118-130); cos / sin come from an fp32 [max_pos, head_dim/2] table.
template <class T>
__global__ void __launch_bounds__(256)
qk_norm_rope_kernel(T* __restrict__ q, T* __restrict__ k, const int* __restrict__ pos_ids,
                    const float* __restrict__ cos_tab, const float* __restrict__ sin_tab,
                    const T* __restrict__ q_gamma, const T* __restrict__ k_gamma, int T_, int nh,
                    int nkv, int dh, int ld_q, int ld_k, float eps) {
  ptx::grid_dependency_sync();
  const int lane = threadIdx.x & 31;
  const long long w = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int heads = nh + nkv;
  if (w >= static_cast<long long>(T_) * heads) return;
  const int tok = static_cast<int>(w / heads);
  const int h = static_cast<int>(w % heads);
  T* base = h < nh ? q + static_cast<size_t>(tok) * ld_q + h * dh
                   : k + static_cast<size_t>(tok) * ld_k + (h - nh) * dh;
  const T* gamma = h < nh ? q_gamma : k_gamma;
  const int half = dh >> 1;
  const float* cs = cos_tab + static_cast<size_t>(pos_ids[tok]) * half;
  const float* sn = sin_tab + static_cast<size_t>(pos_ids[tok]) * half;
  // head_dim <= 256: at most 4 pairs per lane.
  float a[4], b[4];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int j = lane + i * 32;
    if (j < half) {
      a[i] = ldf<T>(base[j]);
      b[i] = ldf<T>(base[j + half]);
      ss += a[i] * a[i] + b[i] * b[i];
    }
  }
  if (gamma) {
    ss = warp_sum(ss);
    const float r = rsqrtf(ss / static_cast<float>(dh) + eps);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int j = lane + i * 32;
      if (j < half) {
        a[i] = a[i] * r * ldf<T>(gamma[j]);
        b[i] = b[i] * r * ldf<T>(gamma[j + half]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int j = lane + i * 32;
    if (j < half) {
      const float c = cs[j], s = sn[j];
      base[j] = stf<T>(a[i] * c - b[i] * s);
      base[j + half] = stf<T>(b[i] * c + a[i] * s);
    }
  }
}

// The same for head_dim 32, 64 and 128 with 16-byte accesses: DH / 16 lanes share one (token, head);
// each lane owns 8 consecutive elements of the first half and the 8 they pair with in the
// second half, so every load and store is a full 16 bytes and a warp covers 8 (or 4) heads of a
// token at once.  The RMSNorm sum is reduced across the lanes of the group.
template <class T, int DH>
__global__ void __launch_bounds__(256)
qk_norm_rope_vec_kernel(T* __restrict__ q, T* __restrict__ k, const int* __restrict__ pos_ids,
                        const float* __restrict__ cos_tab, const float* __restrict__ sin_tab,
                        const T* __restrict__ q_gamma, const T* __restrict__ k_gamma, int T_, int nh,
                        int nkv, int ld_q, int ld_k, float eps) {
  ptx::grid_dependency_sync();
  constexpr int G = DH / 16;     // lanes per (token, head)
  constexpr int HALF = DH / 2;
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int heads = nh + nkv;
  const long long total = static_cast<long long>(T_) * heads;
  long long w = tid / G;
  const int sub = static_cast<int>(tid % G);
  const bool valid = w < total;   // whole groups are valid or not; no early exit (warp shuffles)
  if (!valid) w = total - 1;
  const int tok = static_cast<int>(w / heads);
  const int h = static_cast<int>(w % heads);
  T* base = (h < nh ? q + static_cast<size_t>(tok) * ld_q + h * DH
                    : k + static_cast<size_t>(tok) * ld_k + (h - nh) * DH) + sub * 8;
  const T* gamma = h < nh ? q_gamma : k_gamma;
  float a[8], b[8];
  unpack8<T>(ld16(base), a);
  unpack8<T>(ld16(base + HALF), b);
  if (gamma) {
    float ss = ropemath::ss8(a, b);
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, o));
    const float r = ropemath::rms_scale(ss, DH, eps);
    float ga[8], gb[8];
    unpack8<T>(ld16(gamma + sub * 8), ga);
    unpack8<T>(ld16(gamma + HALF + sub * 8), gb);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      a[i] = ropemath::normed(a[i], r, ga[i]);
      b[i] = ropemath::normed(b[i], r, gb[i]);
    }
  }
  const size_t trow = static_cast<size_t>(pos_ids[tok]) * HALF + sub * 8;
  const float4 c0 = *reinterpret_cast<const float4*>(cos_tab + trow);
  const float4 c1 = *reinterpret_cast<const float4*>(cos_tab + trow + 4);
  const float4 s0 = *reinterpret_cast<const float4*>(sin_tab + trow);
  const float4 s1 = *reinterpret_cast<const float4*>(sin_tab + trow + 4);
  const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
  const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
  float oa[8], ob[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    oa[i] = ropemath::rot_lo(a[i], b[i], c[i], sn[i]);
    ob[i] = ropemath::rot_hi(a[i], b[i], c[i], sn[i]);
  }
  if (valid) {
    *reinterpret_cast<uint4*>(base) = pack8<T>(oa);
    *reinterpret_cast<uint4*>(base + HALF) = pack8<T>(ob);
  }
}

// ------------------------------------------------------------------ segmented pooling
// One block per (output row, slab of 256 columns); 32 column groups of 8 x 8 row lanes.
// mode 0: first row of the sequence, 3: last row, 1: mean over the rows, 2: max over the rows
// (flash_bert.rs:396-490).  Writes fp32.
template <class T>
__global__ void __launch_bounds__(256)
pool_kernel(const T* __restrict__ x, const int* __restrict__ cu, const int* __restrict__ seq_index,
            float* __restrict__ out, int H, int mode) {
  ptx::grid_dependency_sync();
  const int o = blockIdx.x;
  const int s = seq_index[o];
  const int start = cu[s], end = cu[s + 1];
  const int cg = threadIdx.x & 31;
  const int rl = threadIdx.x >> 5;
  const int col = blockIdx.y * 256 + cg * 8;
  __shared__ float red[8][32][8];
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = (mode == 2) ? -INFINITY : 0.f;
  if (col < H) {
    if (mode == 0 || mode == 3) {
      if (rl == 0 && end > start) {
        const int r = mode == 0 ? start : end - 1;
        unpack8<T>(ld16(x + static_cast<size_t>(r) * H + col), acc);
      }
    } else {
      for (int r = start + rl; r < end; r += 8) {
        float f[8];
        unpack8<T>(ld16(x + static_cast<size_t>(r) * H + col), f);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = (mode == 2) ? fmaxf(acc[i], f[i]) : acc[i] + f[i];
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) red[rl][cg][i] = acc[i];
  __syncthreads();
  if (rl == 0 && col < H) {
    if (mode == 1 || mode == 2) {
#pragma unroll
      for (int r = 1; r < 8; ++r) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          acc[i] = (mode == 2) ? fmaxf(acc[i], red[r][cg][i]) : acc[i] + red[r][cg][i];
        }
      }
      if (mode == 1) {
        const float inv = 1.0f / static_cast<float>(end - start);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] *= inv;
      }
    }
    float* dst = out + static_cast<size_t>(o) * H + col;
    *reinterpret_cast<float4*>(dst) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    *reinterpret_cast<float4*>(dst + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
  }
}

// In-place L2 normalisation of fp32 rows (core/src/infer.rs:288-303 does this on the host).
__global__ void __launch_bounds__(256) l2_normalise_kernel(float* __restrict__ x, int rows, int H) {
  ptx::grid_dependency_sync();
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  float* r = x + static_cast<size_t>(row) * H;
  float ss = 0.f;
  for (int j = lane; j < H; j += 32) ss += r[j] * r[j];
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss);
  for (int j = lane; j < H; j += 32) r[j] *= inv;
}

template <class T>
__global__ void __launch_bounds__(256)
gather_rows_kernel(const T* __restrict__ x, const int* __restrict__ row_index,
                   float* __restrict__ out, int n_rows, int H) {
  ptx::grid_dependency_sync();
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const T* src = x + static_cast<size_t>(row_index[row]) * H;
  float* dst = out + static_cast<size_t>(row) * H;
  for (int ch = lane; ch < (H >> 3); ch += 32) {
    float f[8];
    unpack8<T>(ld16(src + ch * 8), f);
    *reinterpret_cast<float4*>(dst + ch * 8) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(dst + ch * 8 + 4) = make_float4(f[4], f[5], f[6], f[7]);
  }
}

// out[r, n] = act(sum_k in[r, k] * w[n, k] + b[n]); one warp per output element.  Used for the
// classification heads (models/bert.rs:405-465) and Dense modules, whose inputs are a few
// hundred pooled rows at most.
template <class T>
__global__ void __launch_bounds__(256)
head_linear_kernel(const float* __restrict__ in, const T* __restrict__ w, const T* __restrict__ b,
                   float* __restrict__ out, int rows, int N, int K, int act) {
  ptx::grid_dependency_sync();
  const int lane = threadIdx.x & 31;
  const long long wid = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (wid >= static_cast<long long>(rows) * N) return;
  const int r = static_cast<int>(wid / N);
  const int n = static_cast<int>(wid % N);
  const float* x = in + static_cast<size_t>(r) * K;
  const T* wr = w + static_cast<size_t>(n) * K;
  float s = 0.f;
  for (int k = lane; k < K; k += 32) s += x[k] * ldf<T>(wr[k]);
  s = warp_sum(s);
  if (lane == 0) {
    if (b) s += ldf<T>(b[n]);
    if (act == ACT_TANH) s = tanhf(s);
    else if (act == ACT_RELU) s = fmaxf(s, 0.f);
    else if (act == ACT_GELU) {
      const float u = 0.7978845608028654f * (s + 0.044715f * s * s * s);
      s = 0.5f * s * (1.0f + tanhf(u));
    }
    out[static_cast<size_t>(r) * N + n] = s;
  }
}

// ------------------------------------------------------------------ mixture of experts
constexpr int kMoeMaxExperts = 64, kMoeMaxTopK = 8;

template <class T>
__global__ void __launch_bounds__(256)
moe_route_kernel(const T* __restrict__ logits, int ld, int T_, int E, int k, int* __restrict__ topk_e,
                 float* __restrict__ topk_w, int* __restrict__ pos, int* __restrict__ counts) {
  ptx::grid_dependency_sync();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T_) return;
  float pr[kMoeMaxExperts];
  float mx = -INFINITY;
  for (int e = 0; e < E; ++e) {
    pr[e] = ldf<T>(logits[static_cast<size_t>(t) * ld + e]);
    mx = fmaxf(mx, pr[e]);
  }
  float sum = 0.f;
  for (int e = 0; e < E; ++e) {
    pr[e] = expf(pr[e] - mx);
    sum += pr[e];
  }
  const float inv = 1.0f / sum;
  for (int s = 0; s < k; ++s) {
    int best = 0;
    float bv = -1.f;
    for (int e = 0; e < E; ++e) {
      if (pr[e] > bv) {
        bv = pr[e];
        best = e;
      }
    }
    pr[best] = -2.f;  // taken
    topk_e[t * k + s] = best;
    topk_w[t * k + s] = ldf<T>(stf<T>(bv * inv));  // the reference casts the weights to the model dtype
    pos[t * k + s] = atomicAdd(&counts[best], 1);
  }
}

template <class T>
__global__ void __launch_bounds__(256)
moe_gather_kernel(const T* __restrict__ x, const int* __restrict__ topk_e, const int* __restrict__ pos,
                  T* __restrict__ xg, int n_picks, int k, int H, long long cap) {
  ptx::grid_dependency_sync();
  const int lane = threadIdx.x & 31;
  const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= n_picks) return;
  const T* src = x + static_cast<size_t>(w / k) * H;
  T* dst = xg + (static_cast<size_t>(topk_e[w]) * cap + pos[w]) * H;
  for (int ch = lane; ch < (H >> 3); ch += 32) {
    *reinterpret_cast<uint4*>(dst + ch * 8) = ld16(src + ch * 8);
  }
}

template <class T>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const T* __restrict__ yg, const int* __restrict__ topk_e, const float* __restrict__ topk_w,
                   const int* __restrict__ pos, const T* __restrict__ bias, T* __restrict__ out, int T_,
                   int k, int H, long long cap) {
  ptx::grid_dependency_sync();
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T_) return;
  for (int ch = lane; ch < (H >> 3); ch += 32) {
    float acc[8];
    if (bias) {
      unpack8<T>(ld16(bias + ch * 8), acc);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    }
    for (int s = 0; s < k; ++s) {
      const int p = t * k + s;
      float v[8];
      unpack8<T>(ld16(yg + (static_cast<size_t>(topk_e[p]) * cap + pos[p]) * H + ch * 8), v);
      const float w = topk_w[p];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += w * v[i];
    }
    *reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H + ch * 8) = pack8<T>(acc);
  }
}

template <class S, class D>
__global__ void __launch_bounds__(256) convert_kernel(const S* __restrict__ src, D* __restrict__ dst, size_t n) {
  ptx::grid_dependency_sync();
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    float v;
    if constexpr (sizeof(S) == 4) v = src[i];
    else v = ldf<S>(src[i]);
    if constexpr (sizeof(D) == 4) dst[i] = v;
    else dst[i] = stf<D>(v);
  }
}

inline int last_error() { return static_cast<int>(cudaGetLastError()); }

template <class S>
int convert_from(const void* src, void* dst, int dst_kind, size_t n, cudaStream_t st) {
  const size_t want = (n + 255) / 256;
  const unsigned grid = static_cast<unsigned>(want < 4096 ? (want ? want : 1) : 4096);
  const S* s = reinterpret_cast<const S*>(src);
  if (dst_kind == DT_F16) launch_dependent(convert_kernel<S, __half>, dim3(grid), dim3(256), 0, st, s, reinterpret_cast<__half*>(dst), n);
  else if (dst_kind == DT_BF16) launch_dependent(convert_kernel<S, __nv_bfloat16>, dim3(grid), dim3(256), 0, st, s, reinterpret_cast<__nv_bfloat16*>(dst), n);
  else if (dst_kind == 2) launch_dependent(convert_kernel<S, float>, dim3(grid), dim3(256), 0, st, s, reinterpret_cast<float*>(dst), n);
  else return static_cast<int>(cudaErrorInvalidValue);
  return last_error();
}

template <class T>
int embed_typed(const EmbedArgs& e, cudaStream_t st) {
  const int warps = 8;
  const int grid = (e.T + warps - 1) / warps;
  const int n_chunks = e.H / 8;
#define TEI_EMBED(MAXC)                                                                          \
  launch_dependent(embed_ln_kernel<T, MAXC>, dim3(grid), dim3(warps * 32), 0, st,                                          \
      e.ids, e.type_ids, e.pos_ids, reinterpret_cast<const T*>(e.word),                          \
      reinterpret_cast<const T*>(e.type_tab), reinterpret_cast<const T*>(e.pos_tab),             \
      reinterpret_cast<const T*>(e.gamma), reinterpret_cast<const T*>(e.beta),                   \
      reinterpret_cast<T*>(e.out), e.T, e.H, e.eps)
  if (n_chunks <= 32 * 3) TEI_EMBED(3);
  else if (n_chunks <= 32 * 4) TEI_EMBED(4);
  else if (n_chunks <= 32 * 8) TEI_EMBED(8);
  else TEI_EMBED(16);
#undef TEI_EMBED
  return last_error();
}

template <class T, bool RMS, bool F32RES>
int norm_typed(const NormArgs& n, cudaStream_t st) {
  const int warps = 8;
  const int grid = (n.T + warps - 1) / warps;
  const int n_chunks = n.H / 8;
#define TEI_NORM(MAXC)                                                                           \
  launch_dependent(add_norm_kernel<T, MAXC, RMS, F32RES>, dim3(grid), dim3(warps * 32), 0, st,                                     \
      reinterpret_cast<const T*>(n.x), n.residual, reinterpret_cast<const T*>(n.gamma),          \
      reinterpret_cast<const T*>(n.beta), reinterpret_cast<T*>(n.out),                           \
      reinterpret_cast<float*>(n.sum_out), n.T, n.H, n.eps)
  if (n_chunks <= 32 * 3) TEI_NORM(3);
  else if (n_chunks <= 32 * 4) TEI_NORM(4);
  else if (n_chunks <= 32 * 8) TEI_NORM(8);
  else TEI_NORM(16);
#undef TEI_NORM
  return last_error();
}

}  // namespace

int launch_embed_layernorm(const EmbedArgs& e, cudaStream_t st) {
  if (e.T <= 0) return 0;
  if (e.H % 8 != 0 || e.H > 4096) return static_cast<int>(cudaErrorInvalidValue);
  return e.dtype == DT_F16 ? embed_typed<__half>(e, st) : embed_typed<__nv_bfloat16>(e, st);
}

int launch_add_norm(const NormArgs& n, cudaStream_t st) {
  if (n.T <= 0) return 0;
  if (n.H % 8 != 0 || n.H > 4096) return static_cast<int>(cudaErrorInvalidValue);
  const bool f32res = n.residual_f32 < 0 ? n.rms != 0 : n.residual_f32 != 0;
  if (n.rms && !f32res) return static_cast<int>(cudaErrorInvalidValue);
  if (n.dtype == DT_F16) {
    if (n.rms) return norm_typed<__half, true, true>(n, st);
    return f32res ? norm_typed<__half, false, true>(n, st) : norm_typed<__half, false, false>(n, st);
  }
  if (n.rms) return norm_typed<__nv_bfloat16, true, true>(n, st);
  return f32res ? norm_typed<__nv_bfloat16, false, true>(n, st) : norm_typed<__nv_bfloat16, false, false>(n, st);
}

int launch_layernorm_rows_f32(float* x, const void* gamma, int rows, int H, float eps, int dtype,
                              cudaStream_t st) {
  if (rows <= 0) return 0;
  const int warps = 8;
  const int grid = (rows + warps - 1) / warps;
  if (dtype == DT_F16) {
    launch_dependent(layernorm_rows_f32_kernel<__half>, dim3(grid), dim3(warps * 32), 0, st, x, reinterpret_cast<const __half*>(gamma), rows, H, eps);
  } else {
    launch_dependent(layernorm_rows_f32_kernel<__nv_bfloat16>, dim3(grid), dim3(warps * 32), 0, st, 
        x, reinterpret_cast<const __nv_bfloat16*>(gamma), rows, H, eps);
  }
  return last_error();
}

// One row per sequence, the first (last = 0) or the last (last = 1): gather
// (dst[b] = src[row_b]) or scatter (dst[row_b] = src[b]), 16 bytes per thread.
__global__ void __launch_bounds__(256) first_rows_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                                         const int* __restrict__ cu, int B, int vec_per_row,
                                                         int scatter, int last) {
  ptx::grid_dependency_sync();
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<long long>(B) * vec_per_row) return;
  const int b = static_cast<int>(i / vec_per_row), v = static_cast<int>(i % vec_per_row);
  const size_t packed = static_cast<size_t>(b) * vec_per_row + v;
  const size_t in_batch = static_cast<size_t>(last ? cu[b + 1] - 1 : cu[b]) * vec_per_row + v;
  if (scatter) dst[in_batch] = src[packed];
  else dst[packed] = src[in_batch];
}

int launch_first_rows(const void* src, void* dst, const int* cu_seqlens, int B, int row_bytes, int scatter,
                      int last, cudaStream_t st) {
  if (B <= 0) return 0;
  if (row_bytes % 16 != 0) return static_cast<int>(cudaErrorInvalidValue);
  const long long n = static_cast<long long>(B) * (row_bytes / 16);
  launch_dependent(first_rows_kernel, dim3(static_cast<unsigned>((n + 255) / 256)), dim3(256), 0, st, 
      static_cast<const uint4*>(src), static_cast<uint4*>(dst), cu_seqlens, B, row_bytes / 16, scatter, last);
  return last_error();
}

int launch_layernorm_qk(void* q, void* k, int ld, const void* gq, const void* bq, const void* gk,
                        const void* bk, int T, int H, float eps, int dtype, cudaStream_t st) {
  if (T <= 0) return 0;
  const int warps = 8;
  const int grid = (2 * T + warps - 1) / warps;
  if (dtype == DT_F16) {
    using X = __half;
    launch_dependent(layernorm_qk_kernel<X>, dim3(grid), dim3(warps * 32), 0, st, 
        static_cast<X*>(q), static_cast<X*>(k), ld, static_cast<const X*>(gq), static_cast<const X*>(bq),
        static_cast<const X*>(gk), static_cast<const X*>(bk), T, H, eps);
  } else {
    using X = __nv_bfloat16;
    launch_dependent(layernorm_qk_kernel<X>, dim3(grid), dim3(warps * 32), 0, st, 
        static_cast<X*>(q), static_cast<X*>(k), ld, static_cast<const X*>(gq), static_cast<const X*>(bq),
        static_cast<const X*>(gk), static_cast<const X*>(bk), T, H, eps);
  }
  return last_error();
}

int launch_qk_norm_rope(const RopeArgs& r, cudaStream_t st) {
  if (r.T <= 0) return 0;
  if (r.head_dim % 2 != 0 || r.head_dim > 256) return static_cast<int>(cudaErrorInvalidValue);
  const long long warps_total = static_cast<long long>(r.T) * (r.n_heads + r.n_kv_heads);
  const bool aligned = r.ld_q % 8 == 0 && r.ld_k % 8 == 0 &&
                       (reinterpret_cast<uintptr_t>(r.q) & 15) == 0 && (reinterpret_cast<uintptr_t>(r.k) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(r.q_gamma) & 15) == 0 && (reinterpret_cast<uintptr_t>(r.k_gamma) & 15) == 0;
  if (aligned && (r.head_dim == 32 || r.head_dim == 64 || r.head_dim == 128)) {
    const long long threads = warps_total * (r.head_dim / 16);
    const unsigned grid_v = static_cast<unsigned>((threads + 255) / 256);
#define TEI_ROPE_VEC(TYPE, DH)                                                                     \
  launch_dependent(qk_norm_rope_vec_kernel<TYPE, DH>, dim3(grid_v), dim3(256), 0, st,                                        \
      reinterpret_cast<TYPE*>(r.q), reinterpret_cast<TYPE*>(r.k), r.pos_ids, r.cos_tab, r.sin_tab, \
      reinterpret_cast<const TYPE*>(r.q_gamma), reinterpret_cast<const TYPE*>(r.k_gamma), r.T,     \
      r.n_heads, r.n_kv_heads, r.ld_q, r.ld_k, r.eps)
    if (r.dtype == DT_F16) {
      if (r.head_dim == 32) TEI_ROPE_VEC(__half, 32);
      else if (r.head_dim == 64) TEI_ROPE_VEC(__half, 64);
      else TEI_ROPE_VEC(__half, 128);
    } else {
      if (r.head_dim == 32) TEI_ROPE_VEC(__nv_bfloat16, 32);
      else if (r.head_dim == 64) TEI_ROPE_VEC(__nv_bfloat16, 64);
      else TEI_ROPE_VEC(__nv_bfloat16, 128);
    }
#undef TEI_ROPE_VEC
    return last_error();
  }
  const int warps = 8;
  const long long grid = (warps_total + warps - 1) / warps;
  if (r.dtype == DT_F16) {
    launch_dependent(qk_norm_rope_kernel<__half>, dim3(static_cast<unsigned>(grid)), dim3(warps * 32), 0, st, 
        reinterpret_cast<__half*>(r.q), reinterpret_cast<__half*>(r.k), r.pos_ids, r.cos_tab,
        r.sin_tab, reinterpret_cast<const __half*>(r.q_gamma),
        reinterpret_cast<const __half*>(r.k_gamma), r.T, r.n_heads, r.n_kv_heads, r.head_dim,
        r.ld_q, r.ld_k, r.eps);
  } else {
    launch_dependent(qk_norm_rope_kernel<__nv_bfloat16>, dim3(static_cast<unsigned>(grid)), dim3(warps * 32), 0, st, 
        reinterpret_cast<__nv_bfloat16*>(r.q), reinterpret_cast<__nv_bfloat16*>(r.k), r.pos_ids,
        r.cos_tab, r.sin_tab, reinterpret_cast<const __nv_bfloat16*>(r.q_gamma),
        reinterpret_cast<const __nv_bfloat16*>(r.k_gamma), r.T, r.n_heads, r.n_kv_heads,
        r.head_dim, r.ld_q, r.ld_k, r.eps);
  }
  return last_error();
}

int launch_pool(const PoolArgs& p, cudaStream_t st) {
  if (p.n_out <= 0) return 0;
  if (p.H % 8 != 0) return static_cast<int>(cudaErrorInvalidValue);
  dim3 grid(p.n_out, (p.H + 255) / 256);
  if (p.dtype == DT_F16) {
    launch_dependent(pool_kernel<__half>, dim3(grid), dim3(256), 0, st, reinterpret_cast<const __half*>(p.x), p.cu_seqlens,
                                              p.seq_index, p.out, p.H, p.mode);
  } else {
    launch_dependent(pool_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, st, reinterpret_cast<const __nv_bfloat16*>(p.x),
                                                     p.cu_seqlens, p.seq_index, p.out, p.H,
                                                     p.mode);
  }
  int rc = last_error();
  if (rc) return rc;
  if (p.normalize) {
    const int warps = 8;
    launch_dependent(l2_normalise_kernel, dim3((p.n_out + warps - 1) / warps), dim3(warps * 32), 0, st, p.out, p.n_out, p.H);
    rc = last_error();
  }
  return rc;
}

int launch_l2_normalise(float* x, int rows, int H, cudaStream_t st) {
  if (rows <= 0) return 0;
  const int warps = 8;
  launch_dependent(l2_normalise_kernel, dim3((rows + warps - 1) / warps), dim3(warps * 32), 0, st, x, rows, H);
  return last_error();
}

int launch_gather_rows_f32(const void* x, const int* row_index, float* out, int n_rows, int H,
                           int dtype, cudaStream_t st) {
  if (n_rows <= 0) return 0;
  if (H % 8 != 0) return static_cast<int>(cudaErrorInvalidValue);
  const int warps = 8;
  const int grid = (n_rows + warps - 1) / warps;
  if (dtype == DT_F16) {
    launch_dependent(gather_rows_kernel<__half>, dim3(grid), dim3(warps * 32), 0, st, reinterpret_cast<const __half*>(x),
                                                            row_index, out, n_rows, H);
  } else {
    launch_dependent(gather_rows_kernel<__nv_bfloat16>, dim3(grid), dim3(warps * 32), 0, st, 
        reinterpret_cast<const __nv_bfloat16*>(x), row_index, out, n_rows, H);
  }
  return last_error();
}

int launch_moe_route(const void* logits, int ld_logits, int T, int E, int k, int* topk_e, float* topk_w,
                     int* pos, int* counts, int dtype, cudaStream_t st) {
  if (T <= 0) return 0;
  if (E <= 0 || E > kMoeMaxExperts || k <= 0 || k > kMoeMaxTopK || k > E) return static_cast<int>(cudaErrorInvalidValue);
  const int grid = (T + 255) / 256;
  if (dtype == DT_F16) {
    launch_dependent(moe_route_kernel<__half>, dim3(grid), dim3(256), 0, st, reinterpret_cast<const __half*>(logits), ld_logits, T, E, k,
                                                  topk_e, topk_w, pos, counts);
  } else {
    launch_dependent(moe_route_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, st, reinterpret_cast<const __nv_bfloat16*>(logits),
                                                         ld_logits, T, E, k, topk_e, topk_w, pos, counts);
  }
  return last_error();
}

int launch_moe_gather(const void* x, const int* topk_e, const int* pos, void* xg, int T, int k, int H,
                      long long cap, int dtype, cudaStream_t st) {
  if (T <= 0) return 0;
  if (H % 8 != 0) return static_cast<int>(cudaErrorInvalidValue);
  const int n = T * k, warps = 8;
  const int grid = (n + warps - 1) / warps;
  if (dtype == DT_F16) {
    launch_dependent(moe_gather_kernel<__half>, dim3(grid), dim3(warps * 32), 0, st, reinterpret_cast<const __half*>(x), topk_e, pos,
                                                           reinterpret_cast<__half*>(xg), n, k, H, cap);
  } else {
    launch_dependent(moe_gather_kernel<__nv_bfloat16>, dim3(grid), dim3(warps * 32), 0, st, 
        reinterpret_cast<const __nv_bfloat16*>(x), topk_e, pos, reinterpret_cast<__nv_bfloat16*>(xg), n, k, H, cap);
  }
  return last_error();
}

int launch_moe_combine(const void* yg, const int* topk_e, const float* topk_w, const int* pos,
                       const void* bias, void* out, int T, int k, int H, long long cap, int dtype,
                       cudaStream_t st) {
  if (T <= 0) return 0;
  if (H % 8 != 0) return static_cast<int>(cudaErrorInvalidValue);
  const int warps = 8;
  const int grid = (T + warps - 1) / warps;
  if (dtype == DT_F16) {
    launch_dependent(moe_combine_kernel<__half>, dim3(grid), dim3(warps * 32), 0, st, 
        reinterpret_cast<const __half*>(yg), topk_e, topk_w, pos, reinterpret_cast<const __half*>(bias),
        reinterpret_cast<__half*>(out), T, k, H, cap);
  } else {
    launch_dependent(moe_combine_kernel<__nv_bfloat16>, dim3(grid), dim3(warps * 32), 0, st, 
        reinterpret_cast<const __nv_bfloat16*>(yg), topk_e, topk_w, pos,
        reinterpret_cast<const __nv_bfloat16*>(bias), reinterpret_cast<__nv_bfloat16*>(out), T, k, H, cap);
  }
  return last_error();
}

int launch_convert(const void* src, int src_kind, void* dst, int dst_kind, size_t n,
                   cudaStream_t st) {
  if (n == 0) return 0;
  if (src_kind == 0) return convert_from<float>(src, dst, dst_kind, n, st);
  if (src_kind == 1) return convert_from<__half>(src, dst, dst_kind, n, st);
  if (src_kind == 2) return convert_from<__nv_bfloat16>(src, dst, dst_kind, n, st);
  return static_cast<int>(cudaErrorInvalidValue);
}

int launch_head_linear(const float* in, const void* w, const void* b, float* out, int rows, int N,
                       int K, int act, int dtype, cudaStream_t st) {
  if (rows <= 0 || N <= 0) return 0;
  const long long total = static_cast<long long>(rows) * N;
  const int warps = 8;
  const long long grid = (total + warps - 1) / warps;
  if (dtype == DT_F16) {
    launch_dependent(head_linear_kernel<__half>, dim3(static_cast<unsigned>(grid)), dim3(warps * 32), 0, st, 
        in, reinterpret_cast<const __half*>(w), reinterpret_cast<const __half*>(b), out, rows, N, K,
        act);
  } else {
    launch_dependent(head_linear_kernel<__nv_bfloat16>, dim3(static_cast<unsigned>(grid)), dim3(warps * 32), 0, st, 
        in, reinterpret_cast<const __nv_bfloat16*>(w), reinterpret_cast<const __nv_bfloat16*>(b),
        out, rows, N, K, act);
  }
  return last_error();
}

}  // namespace tei
