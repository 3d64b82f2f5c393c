// The arithmetic of per-head RMSNorm + rotary embedding, shared by the standalone kernel
// (rowwise.cu) and the QKV GEMM epilogue (gemm.cu) so that both give the same bits: every
// operation is spelled out with rounding intrinsics (no contraction left to the compiler) and the
// sum of squares is combined in one fixed order.
//
// Reference semantics: per-head RMSNorm of q and k (flash_qwen3.rs:150-151; statistics in fp32,
// layers/rms_norm.rs:40-50), then x * cos + rotate_half(x) * sin on the pairs (j, j + D/2)
// (layers/rotary.rs:118-130), cos / sin from an fp32 table row of the token's position.
#pragma once

namespace tei {
namespace ropemath {

// Sum of squares of 8 elements of the first half of a head and the 8 they pair with.
__device__ __forceinline__ float ss8(const float* a, const float* b) {
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) ss = __fadd_rn(ss, __fmaf_rn(a[i], a[i], __fmul_rn(b[i], b[i])));
  return ss;
}

// The G = D / 16 partial sums of a head combined in the order a xor-shuffle reduction over G
// lanes (offsets G/2 ... 1) gives every lane.
template <int G>
__device__ __forceinline__ float combine(const float* p);
template <>
__device__ __forceinline__ float combine<2>(const float* p) {
  return __fadd_rn(p[0], p[1]);
}
template <>
__device__ __forceinline__ float combine<4>(const float* p) {
  return __fadd_rn(__fadd_rn(p[0], p[2]), __fadd_rn(p[1], p[3]));
}
template <>
__device__ __forceinline__ float combine<8>(const float* p) {
  return __fadd_rn(__fadd_rn(__fadd_rn(p[0], p[4]), __fadd_rn(p[2], p[6])),
                   __fadd_rn(__fadd_rn(p[1], p[5]), __fadd_rn(p[3], p[7])));
}

// 1 / sqrt(mean of squares + eps); D is a power of two, so the division is exact.
__device__ __forceinline__ float rms_scale(float ss, int D, float eps) {
  return rsqrtf(__fmaf_rn(ss, 1.0f / static_cast<float>(D), eps));
}
__device__ __forceinline__ float normed(float x, float r, float gamma) {
  return __fmul_rn(__fmul_rn(x, r), gamma);
}
// (a, b) = (x[j], x[j + D/2]) -> (a cos - b sin, b cos + a sin)
__device__ __forceinline__ float rot_lo(float a, float b, float c, float s) {
  return __fmaf_rn(a, c, -__fmul_rn(b, s));
}
__device__ __forceinline__ float rot_hi(float a, float b, float c, float s) {
  return __fmaf_rn(b, c, __fmul_rn(a, s));
}

}  // namespace ropemath
}  // namespace tei
