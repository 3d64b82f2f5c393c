#include "tmap.h"

#include <atomic>
#include <cstring>
#include <mutex>
#include <unordered_map>

namespace tei {
namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

std::once_flag g_once;
EncodeTiledFn g_encode = nullptr;

void resolve_encode() {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess) {
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
}

// Encoded maps are kept per thread (a replica is driven by one thread at a time): weights never
// move and the activation buffers only when the workspace grows, so a forward at a batch size
// seen before encodes nothing.  A map depends on nothing but the key's fields; the device it is
// used on is implied by the base address (unified addressing).
struct TmapKey {
  uint64_t base, inner, outer, stride;
  uint32_t dt, box_inner, box_outer, pad;
  bool operator==(const TmapKey& o) const { return std::memcmp(this, &o, sizeof(TmapKey)) == 0; }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    uint64_t h = 0x9E3779B97F4A7C15ull;
    const uint64_t v[6] = {k.base, k.inner, k.outer, k.stride, (static_cast<uint64_t>(k.dt) << 32) | k.box_inner, k.box_outer};
    for (uint64_t x : v) {
      h ^= x + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
    }
    return static_cast<size_t>(h);
  }
};
constexpr size_t kTmapCacheLimit = 8192;  // entries per thread (1.2 MB); cleared when full

constexpr int kMaxDevices = 64;
std::atomic<int> g_sms[kMaxDevices];

}  // namespace

int make_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int elem_bytes,
                 uint64_t inner, uint64_t outer, uint64_t row_stride_bytes, uint32_t box_inner,
                 uint32_t box_outer) {
  std::call_once(g_once, resolve_encode);
  if (!g_encode) return static_cast<int>(cudaErrorNotSupported);
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (row_stride_bytes & 15) ||
      (box_inner * elem_bytes != 128 && box_inner * elem_bytes != 64) || box_outer == 0 || box_outer > 256) {
    return static_cast<int>(cudaErrorInvalidValue);
  }
  // The swizzle span equals the box row: 128-byte rows for head sizes and GEMM tiles of 64
  // elements and more, 64-byte rows for head_dim 32.
  const CUtensorMapSwizzle swz = box_inner * elem_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  thread_local std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  TmapKey key;
  std::memset(&key, 0, sizeof key);
  key.base = reinterpret_cast<uint64_t>(base);
  key.inner = inner;
  key.outer = outer;
  key.stride = row_stride_bytes;
  key.dt = static_cast<uint32_t>(dt);
  key.box_inner = box_inner;
  key.box_outer = box_outer;
  auto hit = cache.find(key);
  if (hit != cache.end()) {
    *out = hit->second;
    return 0;
  }
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_SUCCESS) {
    if (cache.size() >= kTmapCacheLimit) cache.clear();
    cache.emplace(key, *out);
  }
  return static_cast<int>(r);
}

int current_device() {
  int d = 0;
  cudaGetDevice(&d);
  return d;
}

int num_sms() {
  const int d = current_device();
  if (d < 0 || d >= kMaxDevices) return 148;
  int v = g_sms[d].load(std::memory_order_relaxed);
  if (v == 0) {
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, d);
    if (v <= 0) v = 148;
    g_sms[d].store(v, std::memory_order_relaxed);
  }
  return v;
}

}  // namespace tei
