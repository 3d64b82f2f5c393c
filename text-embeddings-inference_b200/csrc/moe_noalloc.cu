// Mixture-of-experts routing for callers that must not allocate device memory.
//
// tei_b200_op_moe_route needs n_experts counters in global memory next to its inputs and
// outputs (one atomic row counter per expert) and takes them from the caller.  Some hosts
// cannot provide that: a serving process that handed the whole GPU to its own arena at
// start-up and treats any later cudaMalloc as a bug (it synchronises the device and can fail
// under pressure in the middle of a request), or a plugin that only ever receives the tensors
// of the operator it implements and has no allocator of its own.  For them this variant keeps
// the counters in an array that is part of the library image: every GPU that loads the library
// holds these 256 bytes until the process exits, and no call here allocates or frees anything.
//
// Consequences of the shared array, all of them the caller's business:
//   * at most kMaxExperts experts; more is refused with an error message;
//   * the array keeps what the previous call left, so every call clears the part it uses first;
//   * two calls that overlap on one GPU (different streams, or the same stream from two
//     threads without ordering) would count into the same counters and corrupt each other:
//     callers serialise them;
//   * the first call on a device looks the array's address up (a host-side symbol is not a
//     device address) and remembers it; make that first call before any stream capture starts.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <mutex>

#include "kernels.h"
#include "../../include/tei_b200_ops.h"

namespace {

constexpr int kMaxExperts = 64;   // also the limit of the routing kernel itself
constexpr int kMaxDevices = 64;

// The counters.  Device code may name the array; host code may only pass the address obtained
// below to a kernel.
static __device__ __align__(256) int g_route_counters[kMaxExperts];

std::mutex g_setup_mutex;
int* g_counters_addr[kMaxDevices] = {};
bool g_counters_known[kMaxDevices] = {};

void set_err(char* err, size_t cap, const char* msg) {
  if (!err || cap == 0) return;
  std::strncpy(err, msg, cap - 1);
  err[cap - 1] = '\0';
}

// Address of the counters on the current device; looked up once per device, with that device
// current (the caller's).  Returns a CUDA error code.
int counters_for_current_device(int** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kMaxDevices) return static_cast<int>(cudaErrorInvalidDevice);
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_counters_known[dev]) {
    int* ptr = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_route_counters);
    if (e != cudaSuccess) return static_cast<int>(e);
    g_counters_addr[dev] = ptr;
    g_counters_known[dev] = true;
  }
  *out = g_counters_addr[dev];
  return 0;
}

}  // namespace

extern "C" int tei_b200_op_moe_route_noalloc(const void* logits_dev, int ld_logits, int n_tokens,
                                             int n_experts, int top_k, int32_t* topk_expert_dev,
                                             float* topk_weight_dev, int32_t* pos_dev,
                                             int32_t* counts_out_dev, int dtype, void* stream,
                                             char* err, size_t err_cap) {
  if (n_experts < 1 || n_experts > kMaxExperts) {
    char msg[160];
    std::snprintf(msg, sizeof(msg),
                  "tei_b200_op_moe_route_noalloc: n_experts = %d, but the built-in counters hold at most %d experts",
                  n_experts, kMaxExperts);
    set_err(err, err_cap, msg);
    return static_cast<int>(cudaErrorInvalidValue);
  }
  if (top_k < 1 || top_k > 8 || top_k > n_experts) {
    set_err(err, err_cap, "tei_b200_op_moe_route_noalloc: top_k must be between 1 and min(8, n_experts)");
    return static_cast<int>(cudaErrorInvalidValue);
  }
  int* counters = nullptr;
  int rc = counters_for_current_device(&counters);
  if (rc) {
    set_err(err, err_cap, "tei_b200_op_moe_route_noalloc: could not look up the counters on this device");
    return rc;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // whatever the last call counted is still there
  cudaError_t e = cudaMemsetAsync(counters, 0, static_cast<size_t>(n_experts) * sizeof(int), st);
  if (e != cudaSuccess) {
    set_err(err, err_cap, cudaGetErrorString(e));
    return static_cast<int>(e);
  }
  rc = tei::launch_moe_route(logits_dev, ld_logits, n_tokens, n_experts, top_k, topk_expert_dev,
                             topk_weight_dev, pos_dev, counters, dtype, st);
  if (rc) {
    set_err(err, err_cap, "tei_b200_op_moe_route_noalloc: the routing kernel refused its arguments");
    return rc;
  }
  if (counts_out_dev) {
    e = cudaMemcpyAsync(counts_out_dev, counters, static_cast<size_t>(n_experts) * sizeof(int),
                        cudaMemcpyDeviceToDevice, st);
    if (e != cudaSuccess) {
      set_err(err, err_cap, cudaGetErrorString(e));
      return static_cast<int>(e);
    }
  }
  return 0;
}
