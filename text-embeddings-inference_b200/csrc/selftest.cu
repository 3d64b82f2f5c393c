// The failure path of the bounded waits, made to run without a failure: what a kernel does when
// a wait runs out (write a DEV_TIMEOUT_* code to the status word and return), and what the host
// makes of it (TIMEOUT -> BackendError::Inference, the handle unhealthy until a probe passes,
// backends/src/lib.rs:393-409,621-642).  Nothing here spins, traps or faults.
#include "kernels.h"
#include "ptx.cuh"

namespace tei {
namespace {

// Stands in for a kernel whose wait ran out: it only reports.
__global__ void report_status_kernel(int* status, int code) {
  if (threadIdx.x == 0 && blockIdx.x == 0) atomicExch(status, code);
}

// One CTA waits on an mbarrier that nobody arrives at, with the same wait primitive the GEMM and
// attention kernels use but a limit of a few hundred probes; the wait gives up, the thread
// reports and the kernel returns.  polls_out receives 1 when the wait gave up, 0 when it (wrongly)
// saw the barrier complete.
__global__ void __launch_bounds__(32) bounded_wait_probe_kernel(int* status, uint32_t limit, int* gave_up) {
  __shared__ __align__(8) uint64_t bar;
  if (threadIdx.x == 0) {
    ptx::mbar_init(&bar, 1);
    ptx::fence_mbar_init();
  }
  __syncwarp();
  if (threadIdx.x == 0) {
    const bool ok = ptx::mbar_wait_limit(&bar, 0, limit);
    if (!ok) atomicExch(status, DEV_TIMEOUT_PRODUCER);
    if (gave_up) *gave_up = ok ? 0 : 1;
  }
}

}  // namespace

int launch_report_status(int* status, int code, cudaStream_t stream) {
  if (status == nullptr) return static_cast<int>(cudaErrorInvalidValue);
  report_status_kernel<<<1, 32, 0, stream>>>(status, code);
  return static_cast<int>(cudaGetLastError());
}

int launch_bounded_wait_probe(int* status, int limit, int* gave_up, cudaStream_t stream) {
  // The limit is capped: this is a probe of the give-up path, not a way to keep a GPU busy.
  if (status == nullptr || limit < 1 || limit > 4096) return static_cast<int>(cudaErrorInvalidValue);
  bounded_wait_probe_kernel<<<1, 32, 0, stream>>>(status, static_cast<uint32_t>(limit), gave_up);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace tei
