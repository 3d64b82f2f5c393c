// Host helpers shared by the kernel launchers: TMA tensor-map encoding through the driver entry
// point (looked up at run time so the library links against the CUDA runtime only) and cached
// per-device properties.
#pragma once
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

#include <utility>

namespace tei {

// Encodes a 2-D row-major tensor map with zero fill outside the tensor; the swizzle span is the
// box row (128 or 64 bytes).
//   inner / outer: extent in elements of the contiguous dimension / number of rows;
//   row_stride_bytes: distance between rows (multiple of 16);
//   box_inner * elem_bytes must be 128 or 64 (one swizzle row); box_outer <= 256.
// Returns 0 or a non-zero error code (CUresult or cudaError_t value).
int make_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int elem_bytes,
                 uint64_t inner, uint64_t outer, uint64_t row_stride_bytes, uint32_t box_inner,
                 uint32_t box_outer);

// Launches a kernel that begins with ptx::grid_dependency_sync() with programmatic stream
// serialisation allowed: it may start while its predecessor in the stream drains and waits for
// it on the device.
template <class... P, class... A>
inline cudaError_t launch_dependent(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    A&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
#ifdef TEI_NO_PDL
  attr[0].val.programmaticStreamSerializationAllowed = 0;
#else
  attr[0].val.programmaticStreamSerializationAllowed = 1;
#endif
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<P>(args)...);
}

// Number of SMs of the current device (cached).
int num_sms();
// Index of the current device.
int current_device();

}  // namespace tei
