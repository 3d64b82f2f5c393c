// Host helpers shared by the kernel launchers: TMA tensor-map encoding through the driver entry
// point (looked up at run time so the library links against the CUDA runtime only) and cached
// per-device properties.
#pragma once
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

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

// Number of SMs of the current device (cached).
int num_sms();
// Index of the current device.
int current_device();

}  // namespace tei
