// Shared host-side helpers of the kernel library: status recording, launch
// accounting and launch-geometry constants for B200.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/polar_b200.h"

namespace polar_b200 {

// B200: 148 SMs.  Grids of persistent (grid-stride) kernels are sized as a
// multiple of the SM count the device reports.
int sm_count();

// Records `msg` (and the CUDA error text, if any) as the calling thread's last
// error and returns `status`.
int fail(int status, const char* msg, cudaError_t err = cudaSuccess);
void clear_error();
void count_launch(uint64_t n = 1);

// Checks the launch that was just issued.
inline int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(POLAR_B200_ERR_CUDA, what, e);
  count_launch();
  return POLAR_B200_OK;
}

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace polar_b200
