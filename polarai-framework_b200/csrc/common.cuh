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

#ifdef __CUDACC__
// fsigmoid's arithmetic, shared by the elementwise builtin and the fused matmul
// epilogue so that both give the same bits: r = 1/(1+exp(-x)), then the reference's
// clamp to [1e-5, 1-1e-5] (opencl/kernels.h:141-156 of the reference).
__device__ __forceinline__ float sigmoid_clamped(float x) {
  const float eps = 1e-5f;
  // 1/d as the correctly rounded reciprocal: the same bits as IEEE division of 1 by d,
  // without the division's slow-path branch (which keeps independent elements from
  // being interleaved in the matmul epilogue).
  float r = __frcp_rn(__fadd_rn(1.0f, expf(-x)));
  const float hi = __fadd_rn(1.0f, -eps);
  r = (fabsf(__fadd_rn(r, -1.0f)) < eps) ? hi : ((fabsf(r) < eps) ? eps : r);
  return r;
}
// The reference's Sigmoid derivative chain on one element, with its three roundings:
// fadd(ones,1,s,-1) -> fmul(.,s) -> fmul(grad,.)  (SigmoidOperationInternal.cpp:107-135).
__device__ __forceinline__ float sigmoid_grad_chain(float g, float s) {
  float one_minus = __fadd_rn(__fmul_rn(1.0f, 1.0f), __fmul_rn(s, -1.0f));
  return __fmul_rn(g, __fmul_rn(one_minus, s));
}
#endif

}  // namespace polar_b200
