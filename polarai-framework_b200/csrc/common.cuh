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

// ---- status words and wait limits of the bounded device-side waits -----------------------
// One status word per device, in pinned host memory every device can write (so the host reads
// it without a CUDA call, even while a kernel is still running).  A kernel whose wait gives
// up stores its code with atomicCAS(word, 0, code): the first code since the last clear stays.
// Returns the device-visible pointer of the CURRENT device's word (nullptr + *rc on failure).
int* device_status_word(int* rc);
int device_status_read(int device);     // device < 0: the first non-zero word of any device
void device_status_clear_all();
// The host's wait bound in nanoseconds, or `fallback` when none was set.
unsigned long long wait_limit_ns(unsigned long long fallback);

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Every launching entry point opens one of these.  A kernel must be launched with the device
// of its stream current; a caller that drives several GPUs from one thread (or a plugin that
// enumerated them) may arrive with another device current.  With a real stream handle the
// stream's own device is made current for the duration of the call; with the NULL (legacy
// default) stream, which every device has, the device that owns `ptr` (one of the call's
// device buffers) decides.  The caller's current device is put back on exit.  Costs two
// runtime queries per launch when nothing needs switching.
class LaunchDeviceScope {
public:
  LaunchDeviceScope(void* stream, const void* ptr) {
    int want = -1, cur = -1;
    if (cudaGetDevice(&cur) != cudaSuccess) {
      cudaGetLastError();
      return;
    }
    if (stream && stream != (void*)cudaStreamLegacy && stream != (void*)cudaStreamPerThread) {
      // A stream under capture is left alone (only the capture-status query is allowed on it
      // without risk to the capture): whoever captures has made the stream's device current.
      cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
      if (cudaStreamIsCapturing(as_stream(stream), &capturing) != cudaSuccess) {
        cudaGetLastError();
        return;
      }
      if (capturing != cudaStreamCaptureStatusNone) return;
      if (cudaStreamGetDevice(as_stream(stream), &want) != cudaSuccess) {
        cudaGetLastError();
        return;
      }
    } else if (ptr) {
      cudaPointerAttributes attr;
      if (cudaPointerGetAttributes(&attr, ptr) != cudaSuccess) {
        cudaGetLastError();
        return;
      }
      if (attr.type != cudaMemoryTypeDevice && attr.type != cudaMemoryTypeManaged) return;
      want = attr.device;
    }
    if (want >= 0 && want != cur && cudaSetDevice(want) == cudaSuccess) {
      prev_ = cur;
      switched_ = true;
    }
  }
  ~LaunchDeviceScope() {
    if (switched_ && cudaSetDevice(prev_) != cudaSuccess) cudaGetLastError();
  }
  LaunchDeviceScope(const LaunchDeviceScope&) = delete;
  LaunchDeviceScope& operator=(const LaunchDeviceScope&) = delete;

private:
  int prev_ = -1;
  bool switched_ = false;
};

#ifdef __CUDACC__
// fsigmoid's arithmetic, shared by the elementwise builtin and the fused matmul
// epilogue so that both give the same bits: r = 1/(1+exp(-x)), then the reference's
// clamp to [1e-5, 1-1e-5] (opencl/kernels.h:141-156 of the reference).
__device__ __forceinline__ float sigmoid_clamped(float x) {
  // Six instructions, two of them on the special-function unit: ex2.approx of -x * log2 e, 1 + e,
  // rcp.approx, and the clamp as one min and one max.  In the tensor-core epilogue, which cannot
  // overlap the next tile's k loop with 256-row tiles, the sigmoid is a large part of the drain,
  // and a dozen instructions per element (IEEE reciprocal, compare-and-select clamp) made the
  // drain issue-bound.
  //  - Error: ex2.approx is good to 2 ulp, the product -x * log2 e adds |x| * 6e-8 relative to the
  //    exponential (at most 8e-7 where it still matters: |x| < 11.6, beyond which the clamp takes
  //    over), rcp.approx 1 ulp: within the 1e-5 the builtin is held to, by a factor 10.
  //  - The clamp: r lies in [0, 1], so the reference's "|r - 1| < eps -> 1 - eps, else |r| < eps
  //    -> eps" is min(r, fl(1 - eps)) followed by max(., eps); the .NaN forms keep a NaN a NaN,
  //    as the reference's comparisons (all false) do.
  const float eps = 1e-5f;
  const float hi = 1.0f - eps;   // folded at compile time, the same float as fadd(1, -eps)
  float d = __fadd_rn(1.0f, __expf(-x)), r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(d));
  asm("min.NaN.f32 %0, %0, %1;" : "+f"(r) : "f"(hi));
  asm("max.NaN.f32 %0, %0, %1;" : "+f"(r) : "f"(eps));
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
