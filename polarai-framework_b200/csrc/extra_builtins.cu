// The remaining operation builtins of the catalogue
// (include/polarai/core/internal/GenBuiltins.hpp:25-52 of the reference): frelu,
// fsoftmax, fpool, fconv2d, ftranspose, fslice.  None of them is on the benchmarked path; they are here so
// that any graph the reference's operations can express runs on this runtime.  Small
// 2-D single-channel problems: one thread per output element.
#include "common.cuh"

namespace polar_b200 {
namespace {

constexpr int kThreads = 256;

__global__ void __launch_bounds__(kThreads) relu_kernel(const float* in, float* out, uint64_t n) {
  const uint64_t stride = (uint64_t)gridDim.x * kThreads;
  for (uint64_t i = (uint64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) {
    float v = in[i];
    out[i] = v > 0.0f ? v : 0.0f;   // ordered compare: NaN gives 0, as the reference's select does
  }
}

// total += sum of expf(in[i]) (double accumulation; one atomic per block)
__global__ void __launch_bounds__(kThreads) exp_sum_kernel(const float* in, double* total, uint64_t n) {
  double acc = 0.0;
  const uint64_t stride = (uint64_t)gridDim.x * kThreads;
  for (uint64_t i = (uint64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) acc += (double)expf(in[i]);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  __shared__ double warp_sums[kThreads / 32];
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double s = 0.0;
    for (int w = 0; w < kThreads / 32; ++w) s += warp_sums[w];
    atomicAdd(total, s);
  }
}

__global__ void __launch_bounds__(kThreads) softmax_div_kernel(const float* in, const double* total, float* out,
                                                               uint64_t n) {
  const float t = (float)*total;
  const uint64_t stride = (uint64_t)gridDim.x * kThreads;
  for (uint64_t i = (uint64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride)
    out[i] = __fdiv_rn(expf(in[i]), t);
}

__global__ void __launch_bounds__(kThreads) pool_kernel(const float* in, uint64_t h, uint64_t w, uint64_t wh,
                                                        uint64_t ww, uint64_t sh, uint64_t sw, float* out,
                                                        uint64_t oh, uint64_t ow) {
  const uint64_t e = (uint64_t)blockIdx.x * kThreads + threadIdx.x;
  if (e >= oh * ow) return;
  const uint64_t i = e / ow, j = e % ow;
  float best = -10e5f;
  for (uint64_t a = 0; a < wh; ++a)
    for (uint64_t b = 0; b < ww; ++b) {
      float v = in[(i * sh + a) * w + j * sw + b];
      best = v > best ? v : best;
    }
  out[e] = best;
}

__global__ void __launch_bounds__(kThreads) conv2d_kernel(const float* in, uint64_t h, uint64_t w, const float* ker,
                                                          uint64_t kh, uint64_t kw, float* out, uint64_t oh,
                                                          uint64_t ow) {
  const uint64_t e = (uint64_t)blockIdx.x * kThreads + threadIdx.x;
  if (e >= oh * ow) return;
  const uint64_t i = e / ow, j = e % ow;
  float acc = 0.0f;
  for (uint64_t a = 0; a < kh; ++a)
    for (uint64_t b = 0; b < kw; ++b)
      acc = __fadd_rn(__fmul_rn(in[(i + a) * w + j + b], ker[a * kw + b]), acc);   // product rounded, then added
  out[e] = acc;
}

// out[c, r] = in[r, c] through a 32 x 33 shared-memory tile: both the reads and the writes
// are coalesced rows of 32 floats.  One tile per CTA (32 x 8 threads, four rows each).
constexpr int kTile = 32;
__global__ void __launch_bounds__(kTile * 8) transpose_kernel(const float* __restrict__ in, float* __restrict__ out,
                                                              uint64_t rows, uint64_t cols, uint32_t tiles_c) {
  __shared__ float tile[kTile][kTile + 1];
  const uint64_t tr = blockIdx.x / tiles_c, tc = blockIdx.x % tiles_c;
  const uint64_t r0 = tr * kTile, c0 = tc * kTile;
  for (int j = threadIdx.y; j < kTile; j += 8) {
    const uint64_t r = r0 + j, c = c0 + threadIdx.x;
    if (r < rows && c < cols) tile[j][threadIdx.x] = in[r * cols + c];
  }
  __syncthreads();
  for (int j = threadIdx.y; j < kTile; j += 8) {
    const uint64_t c = c0 + j, r = r0 + threadIdx.x;      // out is [cols, rows]
    if (c < cols && r < rows) out[c * rows + r] = tile[threadIdx.x][j];
  }
}

unsigned blocks_for(uint64_t n) {
  uint64_t need = (n + kThreads - 1) / kThreads;
  uint64_t cap = (uint64_t)sm_count() * 8;
  if (need < 1) need = 1;
  return (unsigned)(need < cap ? need : cap);
}

}  // namespace
}  // namespace polar_b200

using namespace polar_b200;

extern "C" {

int polar_b200_frelu(const float* in, float* out, uint64_t n, void* stream) {
  clear_error();
  if (n == 0) return POLAR_B200_OK;
  if (!in || !out) return fail(POLAR_B200_ERR_INVALID, "null device pointer");
  LaunchDeviceScope on(stream, out);
  relu_kernel<<<blocks_for(n), kThreads, 0, as_stream(stream)>>>(in, out, n);
  return check_launch("frelu");
}

int polar_b200_fsoftmax(const float* in, float* out, uint64_t n, void* workspace, uint64_t workspace_bytes,
                        void* stream) {
  clear_error();
  if (n == 0) return POLAR_B200_OK;
  if (!in || !out) return fail(POLAR_B200_ERR_INVALID, "null device pointer");
  LaunchDeviceScope on(stream, out);
  cudaStream_t st = as_stream(stream);
  double* total = static_cast<double*>(workspace);
  bool own = false;
  if (!total) {
    cudaError_t e = cudaMallocAsync(reinterpret_cast<void**>(&total), sizeof(double), st);
    if (e != cudaSuccess) return fail(POLAR_B200_ERR_CUDA, "cudaMallocAsync(softmax total)", e);
    own = true;
  } else if (workspace_bytes < sizeof(double) || (reinterpret_cast<uintptr_t>(workspace) & 7)) {
    return fail(POLAR_B200_ERR_WORKSPACE, "fsoftmax needs 8 bytes of 8-byte aligned workspace");
  }
  cudaError_t e = cudaMemsetAsync(total, 0, sizeof(double), st);
  if (e != cudaSuccess) return fail(POLAR_B200_ERR_CUDA, "cudaMemsetAsync", e);
  exp_sum_kernel<<<blocks_for(n), kThreads, 0, st>>>(in, total, n);
  int rc = check_launch("fsoftmax_sum");
  if (rc == POLAR_B200_OK) {
    softmax_div_kernel<<<blocks_for(n), kThreads, 0, st>>>(in, total, out, n);
    rc = check_launch("fsoftmax");
  }
  if (own) cudaFreeAsync(total, st);
  return rc;
}

int polar_b200_fpool(const float* in, uint64_t h, uint64_t w, uint64_t windowH, uint64_t windowW, uint64_t strideH,
                     uint64_t strideW, float* out, void* stream) {
  clear_error();
  if (windowH == 0 || windowW == 0 || strideH == 0 || strideW == 0 || windowH > h || windowW > w)
    return fail(POLAR_B200_ERR_INVALID, "fpool: window and stride must be positive and fit the input");
  const uint64_t oh = (h - windowH) / strideH + 1, ow = (w - windowW) / strideW + 1;
  if (!in || !out) return fail(POLAR_B200_ERR_INVALID, "null device pointer");
  LaunchDeviceScope on(stream, out);
  pool_kernel<<<(unsigned)((oh * ow + kThreads - 1) / kThreads), kThreads, 0, as_stream(stream)>>>(
      in, h, w, windowH, windowW, strideH, strideW, out, oh, ow);
  return check_launch("fpool");
}

int polar_b200_fconv2d(const float* in, uint64_t h, uint64_t w, const float* kernel, uint64_t kh, uint64_t kw,
                       float* out, void* stream) {
  clear_error();
  if (kh == 0 || kw == 0 || kh > h || kw > w) return fail(POLAR_B200_ERR_INVALID, "fconv2d: kernel must fit the input");
  // The reference walks offsets -k/2 .. k/2, which is the kernel only when k is odd.
  if ((kh & 1) == 0 || (kw & 1) == 0) return fail(POLAR_B200_ERR_UNSUPPORTED, "fconv2d: kernel extents must be odd");
  if (!in || !kernel || !out) return fail(POLAR_B200_ERR_INVALID, "null device pointer");
  const uint64_t oh = h - kh + 1, ow = w - kw + 1;
  LaunchDeviceScope on(stream, out);
  conv2d_kernel<<<(unsigned)((oh * ow + kThreads - 1) / kThreads), kThreads, 0, as_stream(stream)>>>(
      in, h, w, kernel, kh, kw, out, oh, ow);
  return check_launch("fconv2d");
}

int polar_b200_ftranspose(const float* in, uint64_t rows, uint64_t cols, float* out, void* stream) {
  clear_error();
  if (rows == 0 || cols == 0) return POLAR_B200_OK;
  if (!in || !out) return fail(POLAR_B200_ERR_INVALID, "null device pointer");
  if (in == out) return fail(POLAR_B200_ERR_INVALID, "ftranspose cannot run in place");
  const uint64_t tiles_r = (rows + kTile - 1) / kTile, tiles_c = (cols + kTile - 1) / kTile;
  if (tiles_r * tiles_c > 0x7fffffffull) return fail(POLAR_B200_ERR_INVALID, "matrix too large");
  LaunchDeviceScope on(stream, out);
  transpose_kernel<<<(unsigned)(tiles_r * tiles_c), dim3(kTile, 8), 0, as_stream(stream)>>>(in, out, rows, cols,
                                                                                         (uint32_t)tiles_c);
  return check_launch("ftranspose");
}

int polar_b200_fslice(const float* in, uint64_t first_dim, uint64_t inner, uint64_t index, float* out, void* stream) {
  clear_error();
  if (index >= first_dim) return fail(POLAR_B200_ERR_INVALID, "fslice: index outside the first dimension");
  if (inner && !in) return fail(POLAR_B200_ERR_INVALID, "null device pointer");
  return polar_b200_fcopy(in + index * inner, out, inner, stream);   // a bit-exact copy of one sub-tensor
}

}  // extern "C"
