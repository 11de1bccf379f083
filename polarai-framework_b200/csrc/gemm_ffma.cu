// fmatmul on the CUDA cores: one FFMA per term, fp32 accumulate, k ascending for
// every output element.  It is the device-side cross-check of the tensor-core
// path and the fallback for shapes the TMA descriptors cannot express (row
// pitches that are not multiples of 16 bytes).  64x64 output tile per CTA,
// 16-deep k slabs staged in shared memory, 4x4 outputs per thread; all four
// transpose forms through element strides.
#include "common.cuh"

namespace polar_b200 {
namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;
constexpr int kThreads = (BM / TM) * (BN / TN);  // 256

// L'(i,k) = left[i*lsi + k*lsk]; R'(k,j) = right[k*rsk + j*rsj].
__global__ void __launch_bounds__(kThreads)
ffma_kernel(const float* __restrict__ left, const float* __restrict__ right, float* __restrict__ out,
            uint64_t m, uint64_t n, uint64_t k, uint64_t lsi, uint64_t lsk, uint64_t rsk,
            uint64_t rsj) {
  __shared__ float sa[BK][BM + 1];
  __shared__ float sb[BK][BN + 1];
  const uint64_t row0 = (uint64_t)blockIdx.y * BM;
  const uint64_t col0 = (uint64_t)blockIdx.x * BN;
  const int tx = threadIdx.x % (BN / TN);
  const int ty = threadIdx.x / (BN / TN);
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (uint64_t k0 = 0; k0 < k; k0 += BK) {
    // Stage the two slabs.  The index that is contiguous in memory varies
    // fastest across threads: k for a row-major left, i for a transposed one.
    for (int e = threadIdx.x; e < BM * BK; e += kThreads) {
      int kk, ii;
      if (lsk == 1) { kk = e % BK; ii = e / BK; } else { ii = e % BM; kk = e / BM; }
      uint64_t gi = row0 + ii, gk = k0 + kk;
      sa[kk][ii] = (gi < m && gk < k) ? left[gi * lsi + gk * lsk] : 0.f;
    }
    for (int e = threadIdx.x; e < BN * BK; e += kThreads) {
      int kk, jj;
      if (rsj == 1) { jj = e % BN; kk = e / BN; } else { kk = e % BK; jj = e / BK; }
      uint64_t gj = col0 + jj, gk = k0 + kk;
      sb[kk][jj] = (gj < n && gk < k) ? right[gk * rsk + gj * rsj] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = sa[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = sb[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    uint64_t gi = row0 + ty * TM + i;
    if (gi >= m) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      uint64_t gj = col0 + tx * TN + j;
      if (gj < n) out[gi * n + gj] = acc[i][j];
    }
  }
}

}  // namespace

int launch_ffma(int tl, int tr, uint64_t m, uint64_t n, uint64_t k, const float* left,
                const float* right, float* out, cudaStream_t stream) {
  uint64_t gx = (n + BN - 1) / BN, gy = (m + BM - 1) / BM;
  if (gy > 65535) return fail(POLAR_B200_ERR_UNSUPPORTED, "ffma matmul: more than 65535 row tiles");
  dim3 grid((unsigned)gx, (unsigned)gy);
  uint64_t lsi = tl ? 1 : k, lsk = tl ? m : 1;
  uint64_t rsk = tr ? 1 : n, rsj = tr ? k : 1;
  ffma_kernel<<<grid, kThreads, 0, stream>>>(left, right, out, m, n, k, lsi, lsk, rsk, rsj);
  return check_launch("fmatmul_ffma");
}

}  // namespace polar_b200
