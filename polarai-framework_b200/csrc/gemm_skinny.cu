// fmatmul for shapes with one tiny dimension - the MLP's 10-wide output layer and
// the logistic regression's single column.  A 128 x 256 tensor-core tile would be
// more than 90 % padding there, and the work is bound by streaming the one large
// operand (or the large result) through HBM once, so these run on the CUDA cores
// with 128-bit coalesced accesses of the large matrix and the small one in shared
// memory or registers.
//
//   small_n, left K-contiguous  (left stored [m,k]):   C[m, n<=16] = L . R
//       one warp per group of 4 rows; lanes walk k four floats at a time; R sits
//       transposed in shared memory - all of it, loaded once per persistent CTA,
//       when it fits, else one k-slab at a time; warp-shuffle reduction.
//   small_n, left M-contiguous  (left stored [k,m]):   C[m, n<=16] = L^T . R
//       the sum runs over the long (batch) dimension: the k range is split over
//       CTAs, each thread owns 4 consecutive m and n accumulators each, partial
//       sums go to scratch memory [split][m][n] and a second kernel adds the
//       splits in a fixed order (deterministic; no atomics).
//   small_k (k <= 16):                                  C[m,n] = L . R, result-bound
//       each thread keeps its 4 columns of R in registers and streams rows.
//
// Accumulation is fp32 with fmaf; the order of the k sum differs from the
// reference's sequential order, within the fp32 tolerance used for fmatmul.
#include <mutex>

#include "common.cuh"

namespace polar_b200 {
namespace skinny {

constexpr int kThreads = 256;

// ---------------------------------------------------------------- small n, K-major left

constexpr int KT = 1024;          // k-slab staged in shared memory
constexpr int KT_PAD = KT + 4;    // keeps float4 alignment, staggers banks between columns
constexpr int ROWS_PER_WARP = 4;

// After the xor-shuffle reduction every lane holds all ROWS_PER_WARP x NP sums.  The warp's
// rows are contiguous in `out` (n values each), so lane l stores flat elements l, l + 32, ...:
// coalesced stores, and a fused sigmoid costs each lane one or two evaluations, not forty.
template <int NP>
__device__ __forceinline__ void store_row_sums(const float (&acc)[ROWS_PER_WARP][NP], float* __restrict__ out,
                                               uint64_t row0, uint64_t m, uint64_t n, int lane, int act) {
  if (row0 >= m) return;
  const uint32_t rows = (uint32_t)((m - row0 < ROWS_PER_WARP) ? (m - row0) : ROWS_PER_WARP);
  const uint32_t total = rows * (uint32_t)n;
  for (uint32_t f = lane; f < total; f += 32) {
    float v = 0.f;
#pragma unroll
    for (int r = 0; r < ROWS_PER_WARP; ++r)
#pragma unroll
      for (int j = 0; j < NP; ++j)
        if ((uint32_t)j < (uint32_t)n && (uint32_t)r * (uint32_t)n + (uint32_t)j == f) v = acc[r][j];
    out[row0 * n + f] = act ? sigmoid_clamped(v) : v;
  }
}

template <int NP>
__global__ void __launch_bounds__(kThreads)
small_n_kmajor_kernel(const float* __restrict__ left, const float* __restrict__ right,
                      float* __restrict__ out, uint64_t m, uint64_t n, uint64_t k, uint64_t rsk,
                      uint64_t rsj, int act) {
  extern __shared__ float bs[];   // [NP][KT_PAD], k contiguous
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint64_t rows_per_cta = (kThreads / 32) * ROWS_PER_WARP;
  const uint64_t row0 = (uint64_t)blockIdx.x * rows_per_cta + (uint64_t)warp * ROWS_PER_WARP;
  float acc[ROWS_PER_WARP][NP];
#pragma unroll
  for (int r = 0; r < ROWS_PER_WARP; ++r)
#pragma unroll
    for (int j = 0; j < NP; ++j) acc[r][j] = 0.f;

  for (uint64_t k0 = 0; k0 < k; k0 += KT) {
    const int kt = (int)((k - k0 < KT) ? (k - k0) : KT);
    __syncthreads();
    for (int e = threadIdx.x; e < NP * KT; e += kThreads) {
      int j = e % NP, kk = e / NP;
      float v = 0.f;
      if (kk < kt && (uint64_t)j < n) v = right[(k0 + kk) * rsk + (uint64_t)j * rsj];
      bs[j * KT_PAD + kk] = v;
    }
    __syncthreads();
    for (int kk = lane * 4; kk < kt; kk += 128) {   // k is a multiple of 4: no ragged vector
      float4 a[ROWS_PER_WARP];
#pragma unroll
      for (int r = 0; r < ROWS_PER_WARP; ++r) {
        uint64_t row = row0 + r;
        a[r] = row < m ? __ldcs(reinterpret_cast<const float4*>(left + row * k + k0 + kk))
                       : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int j = 0; j < NP; ++j) {
        float4 b = *reinterpret_cast<const float4*>(&bs[j * KT_PAD + kk]);
#pragma unroll
        for (int r = 0; r < ROWS_PER_WARP; ++r) {
          acc[r][j] = fmaf(a[r].x, b.x, acc[r][j]);
          acc[r][j] = fmaf(a[r].y, b.y, acc[r][j]);
          acc[r][j] = fmaf(a[r].z, b.z, acc[r][j]);
          acc[r][j] = fmaf(a[r].w, b.w, acc[r][j]);
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < ROWS_PER_WARP; ++r) {
#pragma unroll
    for (int j = 0; j < NP; ++j) {
      float v = acc[r][j];
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
      acc[r][j] = v;
    }
  }
  store_row_sums<NP>(acc, out, row0, m, n, lane, act);
}

// ---------------------------------------------------------------- small n, K-major left, R resident

// When the whole small operand fits in shared memory (n_padded * (k + 4) floats, e.g.
// 164 KB for the MLP's 4096 x 10 output layer) it is loaded ONCE per CTA; one
// persistent 512-thread CTA per SM then streams row groups of the large operand
// with no barrier in the loop.  Each warp owns 4 rows at a time and keeps two
// k chunks (8 x 128-bit loads per lane) in flight.
constexpr int kResidentThreads = 512;

template <int NP>
__global__ void __launch_bounds__(kResidentThreads, 1)
small_n_kmajor_resident_kernel(const float* __restrict__ left, const float* __restrict__ right,
                               float* __restrict__ out, uint64_t m, uint64_t n, uint64_t k, uint64_t rsk,
                               uint64_t rsj, int act) {
  extern __shared__ float bs[];   // [NP][k + 4], k contiguous
  const uint32_t kpad = (uint32_t)k + 4;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint64_t warps_total = (uint64_t)gridDim.x * (kResidentThreads / 32);
  const uint64_t groups = (m + ROWS_PER_WARP - 1) / ROWS_PER_WARP;
  uint64_t g = (uint64_t)blockIdx.x * (kResidentThreads / 32) + warp;
  // The loads of a chunk (two 128-bit loads per row and lane) are issued one chunk ahead of its
  // arithmetic, and the very first ones before the small operand is staged: with one group of
  // rows per warp (8192 rows on 148 SMs) the kernel is otherwise a chain of memory latencies.
  float4 a0[ROWS_PER_WARP], a1[ROWS_PER_WARP];
  auto load_chunk = [&](uint64_t group, uint32_t kk) {
#pragma unroll
    for (int r = 0; r < ROWS_PER_WARP; ++r) {
      const uint64_t row = group * ROWS_PER_WARP + r;
      const float* src = left + (row < m ? row : m - 1) * k;   // clamped: results of padding rows are dropped
      a0[r] = __ldcs(reinterpret_cast<const float4*>(src + kk));
      a1[r] = (kk + 128 < (uint32_t)k) ? __ldcs(reinterpret_cast<const float4*>(src + kk + 128))
                                       : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  };
  if (g < groups && (uint32_t)lane * 4 < (uint32_t)k) load_chunk(g, lane * 4);
  for (uint64_t e = threadIdx.x; e < (uint64_t)NP * k; e += kResidentThreads) {
    uint32_t j = (uint32_t)(e % NP), kk = (uint32_t)(e / NP);
    bs[j * kpad + kk] = ((uint64_t)j < n) ? right[(uint64_t)kk * rsk + (uint64_t)j * rsj] : 0.f;
  }
  __syncthreads();
  for (; g < groups; g += warps_total) {
    const uint64_t row0 = g * ROWS_PER_WARP;
    float acc[ROWS_PER_WARP][NP];
#pragma unroll
    for (int r = 0; r < ROWS_PER_WARP; ++r)
#pragma unroll
      for (int j = 0; j < NP; ++j) acc[r][j] = 0.f;
    for (uint32_t kk = lane * 4; kk < (uint32_t)k; kk += 256) {
      float4 c0[ROWS_PER_WARP], c1[ROWS_PER_WARP];
#pragma unroll
      for (int r = 0; r < ROWS_PER_WARP; ++r) { c0[r] = a0[r]; c1[r] = a1[r]; }
      const bool second = kk + 128 < (uint32_t)k;
      // the next chunk of this group, or the first chunk of this warp's next group
      if (kk + 256 < (uint32_t)k) load_chunk(g, kk + 256);
      else if (g + warps_total < groups) load_chunk(g + warps_total, lane * 4);
#pragma unroll
      for (int j = 0; j < NP; ++j) {
        const float4 b0 = *reinterpret_cast<const float4*>(&bs[j * kpad + kk]);
#pragma unroll
        for (int r = 0; r < ROWS_PER_WARP; ++r) {
          acc[r][j] = fmaf(c0[r].x, b0.x, acc[r][j]);
          acc[r][j] = fmaf(c0[r].y, b0.y, acc[r][j]);
          acc[r][j] = fmaf(c0[r].z, b0.z, acc[r][j]);
          acc[r][j] = fmaf(c0[r].w, b0.w, acc[r][j]);
        }
      }
      if (second) {
#pragma unroll
        for (int j = 0; j < NP; ++j) {
          const float4 b1 = *reinterpret_cast<const float4*>(&bs[j * kpad + kk + 128]);
#pragma unroll
          for (int r = 0; r < ROWS_PER_WARP; ++r) {
            acc[r][j] = fmaf(c1[r].x, b1.x, acc[r][j]);
            acc[r][j] = fmaf(c1[r].y, b1.y, acc[r][j]);
            acc[r][j] = fmaf(c1[r].z, b1.z, acc[r][j]);
            acc[r][j] = fmaf(c1[r].w, b1.w, acc[r][j]);
          }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < ROWS_PER_WARP; ++r)
#pragma unroll
      for (int j = 0; j < NP; ++j) {
        float v = acc[r][j];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        acc[r][j] = v;
      }
    store_row_sums<NP>(acc, out, row0, m, n, lane, act);
  }
}

// ---------------------------------------------------------------- small n, MN-major left (split k)

constexpr int KS = 128;   // rows of R staged per pass

// Two fused multiply-adds in one instruction (sm_100: fma.rn.f32x2 on register pairs), each
// an IEEE fma like fmaf: (c.lo, c.hi) = (a.lo, a.hi) * (b.lo, b.hi) + (c.lo, c.hi).
__device__ __forceinline__ void ffma2(unsigned long long& c, unsigned long long a, unsigned long long b) {
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(c) : "l"(a), "l"(b));
}
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

// The kernel issues one instruction per two multiply-adds and reads each value of the staged
// operand as a ready-made (b, b) pair: at 16 columns the plain form needs every issue slot of
// the SM to keep up with HBM (64 FMA + 16 shared-memory loads per 16 bytes streamed).
template <int NP>
__global__ void __launch_bounds__(kThreads, 2)
small_n_mnmajor_kernel(const float* __restrict__ left, const float* __restrict__ right,
                       float* __restrict__ partial, uint64_t m, uint64_t n, uint64_t k, uint64_t rsk,
                       uint64_t rsj, uint64_t k_per_split) {
  __shared__ __align__(8) float2 bs[KS][NP];   // every value twice: one 64-bit load yields the pair
  const uint64_t m0 = ((uint64_t)blockIdx.x * kThreads + threadIdx.x) * 4;
  const uint64_t kbeg = (uint64_t)blockIdx.y * k_per_split;
  const uint64_t kend = (kbeg + k_per_split < k) ? kbeg + k_per_split : k;
  unsigned long long acc01[NP], acc23[NP];      // rows (0,1) and (2,3) of the thread's four
#pragma unroll
  for (int j = 0; j < NP; ++j) acc01[j] = acc23[j] = 0ull;
  const bool live = m0 < m;   // m is a multiple of 4
  for (uint64_t k0 = kbeg; k0 < kend; k0 += KS) {
    const int ks = (int)((kend - k0 < KS) ? (kend - k0) : KS);
    __syncthreads();
    for (int e = threadIdx.x; e < KS * NP; e += kThreads) {
      int j = e % NP, kk = e / NP;
      float v = 0.f;
      if (kk < ks && (uint64_t)j < n) v = right[(k0 + kk) * rsk + (uint64_t)j * rsj];
      bs[kk][j] = make_float2(v, v);
    }
    __syncthreads();
    if (live) {
      int kk = 0;
      // eight 128-bit loads in flight per thread: two CTAs of 256 threads per SM then keep
      // 64 KB outstanding, what HBM latency x bandwidth asks of one SM
      for (; kk + 8 <= ks; kk += 8) {
        float4 a[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
          a[u] = __ldcs(reinterpret_cast<const float4*>(left + (k0 + kk + u) * m + m0));
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const unsigned long long a01 = pack2(a[u].x, a[u].y), a23 = pack2(a[u].z, a[u].w);
#pragma unroll
          for (int j = 0; j < NP; ++j) {
            const unsigned long long bb = *reinterpret_cast<const unsigned long long*>(&bs[kk + u][j]);
            ffma2(acc01[j], a01, bb);
            ffma2(acc23[j], a23, bb);
          }
        }
      }
      for (; kk < ks; ++kk) {
        const float4 a = __ldcs(reinterpret_cast<const float4*>(left + (k0 + kk) * m + m0));
        const unsigned long long a01 = pack2(a.x, a.y), a23 = pack2(a.z, a.w);
#pragma unroll
        for (int j = 0; j < NP; ++j) {
          const unsigned long long bb = *reinterpret_cast<const unsigned long long*>(&bs[kk][j]);
          ffma2(acc01[j], a01, bb);
          ffma2(acc23[j], a23, bb);
        }
      }
    }
  }
  if (live) {
    float* dst = partial + ((uint64_t)blockIdx.y * m + m0) * n;
#pragma unroll
    for (int j = 0; j < NP; ++j) {
      float r0, r1, r2, r3;
      unpack2(acc01[j], r0, r1);
      unpack2(acc23[j], r2, r3);
      if ((uint64_t)j < n) {
        dst[j] = r0;
        dst[n + j] = r1;
        dst[2 * n + j] = r2;
        dst[3 * n + j] = r3;
      }
    }
  }
}

// Sum of one element over the splits, ascending split index (a fixed order); the loads of
// eight splits are issued together, the additions stay in order.
__device__ __forceinline__ float sum_splits(const float* __restrict__ partial, uint64_t elems, uint64_t e,
                                            uint32_t splits) {
  float s = 0.f;
  uint32_t sp = 0;
  for (; sp + 8 <= splits; sp += 8) {
    float v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = __ldcg(partial + (uint64_t)(sp + u) * elems + e);
#pragma unroll
    for (int u = 0; u < 8; ++u) s += v[u];
  }
  for (; sp < splits; ++sp) s += __ldcg(partial + (uint64_t)sp * elems + e);
  return s;
}

// out[e] = sum over splits, ascending split index: a fixed order.
__global__ void __launch_bounds__(kThreads)
reduce_splits_kernel(const float* __restrict__ partial, float* __restrict__ out, uint64_t elems,
                     uint32_t splits) {
  const uint64_t stride = (uint64_t)gridDim.x * kThreads;
  for (uint64_t e = (uint64_t)blockIdx.x * kThreads + threadIdx.x; e < elems; e += stride)
    out[e] = sum_splits(partial, elems, e, splits);
}

// The same sum, stored transposed: partial is [split][m][n], out is [n][m].  Used for the
// last few rows of a product whose left operand is stored [k, rows]: they are computed as
// the small-n product of the transposed problem and land as rows of the result.
__global__ void __launch_bounds__(kThreads)
reduce_splits_transposed_kernel(const float* __restrict__ partial, float* __restrict__ out, uint64_t m,
                                uint64_t n, uint32_t splits) {
  const uint64_t elems = m * n, stride = (uint64_t)gridDim.x * kThreads;
  for (uint64_t e = (uint64_t)blockIdx.x * kThreads + threadIdx.x; e < elems; e += stride) {
    out[(e % n) * m + e / n] = sum_splits(partial, elems, e, splits);
  }
}

// ---------------------------------------------------------------- small k

constexpr int RK = 64;   // rows of the left operand staged per CTA

// L'(i,kk) = left[i*lsi + kk*lsk]; R'(kk,j) = right[kk*rsk + j*rsj]; k <= KP.
template <int KP>
__global__ void __launch_bounds__(kThreads)
small_k_kernel(const float* __restrict__ left, const float* __restrict__ right, float* __restrict__ out,
               uint64_t m, uint64_t n, uint64_t k, uint64_t lsi, uint64_t lsk, uint64_t rsk,
               uint64_t rsj, int vec_store, const float* __restrict__ sig) {
  __shared__ float as[RK][KP];
  const uint64_t j0 = ((uint64_t)blockIdx.x * kThreads + threadIdx.x) * 4;
  // Each thread's four columns of the small operand stay in registers while the CTA walks
  // over row blocks (gridDim.y CTAs share the rows of one column block).
  float b[4][KP];
#pragma unroll
  for (int c = 0; c < 4; ++c)
#pragma unroll
    for (int kk = 0; kk < KP; ++kk)
      b[c][kk] = (j0 + c < n && (uint64_t)kk < k) ? right[(uint64_t)kk * rsk + (j0 + c) * rsj] : 0.f;
  const bool vec = vec_store && j0 + 4 <= n;
  // The gridDim.y CTAs of a column block split the rows evenly (contiguous ranges, a multiple
  // of four rows each) and stage them RK at a time.
  const uint64_t rows_per_cta = ((m + gridDim.y - 1) / gridDim.y + 3) & ~3ull;
  const uint64_t row_begin = (uint64_t)blockIdx.y * rows_per_cta;
  const uint64_t row_end = row_begin + rows_per_cta < m ? row_begin + rows_per_cta : m;
  for (uint64_t row0 = row_begin; row0 < row_end; row0 += RK) {
    const int rows = (int)((row_end - row0 < RK) ? (row_end - row0) : RK);
    __syncthreads();   // the previous block's rows are no longer read
    for (int e = threadIdx.x; e < RK * KP; e += kThreads) {
      int kk = e % KP, r = e / KP;
      float v = 0.f;
      if (r < rows && (uint64_t)kk < k) v = left[(row0 + r) * lsi + (uint64_t)kk * lsk];
      as[r][kk] = v;
    }
    __syncthreads();
    if (j0 >= n) continue;
    // Rows in groups of four: the four loads of the sigmoid values are issued before any of
    // the arithmetic, so each thread keeps four 128-bit loads in flight.
    for (int rb = 0; rb < rows; rb += 4) {
      float4 sv[4];
      if (sig) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (rb + u >= rows) continue;
          const float* sp = sig + (row0 + rb + u) * n + j0;
          if (vec) {
            sv[u] = __ldcs(reinterpret_cast<const float4*>(sp));
          } else {
            sv[u].x = sp[0];
            sv[u].y = (j0 + 1 < n) ? sp[1] : 0.f;
            sv[u].z = (j0 + 2 < n) ? sp[2] : 0.f;
            sv[u].w = (j0 + 3 < n) ? sp[3] : 0.f;
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int r = rb + u;
        if (r >= rows) continue;
        float c0 = 0.f, c1 = 0.f, c2 = 0.f, c3 = 0.f;
#pragma unroll
        for (int kk = 0; kk < KP; ++kk) {
          float a = as[r][kk];
          c0 = fmaf(a, b[0][kk], c0);
          c1 = fmaf(a, b[1][kk], c1);
          c2 = fmaf(a, b[2][kk], c2);
          c3 = fmaf(a, b[3][kk], c3);
        }
        if (sig) {
          // fused Sigmoid derivative: out = product * ((1 - s) * s), s = fsigmoid output
          c0 = sigmoid_grad_chain(c0, sv[u].x); c1 = sigmoid_grad_chain(c1, sv[u].y);
          c2 = sigmoid_grad_chain(c2, sv[u].z); c3 = sigmoid_grad_chain(c3, sv[u].w);
        }
        float* dst = out + (row0 + r) * n + j0;
        if (vec) {
          __stcs(reinterpret_cast<float4*>(dst), make_float4(c0, c1, c2, c3));
        } else {
          dst[0] = c0;
          if (j0 + 1 < n) dst[1] = c1;
          if (j0 + 2 < n) dst[2] = c2;
          if (j0 + 3 < n) dst[3] = c3;
        }
      }
    }
  }   // row ranges
}

// ---------------------------------------------------------------- dense layer backward, one pass
//
// The two products of a dense layer's backward pass that read the layer's INPUT activations
//   dW[kh, n]  = H^T . dZ                      (small n, left M-contiguous: the kernel above)
//   dIn[B, kh] = (dZ . W^T) * ((1 - H) * H)    (small k with the Sigmoid derivative fused)
// share everything: both stream H [B, kh] row by row, both want the dZ rows staged in shared
// memory, and in both a thread owns four consecutive hidden columns.  Done separately H
// crosses HBM twice; here once.  Per row a thread loads its four H values (one 128-bit load),
// reads the dZ row from shared memory, accumulates dW for its columns and stores its four
// dIn values.  The arithmetic, its order and the division of the batch rows into splits are
// those of the two kernels above (same fma per term, rows ascending, splits added in
// ascending order), so both results carry the bits of the separate launches.
template <int NP>
__global__ void __launch_bounds__(kThreads, NP > 10 ? 1 : 2)
dense_grad_kernel(const float* __restrict__ H, const float* __restrict__ dz, const float* __restrict__ W,
                  float* __restrict__ din, float* __restrict__ partial, uint64_t rows, uint64_t kh, uint64_t n,
                  uint64_t rows_per_split) {
  __shared__ __align__(8) float2 bs[KS][NP];   // dZ rows, every value twice: one 64-bit load yields the pair
  const uint64_t m0 = ((uint64_t)blockIdx.x * kThreads + threadIdx.x) * 4;
  const uint64_t rbeg = (uint64_t)blockIdx.y * rows_per_split;
  const uint64_t rend = (rbeg + rows_per_split < rows) ? rbeg + rows_per_split : rows;
  const bool live = m0 < kh;   // kh is a multiple of 4
  // W rows of the thread's four columns, packed as (column 0, column 1) and (column 2, column 3)
  unsigned long long w01[NP], w23[NP], acc01[NP], acc23[NP];
#pragma unroll
  for (int j = 0; j < NP; ++j) {
    float v[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) v[c] = (live && (uint64_t)j < n) ? W[(m0 + c) * n + j] : 0.f;
    w01[j] = pack2(v[0], v[1]);
    w23[j] = pack2(v[2], v[3]);
    acc01[j] = acc23[j] = 0ull;
  }
  for (uint64_t r0 = rbeg; r0 < rend; r0 += KS) {
    const int rs = (int)((rend - r0 < KS) ? (rend - r0) : KS);
    __syncthreads();
    for (int e = threadIdx.x; e < KS * NP; e += kThreads) {
      int j = e % NP, rr = e / NP;
      float v = 0.f;
      if (rr < rs && (uint64_t)j < n) v = dz[(r0 + rr) * n + j];
      bs[rr][j] = make_float2(v, v);
    }
    __syncthreads();
    if (!live) continue;
    // six to eight 128-bit loads in flight per thread (two CTAs of 256 threads per SM then keep
    // 48-64 KB outstanding, what HBM latency x bandwidth asks of one SM)
    constexpr int kBatch = NP == 10 ? 6 : 8;   // at ten columns 128 registers hold six rows without spilling
    for (int rr = 0; rr < rs; rr += kBatch) {
      float4 h[kBatch];
#pragma unroll
      for (int u = 0; u < kBatch; ++u)
        if (rr + u < rs) h[u] = __ldcs(reinterpret_cast<const float4*>(H + (r0 + rr + u) * kh + m0));
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        if (rr + u >= rs) continue;
        const unsigned long long h01 = pack2(h[u].x, h[u].y), h23 = pack2(h[u].z, h[u].w);
        unsigned long long c01 = 0ull, c23 = 0ull;   // (dZ . W^T) for the four columns
#pragma unroll
        for (int j = 0; j < NP; ++j) {
          const unsigned long long dd = *reinterpret_cast<const unsigned long long*>(&bs[rr + u][j]);
          ffma2(c01, dd, w01[j]);
          ffma2(c23, dd, w23[j]);
          ffma2(acc01[j], h01, dd);
          ffma2(acc23[j], h23, dd);
        }
        float c0, c1, c2, c3;
        unpack2(c01, c0, c1);
        unpack2(c23, c2, c3);
        const float4 o = make_float4(sigmoid_grad_chain(c0, h[u].x), sigmoid_grad_chain(c1, h[u].y),
                                     sigmoid_grad_chain(c2, h[u].z), sigmoid_grad_chain(c3, h[u].w));
        __stcs(reinterpret_cast<float4*>(din + (r0 + rr + u) * kh + m0), o);
      }
    }
  }
  if (live) {
    float* dst = partial + ((uint64_t)blockIdx.y * kh + m0) * n;
#pragma unroll
    for (int j = 0; j < NP; ++j) {
      float r0, r1, r2, r3;
      unpack2(acc01[j], r0, r1);
      unpack2(acc23[j], r2, r3);
      if ((uint64_t)j < n) {
        dst[j] = r0;
        dst[n + j] = r1;
        dst[2 * n + j] = r2;
        dst[3 * n + j] = r3;
      }
    }
  }
}

// ---------------------------------------------------------------- host side

inline int round_np(uint64_t n) { return n <= 1 ? 1 : n <= 2 ? 2 : n <= 4 ? 4 : n <= 8 ? 8 : n <= 10 ? 10 : 16; }

uint32_t splits_for(uint64_t m, uint64_t k) {
  uint64_t m_blocks = (m / 4 + kThreads - 1) / kThreads;
  uint64_t want = ((uint64_t)sm_count() * 2 + m_blocks - 1) / m_blocks;   // about two CTAs per SM
  uint64_t max_by_k = (k + KS - 1) / KS;
  uint64_t s = want < max_by_k ? want : max_by_k;
  if (s < 1) s = 1;
  if (s > 4096) s = 4096;
  return (uint32_t)s;
}

template <int NP>
int launch_small_n_k(const float* l, const float* r, float* out, uint64_t m, uint64_t n, uint64_t k,
                     uint64_t rsk, uint64_t rsj, cudaStream_t st, int act) {
  // whole small operand resident in shared memory when it fits (and there are rows
  // enough to keep every SM busy); otherwise k slabs
  const size_t resident = (size_t)NP * (k + 4) * sizeof(float);
  if (resident <= 200 * 1024 && m >= 4096) {
    static bool res_attr[64] = {false};
    int d = 0;
    cudaGetDevice(&d);
    if (d >= 0 && d < 64 && !res_attr[d]) {
      cudaError_t e = cudaFuncSetAttribute(small_n_kmajor_resident_kernel<NP>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      if (e != cudaSuccess) return fail(POLAR_B200_ERR_CUDA, "cudaFuncSetAttribute(small_n resident)", e);
      res_attr[d] = true;
    }
    small_n_kmajor_resident_kernel<NP><<<(unsigned)sm_count(), kResidentThreads, resident, st>>>(
        l, r, out, m, n, k, rsk, rsj, act);
    return check_launch("fmatmul_small_n_resident");
  }
  const size_t smem = (size_t)NP * KT_PAD * sizeof(float);
  static bool attr_done[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (smem > 48 * 1024 && dev >= 0 && dev < 64 && !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(small_n_kmajor_kernel<NP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(POLAR_B200_ERR_CUDA, "cudaFuncSetAttribute(small_n)", e);
    attr_done[dev] = true;
  }
  uint64_t rows_per_cta = (kThreads / 32) * ROWS_PER_WARP;
  uint64_t grid = (m + rows_per_cta - 1) / rows_per_cta;
  if (grid > 0x7fffffffull) return fail(POLAR_B200_ERR_UNSUPPORTED, "too many rows");
  small_n_kmajor_kernel<NP><<<(unsigned)grid, kThreads, smem, st>>>(l, r, out, m, n, k, rsk, rsj, act);
  return check_launch("fmatmul_small_n");
}

template <int NP>
int launch_small_n_mn(const float* l, const float* r, float* out, float* ws, uint32_t splits, uint64_t m,
                      uint64_t n, uint64_t k, uint64_t rsk, uint64_t rsj, cudaStream_t st) {
  uint64_t m_blocks = (m / 4 + kThreads - 1) / kThreads;
  uint64_t k_per_split = (k + splits - 1) / splits;
  k_per_split = (k_per_split + 3) & ~3ull;
  dim3 grid((unsigned)m_blocks, splits);
  float* dst = splits > 1 ? ws : out;
  small_n_mnmajor_kernel<NP><<<grid, kThreads, 0, st>>>(l, r, dst, m, n, k, rsk, rsj, k_per_split);
  int rc = check_launch("fmatmul_small_n_split");
  if (rc || splits == 1) return rc;
  uint64_t elems = m * n;
  uint64_t g = (elems + kThreads - 1) / kThreads;
  uint64_t cap = (uint64_t)sm_count() * 4;
  reduce_splits_kernel<<<(unsigned)(g < cap ? g : cap), kThreads, 0, st>>>(ws, out, elems, splits);
  return check_launch("fmatmul_reduce_splits");
}

template <int NP>
int launch_dense_grad_np(const float* H, const float* dz, const float* W, float* din, float* dw, float* ws,
                         uint32_t splits, uint64_t rows, uint64_t kh, uint64_t n, cudaStream_t st) {
  // the same division of the rows as launch_small_n_mn makes for dW = H^T . dZ
  uint64_t m_blocks = (kh / 4 + kThreads - 1) / kThreads;
  uint64_t rows_per_split = (rows + splits - 1) / splits;
  rows_per_split = (rows_per_split + 3) & ~3ull;
  dim3 grid((unsigned)m_blocks, splits);
  float* dst = splits > 1 ? ws : dw;
  dense_grad_kernel<NP><<<grid, kThreads, 0, st>>>(H, dz, W, din, dst, rows, kh, n, rows_per_split);
  int rc = check_launch("fdense_grad");
  if (rc || splits == 1) return rc;
  uint64_t elems = kh * n;
  uint64_t g = (elems + kThreads - 1) / kThreads;
  uint64_t cap = (uint64_t)sm_count() * 4;
  reduce_splits_kernel<<<(unsigned)(g < cap ? g : cap), kThreads, 0, st>>>(ws, dw, elems, splits);
  return check_launch("fdense_grad_reduce");
}

}  // namespace skinny

// out_tail[j, i] = sum_kk left_tail[kk*left_pitch + j] * right[kk*n + i]   (j < rem <= 16, i < n):
// `rem` rows of a t_f product, as the small-n product right^T . left_tail stored transposed.
// Scratch: ragged_rows_workspace_bytes.  n a multiple of 4, right 16-byte aligned.
uint64_t ragged_rows_workspace_bytes(uint64_t rem, uint64_t n, uint64_t k) {
  return (uint64_t)skinny::splits_for(n, k) * n * rem * sizeof(float);
}

int launch_ragged_rows(const float* left_tail, uint64_t left_pitch, const float* right, float* out_tail,
                       float* ws, uint64_t rem, uint64_t n, uint64_t k, cudaStream_t st) {
  using namespace skinny;
  const uint32_t splits = splits_for(n, k);
  uint64_t m_blocks = (n / 4 + kThreads - 1) / kThreads;
  uint64_t k_per_split = (k + splits - 1) / splits;
  k_per_split = (k_per_split + 3) & ~3ull;
  dim3 grid((unsigned)m_blocks, splits);
  const int np = round_np(rem);
  switch (np) {
#define POLAR_RAGGED(NP) \
  case NP: small_n_mnmajor_kernel<NP><<<grid, kThreads, 0, st>>>(right, left_tail, ws, n, rem, k, left_pitch, 1, k_per_split); break;
    POLAR_RAGGED(1) POLAR_RAGGED(2) POLAR_RAGGED(4) POLAR_RAGGED(8) POLAR_RAGGED(10) POLAR_RAGGED(16)
#undef POLAR_RAGGED
    default: return fail(POLAR_B200_ERR_UNSUPPORTED, "ragged rows: more than 16");
  }
  int rc = check_launch("fmatmul_ragged_rows");
  if (rc) return rc;
  uint64_t g = (n * rem + kThreads - 1) / kThreads;
  uint64_t cap = (uint64_t)sm_count() * 4;
  reduce_splits_transposed_kernel<<<(unsigned)(g < cap ? g : cap), kThreads, 0, st>>>(ws, out_tail, n, rem, splits);
  return check_launch("fmatmul_ragged_rows_reduce");
}

// Which skinny kernel, if any, serves this shape: 1 = small n with K-major left,
// 2 = small n with MN-major left (needs scratch), 3 = small k, 0 = none.
int skinny_kind(int tl, int tr, uint64_t m, uint64_t n, uint64_t k, const float* left,
                const float* right, const float* out) {
  (void)tr; (void)right;
  if (n <= 16 && k >= 32) {
    if (!tl && (k & 3) == 0 && aligned16(left)) return 1;
    if (tl && (m & 3) == 0 && aligned16(left)) return 2;
  }
  if (k <= 16 && n >= 32) return 3;
  (void)out;
  return 0;
}

uint64_t skinny_workspace_bytes(int kind, uint64_t m, uint64_t n, uint64_t k) {
  if (kind != 2) return 0;
  uint32_t s = skinny::splits_for(m, k);
  return s > 1 ? (uint64_t)s * m * n * sizeof(float) : 0;
}

// `sig` (small k only): fuse the Sigmoid derivative with this sigmoid output;
// `sigmoid_out` (small n, K-major left only): store fsigmoid of the product.
int launch_skinny(int kind, int tl, int tr, uint64_t m, uint64_t n, uint64_t k, const float* left,
                  const float* right, float* out, float* ws, cudaStream_t st, const float* sig, int sigmoid_out) {
  using namespace skinny;
  const uint64_t rsk = tr ? 1 : n, rsj = tr ? k : 1;
  if (kind == 1 || kind == 2) {
    const int np = round_np(n);
    const uint32_t splits = kind == 2 ? splits_for(m, k) : 1;
#define POLAR_SKINNY_N(NP)                                                                   \
  case NP:                                                                                   \
    return kind == 1 ? launch_small_n_k<NP>(left, right, out, m, n, k, rsk, rsj, st, sigmoid_out) \
                     : launch_small_n_mn<NP>(left, right, out, ws, splits, m, n, k, rsk, rsj, st);
    switch (np) {
      POLAR_SKINNY_N(1)
      POLAR_SKINNY_N(2)
      POLAR_SKINNY_N(4)
      POLAR_SKINNY_N(8)
      POLAR_SKINNY_N(10)
      POLAR_SKINNY_N(16)
    }
#undef POLAR_SKINNY_N
    return fail(POLAR_B200_ERR_UNSUPPORTED, "skinny matmul: unsupported n");
  }
  // small k
  const uint64_t lsi = tl ? 1 : k, lsk = tl ? m : 1;
  uint64_t gx = ((n + 3) / 4 + kThreads - 1) / kThreads, gy = (m + RK - 1) / RK;
  // about three CTAs per SM in all; each takes an equal share of the rows
  const uint64_t gy_cap = ((uint64_t)sm_count() * 3 + gx - 1) / gx;
  if (gy > gy_cap) gy = gy_cap;
  if (gy > 65535) {
    return fail(POLAR_B200_ERR_UNSUPPORTED, "skinny matmul: more than 65535 row blocks");
  }
  dim3 grid((unsigned)gx, (unsigned)gy);
  int vec = ((n & 3) == 0) && aligned16(out) && (!sig || aligned16(sig));
  if (k <= 4)
    small_k_kernel<4><<<grid, kThreads, 0, st>>>(left, right, out, m, n, k, lsi, lsk, rsk, rsj, vec, sig);
  else if (k <= 10)
    small_k_kernel<10><<<grid, kThreads, 0, st>>>(left, right, out, m, n, k, lsi, lsk, rsk, rsj, vec, sig);
  else
    small_k_kernel<16><<<grid, kThreads, 0, st>>>(left, right, out, m, n, k, lsi, lsk, rsk, rsj, vec, sig);
  return check_launch("fmatmul_small_k");
}


// Whether the one-pass dense-layer backward serves these sizes, i.e. whether the two separate
// products would run on the small-n (left M-contiguous) and small-k kernels whose arithmetic it
// reproduces: dZ [rows, n], W [kh, n], H and dIn [rows, kh].
bool dense_grad_ok(uint64_t rows, uint64_t kh, uint64_t n, const float* H, const float* din) {
  return n >= 1 && n <= 16 && rows >= 32 && kh >= 32 && (kh & 3) == 0 && aligned16(H) && aligned16(din);
}
uint64_t dense_grad_workspace_bytes(uint64_t rows, uint64_t kh, uint64_t n) {
  return skinny_workspace_bytes(2, kh, n, rows);
}
int launch_dense_grad(const float* H, const float* dz, const float* W, float* din, float* dw, float* ws,
                      uint64_t rows, uint64_t kh, uint64_t n, cudaStream_t st) {
  using namespace skinny;
  const uint32_t splits = splits_for(kh, rows);
  switch (round_np(n)) {
#define POLAR_DENSE(NP) case NP: return launch_dense_grad_np<NP>(H, dz, W, din, dw, ws, splits, rows, kh, n, st);
    POLAR_DENSE(1) POLAR_DENSE(2) POLAR_DENSE(4) POLAR_DENSE(8) POLAR_DENSE(10) POLAR_DENSE(16)
#undef POLAR_DENSE
  }
  return fail(POLAR_B200_ERR_UNSUPPORTED, "fdense_grad: unsupported n");
}

// ---------------------------------------------------------------- entry point that allocates nothing

// Scratch for polar_b200_fmatmul_tn_small_n_static: the per-split partial sums of
// the split-k kernel above.  It is part of the library image, so every GPU that
// loads the library holds these 16 MiB until the process exits.
constexpr uint64_t kStaticScratchBytes = 16ull << 20;
static __device__ __align__(256) float g_static_scratch[kStaticScratchBytes / sizeof(float)];

namespace {
// In host code `g_static_scratch` is only a handle for the runtime; the address the
// kernels need comes from cudaGetSymbolAddress, asked once per device with that
// device current.
float* static_scratch_for_current_device(int* status) {
  static std::mutex mu;
  static float* cached[64] = {nullptr};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    *status = fail(POLAR_B200_ERR_CUDA, "cudaGetDevice", e);
    return nullptr;
  }
  std::lock_guard<std::mutex> guard(mu);
  if (!cached[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || !p) {
      *status = fail(POLAR_B200_ERR_CUDA, "cudaGetSymbolAddress(static scratch)", e);
      return nullptr;
    }
    cached[dev] = static_cast<float*>(p);
  }
  *status = POLAR_B200_OK;
  return cached[dev];
}
}  // namespace

}  // namespace polar_b200

extern "C" {

uint64_t polar_b200_static_scratch_bytes(void) { return polar_b200::kStaticScratchBytes; }

int polar_b200_fmatmul_tn_small_n_static(int transRight, uint64_t m, uint64_t n, uint64_t k,
                                         const float* left, const float* right, float* out,
                                         void* stream) {
  using namespace polar_b200;
  clear_error();
  if (transRight != 0 && transRight != 1) return fail(POLAR_B200_ERR_INVALID, "transRight must be 0 or 1");
  if (m == 0 || n == 0) return POLAR_B200_OK;
  if (!left || !right || !out) return fail(POLAR_B200_ERR_INVALID, "null device pointer");
  if (n > 16 || k < 32 || (m & 3) != 0 || !aligned16(left))
    return fail(POLAR_B200_ERR_UNSUPPORTED,
                "static-scratch fmatmul serves left stored [k,m] with m a multiple of 4, a 16-byte aligned "
                "left pointer, n <= 16 and k >= 32");
  if (m > (1ull << 31) || k > (1ull << 31)) return fail(POLAR_B200_ERR_INVALID, "matrix dimension too large");
  const uint64_t need = skinny_workspace_bytes(2, m, n, k);
  if (need > kStaticScratchBytes)
    return fail(POLAR_B200_ERR_WORKSPACE,
                "this product needs more than the 16 MiB of built-in scratch; use polar_b200_fmatmul with a "
                "caller workspace");
  LaunchDeviceScope on(stream, out);   // the array's address is looked up on the device that will run the kernels
  int rc = POLAR_B200_OK;
  float* scratch = static_scratch_for_current_device(&rc);
  if (!scratch) return rc;
  // Every partial sum the reduction reads is written by the first kernel of this
  // call, so nothing in the scratch has to be cleared beforehand.
  return launch_skinny(2, 1, transRight, m, n, k, left, right, out, scratch, as_stream(stream), nullptr, 0);
}

}  // extern "C"
