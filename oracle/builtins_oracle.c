/*
 * CPU oracle for the PolarAI builtin kernels.  TEST INFRASTRUCTURE ONLY: nothing
 * shipped by the runtime may link, load or call this file; it exists so that the
 * CUDA kernels can be checked against the reference's arithmetic, and so that
 * the bench can time the same arithmetic on host cores.
 *
 * Each function restates, in plain C, the arithmetic the reference writes down
 * for one builtin.  The citations are paths inside the reference project:
 *   - OpenCL C bodies:  src/backend/generic/runtime/opencl/kernels.h
 *   - in-test oracles:  tests/integration/operations/<Op>Operation.cpp
 *   - MLIR generators:  utils/dialects/lib/PolarGraph/kernels/<Op>Op.cpp
 *
 * Pinning: tests/golden/reference_kats.json holds the inputs of every known
 * answer test the reference has for these builtins together with the outputs of
 * the reference's own OpenCL C kernels compiled as C (oracle/_ref, built by
 * oracle/Makefile); tests/test_oracle.py checks this file against both.
 *
 * Build with -ffp-contract=off: the reference's MLIR form of fadd is
 * mulf, mulf, addf (AddOp.cpp:36-48) - two rounded products, no fused multiply
 * add - and the C compilers that built its test oracles for x86-64 do not
 * contract either.
 *
 * Threading: every loop is an OpenMP loop over independent outputs; the number
 * of threads is set with oracle_set_threads (1 = the scalar port).
 */
#include <math.h>
#include <stdint.h>
#include <stddef.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static int g_threads = 1;

void oracle_set_threads(int n) { g_threads = n < 1 ? 1 : n; }
int oracle_get_threads(void) { return g_threads; }
int oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_num_procs();
#else
  return 1;
#endif
}

#define PAR_FOR _Pragma("omp parallel for num_threads(g_threads) schedule(static)")

/* ffill: out[i] = pattern.  kernels.h:21-30; sycl/kernels/Fill.hpp:71-74. */
void oracle_ffill(float pattern, float* out, uint64_t n) {
  PAR_FOR
  for (int64_t i = 0; i < (int64_t)n; ++i) out[i] = pattern;
}

/* fcopy: out[i] = in[i].  kernels.h:44-53; PolarGraph/kernels/CopyOp.cpp:21-23. */
void oracle_fcopy(const float* in, float* out, uint64_t n) {
  PAR_FOR
  for (int64_t i = 0; i < (int64_t)n; ++i) out[i] = in[i];
}

/* fadd: out[i] = a[i]*scaleA + b[i]*scaleB, each product rounded to fp32 before
 * the sum.  kernels.h:32-42; AddOp.cpp:36-48; CombineOperation.cpp:17-25. */
void oracle_fadd(const float* a, float scaleA, const float* b, float scaleB,
                 float* out, uint64_t n) {
  PAR_FOR
  for (int64_t i = 0; i < (int64_t)n; ++i) {
    float pa = a[i] * scaleA;
    float pb = b[i] * scaleB;
    out[i] = pa + pb;
  }
}

/* fmul: out[i] = a[i]*b[i].  kernels.h:119-128; MulOperation.cpp:17-25. */
void oracle_fmul(const float* a, const float* b, float* out, uint64_t n) {
  PAR_FOR
  for (int64_t i = 0; i < (int64_t)n; ++i) out[i] = a[i] * b[i];
}

/* fdivide: out[i] = num[i]/den[i], IEEE fp32.  kernels.h:55-64;
 * DivideOperation.cpp:17-25. */
void oracle_fdivide(const float* num, const float* den, float* out, uint64_t n) {
  PAR_FOR
  for (int64_t i = 0; i < (int64_t)n; ++i) out[i] = num[i] / den[i];
}

/* fsigmoid: r = 1/(1+exp(-x)); |r-1| < eps -> 1-eps; else |r| < eps -> eps;
 * eps = 1e-5f.  kernels.h:141-156; sycl/kernels/Sigmoid.hpp:32-41;
 * SigmoidOperation.cpp:19-32.  clamp == 0 gives the MLIR form, which has no
 * clamp (SigmoidOp.cpp:37-51). */
void oracle_fsigmoid(const float* in, float* out, uint64_t n, int clamp) {
  const float eps = 1e-5f;
  PAR_FOR
  for (int64_t i = 0; i < (int64_t)n; ++i) {
    float r = 1.0f / (1.0f + expf(-in[i]));
    if (clamp) {
      if (fabsf(r - 1.0f) < eps) {
        r = 1.0f - eps;
      } else if (fabsf(r) < eps) {
        r = eps;
      }
    }
    out[i] = r;
  }
}

/* flogloss: out[i] = -y*log(p+eps) - (1-y)*log(1-p+eps), eps = 1e-5f, with the
 * epsilon inside both logarithms and every step in fp32.  kernels.h:66-78;
 * sycl/kernels/LogLoss.hpp:33-37; LogLossOperation.cpp:19-30. */
void oracle_flogloss(const float* predicted, const float* groundTruth,
                     float* out, uint64_t n) {
  const float eps = 1e-5f;
  PAR_FOR
  for (int64_t i = 0; i < (int64_t)n; ++i) {
    float p = predicted[i];
    float y = groundTruth[i];
    float t0 = -y * logf(p + eps);
    float t1 = (1.0f - y) * logf(1.0f - p + eps);
    out[i] = t0 - t1;
  }
}

/* fmulconcat: out[i] = gradient[0]*local[i].  kernels.h:130-139;
 * MulConcatOp.cpp:37-46; MulConcatOperation.cpp:17-25. */
void oracle_fmulconcat(const float* gradient, const float* local, float* out,
                       uint64_t n) {
  const float g = gradient[0];
  PAR_FOR
  for (int64_t i = 0; i < (int64_t)n; ++i) out[i] = g * local[i];
}

/* frelu: out = in > 0 ? in : 0 (ordered compare: NaN gives 0).
 * utils/dialects/lib/PolarGraph/kernels/ReLUOp.cpp:36-44. */
void oracle_frelu(const float* in, float* out, uint64_t n) {
  PAR_FOR
  for (int64_t i = 0; i < (int64_t)n; ++i) out[i] = in[i] > 0.0f ? in[i] : 0.0f;
}

/* fsoftmax: over the WHOLE tensor, out[i] = exp(in[i]) / sum_j exp(in[j]); the sum is
 * accumulated in fp32 in index order starting from 0, no maximum is subtracted.
 * utils/dialects/lib/PolarGraph/kernels/SoftmaxOp.cpp:38-66 (which recomputes the
 * same sum for every output element). */
void oracle_fsoftmax(const float* in, float* out, uint64_t n) {
  float total = 0.0f;
  for (uint64_t j = 0; j < n; ++j) total = expf(in[j]) + total;
  PAR_FOR
  for (int64_t i = 0; i < (int64_t)n; ++i) out[i] = expf(in[i]) / total;
}

/* fpool: 2-D max pooling; out[i,j] starts at -10e5f and takes every larger input of
 * the window rows i*sh .. i*sh+wh-1, columns j*sw .. j*sw+ww-1; the result is
 * [(h-wh)/sh+1, (w-ww)/sw+1].  Pool2DOp.cpp:44-84;
 * src/operation/internal/Pool2DOperationInternal.cpp:36-41 (shape). */
void oracle_fpool(const float* in, uint64_t h, uint64_t w, uint64_t wh, uint64_t ww, uint64_t sh,
                  uint64_t sw, float* out) {
  const uint64_t oh = (h - wh) / sh + 1, ow = (w - ww) / sw + 1;
  PAR_FOR
  for (int64_t i = 0; i < (int64_t)oh; ++i)
    for (uint64_t j = 0; j < ow; ++j) {
      float best = -10e5f;
      for (uint64_t a = 0; a < wh; ++a)
        for (uint64_t b = 0; b < ww; ++b) {
          float v = in[((uint64_t)i * sh + a) * w + j * sw + b];
          best = v > best ? v : best;
        }
      out[(uint64_t)i * ow + j] = best;
    }
}

/* ftranspose: out[c,r] = in[r,c] for a 2-D tensor, bit-exact.  The reference only names the
 * builtin - include/polarai/core/internal/GenBuiltins.hpp:50 ("Transpose 2D tensor (matrix)"),
 * utils/dialects/include/PolarGraph/PolarGraphOps.td:507-527 (kernel body empty) - and holds no
 * test or vector for it: the restatement is the definition of a matrix transpose. */
void oracle_ftranspose(const float* in, uint64_t rows, uint64_t cols, float* out) {
  PAR_FOR
  for (int64_t r = 0; r < (int64_t)rows; ++r)
    for (uint64_t c = 0; c < cols; ++c) out[c * rows + (uint64_t)r] = in[(uint64_t)r * cols + c];
}

/* fslice: out = the sub-tensor at offset `index` of the first dimension, `inner` floats,
 * bit-exact.  GenBuiltins.hpp:49 ("Get subtensor"); PolarGraphOps.td:134-144 ("Get sub-tensor
 * by first dimension offset"); the result shape drops the first dimension
 * (utils/dialects/lib/PolarGraph/PolarGraphOps.cpp:157-170).  No reference test or vector. */
void oracle_fslice(const float* in, uint64_t inner, uint64_t index, float* out) {
  for (uint64_t i = 0; i < inner; ++i) out[i] = in[index * inner + i];
}

/* fconv2d: single-channel "valid" cross-correlation with an odd-sized kernel;
 * out[i,j] = sum over kernel rows a, columns b (in that order) of in[i+a, j+b]*ker[a,b],
 * each product rounded, then added; the result is [h-kh+1, w-kw+1].
 * Conv2DOp.cpp:35-90; src/operation/internal/Conv2DOperationInternal.cpp:34-39. */
void oracle_fconv2d(const float* in, uint64_t h, uint64_t w, const float* ker, uint64_t kh, uint64_t kw,
                    float* out) {
  const uint64_t oh = h - kh + 1, ow = w - kw + 1;
  PAR_FOR
  for (int64_t i = 0; i < (int64_t)oh; ++i)
    for (uint64_t j = 0; j < ow; ++j) {
      float acc = 0.0f;
      for (uint64_t a = 0; a < kh; ++a)
        for (uint64_t b = 0; b < kw; ++b) {
          float prod = in[((uint64_t)i + a) * w + j + b] * ker[a * kw + b];
          acc = prod + acc;
        }
      out[(uint64_t)i * ow + j] = acc;
    }
}

/* Index walk shared by the matmul forms: the left operand is stored [m,k] or,
 * transposed, [k,m]; the right one [k,n] or, transposed, [n,k].
 * kernels.h:80-117; MatMulOperation.cpp:17-51 (same strides). */
static inline void mm_strides(int tl, int tr, uint64_t m, uint64_t n, uint64_t k,
                              uint64_t row, uint64_t col, uint64_t* li,
                              uint64_t* ls, uint64_t* ri, uint64_t* rs) {
  if (!tl) { *ls = 1; *li = row * k; } else { *ls = m; *li = row; }
  if (!tr) { *rs = n; *ri = col; } else { *rs = 1; *ri = col * k; }
}

/* fmatmul, the reference's order: fp32 accumulator starting at 0, k ascending,
 * product rounded then added.  kernels.h:80-117; MatMulOp.cpp:36-85. */
void oracle_fmatmul(int tl, int tr, uint64_t m, uint64_t n, uint64_t k,
                    const float* left, const float* right, float* out) {
  PAR_FOR
  for (int64_t row = 0; row < (int64_t)m; ++row) {
    for (uint64_t col = 0; col < n; ++col) {
      uint64_t li, ls, ri, rs;
      mm_strides(tl, tr, m, n, k, (uint64_t)row, col, &li, &ls, &ri, &rs);
      float acc = 0.0f;
      for (uint64_t it = 0; it < k; ++it, li += ls, ri += rs) {
        float p = left[li] * right[ri];
        acc = acc + p;
      }
      out[(uint64_t)row * n + col] = acc;
    }
  }
}

/* The same sum carried in double, with sum_k |a||b| beside it: the yardstick a
 * differently ordered fp32 sum is measured against (|c - ref| / abs_sum). */
void oracle_fmatmul_f64(int tl, int tr, uint64_t m, uint64_t n, uint64_t k,
                        const float* left, const float* right, double* out,
                        double* abs_sum) {
  PAR_FOR
  for (int64_t row = 0; row < (int64_t)m; ++row) {
    for (uint64_t col = 0; col < n; ++col) {
      uint64_t li, ls, ri, rs;
      mm_strides(tl, tr, m, n, k, (uint64_t)row, col, &li, &ls, &ri, &rs);
      double acc = 0.0, mag = 0.0;
      for (uint64_t it = 0; it < k; ++it, li += ls, ri += rs) {
        double p = (double)left[li] * (double)right[ri];
        acc += p;
        mag += fabs(p);
      }
      out[(uint64_t)row * n + col] = acc;
      if (abs_sum) abs_sum[(uint64_t)row * n + col] = mag;
    }
  }
}

/* Selected entries (rows[i], cols[i]) of the double-accumulated product, for
 * sizes where the whole product is hours of CPU time. */
void oracle_fmatmul_entries_f64(int tl, int tr, uint64_t m, uint64_t n,
                                uint64_t k, const float* left,
                                const float* right, const uint64_t* rows,
                                const uint64_t* cols, uint64_t count,
                                double* out, double* abs_sum) {
  PAR_FOR
  for (int64_t e = 0; e < (int64_t)count; ++e) {
    uint64_t li, ls, ri, rs;
    mm_strides(tl, tr, m, n, k, rows[e], cols[e], &li, &ls, &ri, &rs);
    double acc = 0.0, mag = 0.0;
    for (uint64_t it = 0; it < k; ++it, li += ls, ri += rs) {
      double p = (double)left[li] * (double)right[ri];
      acc += p;
      mag += fabs(p);
    }
    out[e] = acc;
    if (abs_sum) abs_sum[e] = mag;
  }
}
