/*
 * Host harness (test infrastructure) that runs the reference's OpenCL C builtin
 * kernels - src/backend/generic/runtime/opencl/kernels.h:21-156, extracted at
 * build time into _ref/kernels_ocl.inc - as plain C on the CPU.  An OpenCL
 * NDRange of `size` work-items becomes a loop that sets the work-item id and
 * calls the kernel function once per id; OpenCL's float overloads of log, exp
 * and fabs become logf, expf and fabsf.  Compiled with -ffp-contract=off.
 *
 * The wrappers below only marshal arguments into the reference kernels'
 * parameter order; no arithmetic of the builtins is written here.
 */
#include <math.h>
#include <stdint.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef unsigned long ulong;
#define kernel
#define global
#define log(x) logf(x)
#define exp(x) expf(x)
#define fabs(x) fabsf(x)

static _Thread_local int tls_gid;
static _Thread_local int tls_gsize;
static inline int get_work_dim(void) { return 1; }
static inline int get_global_id(int d) { (void)d; return tls_gid; }
static inline int get_global_size(int d) { (void)d; return tls_gsize; }

/* glibc's libm exports narrowing functions called fadd and fmul; give the
 * kernel functions private names so that calls bind to the reference's code. */
#define ffill ocl_ffill
#define fadd ocl_fadd
#define fcopy ocl_fcopy
#define fdivide ocl_fdivide
#define flogloss ocl_flogloss
#define fmatmul ocl_fmatmul
#define fmul ocl_fmul
#define fmulconcat ocl_fmulconcat
#define fsigmoid ocl_fsigmoid

#include "_ref/kernels_ocl.inc"

#undef log
#undef exp
#undef fabs

static int g_threads = 1;
void ref_set_threads(int n) { g_threads = n < 1 ? 1 : n; }
int ref_max_threads(void) {
#ifdef _OPENMP
  return omp_get_num_procs();
#else
  return 1;
#endif
}

#define NDRANGE(count, call)                                                   \
  _Pragma("omp parallel for num_threads(g_threads) schedule(static)")          \
  for (int64_t gid_ = 0; gid_ < (int64_t)(count); ++gid_) {                    \
    tls_gid = (int)gid_;                                                       \
    tls_gsize = (int)(count);                                                  \
    call;                                                                      \
  }

void ref_ffill(float pattern, float* out, uint64_t n) {
  NDRANGE(n, ffill(pattern, n, out))
}
void ref_fcopy(const float* in, float* out, uint64_t n) {
  NDRANGE(n, fcopy(in, n, out))
}
void ref_fadd(const float* a, float sa, const float* b, float sb, float* out,
              uint64_t n) {
  NDRANGE(n, fadd(a, sa, b, sb, n, out))
}
void ref_fmul(const float* a, const float* b, float* out, uint64_t n) {
  NDRANGE(n, fmul(a, b, n, out))
}
void ref_fdivide(const float* num, const float* den, float* out, uint64_t n) {
  NDRANGE(n, fdivide(num, den, n, out))
}
void ref_fsigmoid(const float* in, float* out, uint64_t n) {
  NDRANGE(n, fsigmoid(in, n, out))
}
void ref_flogloss(const float* p, const float* y, float* out, uint64_t n) {
  NDRANGE(n, flogloss(p, y, n, out))
}
void ref_fmulconcat(const float* grad, const float* local, float* out,
                    uint64_t n) {
  NDRANGE(n, fmulconcat(grad, 1, local, n, out))
}
void ref_fmatmul(int tl, int tr, uint64_t m, uint64_t n, uint64_t k,
                 const float* left, const float* right, float* out) {
  NDRANGE(m * n, fmatmul((ulong)tl, (ulong)tr, m, n, k, left, right, out))
}
