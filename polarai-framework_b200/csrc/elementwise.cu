// Elementwise builtins for B200: ffill, fcopy, fadd, fmul, fdivide, fsigmoid,
// flogloss, fmulconcat, and the fsum reduction.
//
// All of them are HBM-bound streams (4 to 12 bytes per element, a few to a few
// tens of instructions).  One kernel template serves them: every thread moves
// 128-bit vectors, UNROLL independent vectors per input are in flight per
// thread before the first use, loads and stores carry the streaming
// (evict-first) cache hint because no element is touched twice.  Each CTA
// handles ONE tile of 256 x UNROLL vectors and exits: measured on B200 at 2^28
// elements, one tile per CTA streams 12-20 % faster than a grid of 4 CTAs per SM
// walking the array with a grid-stride loop (fadd 7.0 vs 6.2 TB/s, fcopy 6.8 vs
// 5.9, ffill 7.5 vs 6.1), whatever the block size, unroll or cache hint.
// Pointers that are not 16-byte aligned take a scalar kernel of the same shape.
//
// Arithmetic follows the reference bit for bit where IEEE allows it: fadd is
// two rounded multiplies and a rounded add (__fmul_rn/__fadd_rn forbid
// contraction into FMA), fdivide is IEEE division, fsigmoid and flogloss use
// the full-precision expf/logf (1 ulp), not the fast intrinsics.
#include "common.cuh"

namespace polar_b200 {
namespace {

constexpr int kThreads = 256;
constexpr int kCtasPerSm = 4;   // 1024 threads/SM: 64 registers per thread available
constexpr int kUnroll = 4;      // float4 vectors in flight per input per thread

struct FillOp {
  float v;
  __device__ __forceinline__ float operator()(float, float) const { return v; }
};
struct CopyOp {
  __device__ __forceinline__ float operator()(float a, float) const { return a; }
};
struct AddOp {
  float sa, sb;
  __device__ __forceinline__ float operator()(float a, float b) const {
    return __fadd_rn(__fmul_rn(a, sa), __fmul_rn(b, sb));
  }
};
struct MulOp {
  __device__ __forceinline__ float operator()(float a, float b) const { return __fmul_rn(a, b); }
};
struct DivOp {
  __device__ __forceinline__ float operator()(float a, float b) const { return __fdiv_rn(a, b); }
};
template <bool CLAMP>
struct SigmoidOp {
  __device__ __forceinline__ float operator()(float x, float) const {
    if (CLAMP) return sigmoid_clamped(x);
    return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-x)));
  }
};
struct LogLossOp {
  // out = fl(fl(-y * log(p + eps)) - fl((1 - y) * log(1 - p + eps))), eps = 1e-5: the general
  // form, two full-precision logarithms (scalar fallback kernel, and soft labels in the
  // vector kernel below).
  __device__ __forceinline__ float operator()(float p, float y) const {
    const float eps = 1e-5f;
    float t0 = __fmul_rn(-y, logf(__fadd_rn(p, eps)));
    float t1 = __fmul_rn(__fadd_rn(1.0f, -y), logf(__fadd_rn(__fadd_rn(1.0f, -p), eps)));
    return __fadd_rn(t0, -t1);
  }
};
// flogloss for labels that are exactly 0 or 1 (what LogLoss is fed): one of the two weights
// -y and 1-y is then an exact zero, and its product with a logarithm is a signed zero, NaN
// or NaN - whatever the logarithm's low bits are.  So only the OTHER logarithm needs full
// precision; the one under the zero weight comes from the special-function unit
// (lg2.approx), which returns the same NaN / -inf / +inf classes and the same sign.  (The
// sign of that zero is only visible when the full-precision term is itself zero, i.e. its
// argument is exactly 1; the two arguments sum to 1 + 2 eps, so the other one is then about
// 2e-5, far from where an approximate logarithm could have the wrong sign.)  Same bits as
// the two-logarithm form at roughly 60 % of its instructions - two full logf per element make
// the builtin issue-bound instead of HBM-bound.  Branch-free, so the unrolled elements
// interleave.
__device__ __forceinline__ float logloss_binary(float p, float y) {
  const float eps = 1e-5f;
  const float a0 = __fadd_rn(p, eps);
  const float a1 = __fadd_rn(__fadd_rn(1.0f, -p), eps);
  const float w0 = -y, w1 = __fadd_rn(1.0f, -y);
  const bool first = (w1 == 0.0f);                       // y == 1: log(a0) carries the result
  const float fine = logf(first ? a0 : a1);
  const float coarse = __logf(first ? a1 : a0);
  const float t0 = __fmul_rn(w0, first ? fine : coarse);
  const float t1 = __fmul_rn(w1, first ? coarse : fine);
  return __fadd_rn(t0, -t1);
}
// Extended builtin: the three launches the reference's Sigmoid derivative compiles to
// (SigmoidOperationInternal.cpp:107-135: fadd(ones,1,s,-1) -> fmul(.,s) -> fmul(grad,.))
// in one pass, with the same three roundings, so the result is bit-identical.
struct SigmoidGradOp {
  __device__ __forceinline__ float operator()(float g, float s) const {
    return sigmoid_grad_chain(g, s);
  }
};
// Extended builtin: dZ = dL/dP * dP/dZ for LogLoss on a Sigmoid output, the seven launches
// the reference's derivatives compile to (LogLossOperationInternal.cpp:127-170:
// fadd(p,1,y,-1), fmul(p,p), fadd(p,1,pp,-1), fdivide; SigmoidOperationInternal.cpp:107-135:
// fadd(ones,1,p,-1), fmul(.,p), fmul(dLdP,.)) in one pass with the same seven roundings.
struct SigmoidLogLossGradOp {
  __device__ __forceinline__ float operator()(float p, float y) const {
    const float pmy = __fadd_rn(__fmul_rn(p, 1.0f), __fmul_rn(y, -1.0f));
    const float pp = __fmul_rn(p, p);
    const float den = __fadd_rn(__fmul_rn(p, 1.0f), __fmul_rn(pp, -1.0f));
    const float dldp = __fdiv_rn(pmy, den);
    return sigmoid_grad_chain(dldp, p);
  }
};
struct ScaleByFirstOp {  // fmulconcat: the scalar is read once per thread
  float g;
  __device__ __forceinline__ float operator()(float l, float) const { return __fmul_rn(g, l); }
};

__device__ __forceinline__ float4 ld_stream(const float4* p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(float4* p, float4 v) { __stcs(p, v); }

// Per-op tile shape: vectors in flight per input per thread, and CTAs per SM the
// register budget must allow (flat between 2 and 8 vectors per thread for every builtin
// served by this template; flogloss has its own kernel below).
template <class Op> struct Shape { static constexpr int kUnroll = 4, kMinCtas = kCtasPerSm; };

// NIN = number of input streams (0, 1 or 2).
template <int NIN, class Op>
__global__ void __launch_bounds__(kThreads, Shape<Op>::kMinCtas)
ew_vec_kernel(Op op, const float* in0, const float* in1, float* out, uint64_t n) {
  constexpr int kUnroll = Shape<Op>::kUnroll;
  const uint64_t nvec = n >> 2;
  const float4* v0 = reinterpret_cast<const float4*>(in0);
  const float4* v1 = reinterpret_cast<const float4*>(in1);
  float4* vo = reinterpret_cast<float4*>(out);
  const uint64_t tile = (uint64_t)kThreads * kUnroll;
  {
    const uint64_t base = (uint64_t)blockIdx.x * tile;
    float4 a[kUnroll], b[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      uint64_t i = base + (uint64_t)u * kThreads + threadIdx.x;
      if (NIN >= 1 && i < nvec) a[u] = ld_stream(v0 + i);
      if (NIN >= 2 && i < nvec) b[u] = ld_stream(v1 + i);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      uint64_t i = base + (uint64_t)u * kThreads + threadIdx.x;
      if (i < nvec) {
        float4 r;
        r.x = op(NIN >= 1 ? a[u].x : 0.f, NIN >= 2 ? b[u].x : 0.f);
        r.y = op(NIN >= 1 ? a[u].y : 0.f, NIN >= 2 ? b[u].y : 0.f);
        r.z = op(NIN >= 1 ? a[u].z : 0.f, NIN >= 2 ? b[u].z : 0.f);
        r.w = op(NIN >= 1 ? a[u].w : 0.f, NIN >= 2 ? b[u].w : 0.f);
        st_stream(vo + i, r);
      }
    }
  }
  // ragged tail: the last n % 4 elements
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    uint64_t i = (nvec << 2) + threadIdx.x;
    out[i] = op(NIN >= 1 ? in0[i] : 0.f, NIN >= 2 ? in1[i] : 0.f);
  }
}

// flogloss, vector form: one tile per CTA like ew_vec_kernel.  A thread whose labels are all
// exactly 0 or 1 takes the one-logarithm arithmetic for its whole tile (one branch per
// thread, uniform for hard labels); any other label sends the thread to the general form.
constexpr int kLogLossUnroll = 4;
__global__ void __launch_bounds__(kThreads, kCtasPerSm)
logloss_vec_kernel(const float* predicted, const float* truth, float* out, uint64_t n) {
  const uint64_t nvec = n >> 2;
  const float4* vp = reinterpret_cast<const float4*>(predicted);
  const float4* vy = reinterpret_cast<const float4*>(truth);
  float4* vo = reinterpret_cast<float4*>(out);
  const uint64_t base = (uint64_t)blockIdx.x * kThreads * kLogLossUnroll;
  float4 p[kLogLossUnroll], y[kLogLossUnroll];
  bool binary = true;
#pragma unroll
  for (int u = 0; u < kLogLossUnroll; ++u) {
    const uint64_t i = base + (uint64_t)u * kThreads + threadIdx.x;
    if (i < nvec) {
      p[u] = ld_stream(vp + i);
      y[u] = ld_stream(vy + i);
    } else {
      p[u] = make_float4(0.5f, 0.5f, 0.5f, 0.5f);
      y[u] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
#pragma unroll
  for (int u = 0; u < kLogLossUnroll; ++u) {
    const float w[4] = {y[u].x, y[u].y, y[u].z, y[u].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) binary = binary && (w[j] == 0.0f || w[j] == 1.0f);
  }
  LogLossOp general;
#pragma unroll
  for (int u = 0; u < kLogLossUnroll; ++u) {
    const uint64_t i = base + (uint64_t)u * kThreads + threadIdx.x;
    float4 r;
    if (binary) {
      r.x = logloss_binary(p[u].x, y[u].x);
      r.y = logloss_binary(p[u].y, y[u].y);
      r.z = logloss_binary(p[u].z, y[u].z);
      r.w = logloss_binary(p[u].w, y[u].w);
    } else {
      r.x = general(p[u].x, y[u].x);
      r.y = general(p[u].y, y[u].y);
      r.z = general(p[u].z, y[u].z);
      r.w = general(p[u].w, y[u].w);
    }
    if (i < nvec) st_stream(vo + i, r);
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    const uint64_t i = (nvec << 2) + threadIdx.x;
    out[i] = general(predicted[i], truth[i]);
  }
}

template <int NIN, class Op>
__global__ void __launch_bounds__(kThreads, kCtasPerSm)
ew_scalar_kernel(Op op, const float* in0, const float* in1, float* out, uint64_t n) {
  const uint64_t stride = (uint64_t)gridDim.x * kThreads;
  for (uint64_t i = (uint64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) {
    out[i] = op(NIN >= 1 ? in0[i] : 0.f, NIN >= 2 ? in1[i] : 0.f);
  }
}

// fmulconcat reads its scalar from device memory inside the kernel.
__global__ void __launch_bounds__(kThreads, kCtasPerSm)
mulconcat_vec_kernel(const float* gradient, const float* local, float* out, uint64_t n) {
  const float g = gradient[0];
  ScaleByFirstOp op{g};
  const uint64_t nvec = n >> 2;
  const float4* v0 = reinterpret_cast<const float4*>(local);
  float4* vo = reinterpret_cast<float4*>(out);
  const uint64_t tile = (uint64_t)kThreads * kUnroll;
  {
    const uint64_t base = (uint64_t)blockIdx.x * tile;
    float4 a[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      uint64_t i = base + (uint64_t)u * kThreads + threadIdx.x;
      if (i < nvec) a[u] = ld_stream(v0 + i);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      uint64_t i = base + (uint64_t)u * kThreads + threadIdx.x;
      if (i < nvec) {
        float4 r = {op(a[u].x, 0.f), op(a[u].y, 0.f), op(a[u].z, 0.f), op(a[u].w, 0.f)};
        st_stream(vo + i, r);
      }
    }
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    uint64_t i = (nvec << 2) + threadIdx.x;
    out[i] = op(local[i], 0.f);
  }
}

__global__ void __launch_bounds__(kThreads, kCtasPerSm)
mulconcat_scalar_kernel(const float* gradient, const float* local, float* out, uint64_t n) {
  const float g = gradient[0];
  const uint64_t stride = (uint64_t)gridDim.x * kThreads;
  for (uint64_t i = (uint64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride)
    out[i] = __fmul_rn(g, local[i]);
}

// fsum: per-thread double partials, warp shuffle, one atomicAdd(double) per block.
__global__ void __launch_bounds__(kThreads, kCtasPerSm)
sum_kernel(const float* in, double* sum, uint64_t n, int vec_ok) {
  double acc = 0.0;
  if (vec_ok) {
    const uint64_t nvec = n >> 2;
    const float4* v = reinterpret_cast<const float4*>(in);
    const uint64_t stride = (uint64_t)gridDim.x * kThreads;
    for (uint64_t i = (uint64_t)blockIdx.x * kThreads + threadIdx.x; i < nvec; i += stride) {
      float4 x = ld_stream(v + i);
      acc += (double)((x.x + x.y) + (x.z + x.w));
    }
    if (blockIdx.x == 0 && threadIdx.x < (n & 3)) acc += (double)in[(nvec << 2) + threadIdx.x];
  } else {
    const uint64_t stride = (uint64_t)gridDim.x * kThreads;
    for (uint64_t i = (uint64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride)
      acc += (double)in[i];
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  __shared__ double warp_sums[kThreads / 32];
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    double w = threadIdx.x < kThreads / 32 ? warp_sums[threadIdx.x] : 0.0;
#pragma unroll
    for (int off = 4; off > 0; off >>= 1) w += __shfl_xor_sync(0xffffffffu, w, off);
    if (threadIdx.x == 0) atomicAdd(sum, w);
  }
}

// fsum as a builtin with a tensor result: stage 1 leaves one double per CTA in scratch, stage 2
// (one CTA) adds them in index order and stores the rounded float - the same bits run to run.
__global__ void __launch_bounds__(kThreads, kCtasPerSm)
sum_partials_kernel(const float* in, double* partials, uint64_t n, int vec_ok) {
  double acc = 0.0;
  const uint64_t stride = (uint64_t)gridDim.x * kThreads;
  if (vec_ok) {
    const uint64_t nvec = n >> 2;
    const float4* v = reinterpret_cast<const float4*>(in);
    for (uint64_t i = (uint64_t)blockIdx.x * kThreads + threadIdx.x; i < nvec; i += stride) {
      float4 x = ld_stream(v + i);
      acc += (double)((x.x + x.y) + (x.z + x.w));
    }
    if (blockIdx.x == 0 && threadIdx.x < (n & 3)) acc += (double)in[(nvec << 2) + threadIdx.x];
  } else {
    for (uint64_t i = (uint64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) acc += (double)in[i];
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  __shared__ double warp_sums[kThreads / 32];
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double w = 0.0;
    for (int i = 0; i < kThreads / 32; ++i) w += warp_sums[i];
    partials[blockIdx.x] = w;
  }
}
__global__ void __launch_bounds__(32) sum_finish_kernel(const double* partials, uint32_t count, float* out) {
  if (threadIdx.x == 0) {
    double s = 0.0;
    for (uint32_t i = 0; i < count; ++i) s += partials[i];
    out[0] = (float)s;
  }
}

// Grid-stride kernels (scalar fallback, fsum): a few CTAs per SM.
unsigned grid_for(uint64_t work_items, uint64_t per_cta) {
  uint64_t need = (work_items + per_cta - 1) / per_cta;
  uint64_t cap = (uint64_t)sm_count() * kCtasPerSm;
  if (need < 1) need = 1;
  return (unsigned)(need < cap ? need : cap);
}
// One tile per CTA (vector kernels).
unsigned tiles_for(uint64_t nvec, int unroll = kUnroll) {
  uint64_t per_cta = (uint64_t)kThreads * unroll;
  uint64_t need = (nvec + per_cta - 1) / per_cta;
  return (unsigned)(need < 1 ? 1 : need);
}

template <int NIN, class Op>
int launch_ew(const char* name, Op op, const float* in0, const float* in1, float* out,
              uint64_t n, void* stream) {
  clear_error();
  if (n == 0) return POLAR_B200_OK;
  if (!out || (NIN >= 1 && !in0) || (NIN >= 2 && !in1))
    return fail(POLAR_B200_ERR_INVALID, "null device pointer");
  if (n > (1ull << 40)) return fail(POLAR_B200_ERR_INVALID, "element count too large");
  LaunchDeviceScope on(stream, out);
  bool vec = aligned16(out) && (NIN < 1 || aligned16(in0)) && (NIN < 2 || aligned16(in1)) && n >= 4;
  if (vec) {
    unsigned grid = tiles_for(n >> 2, Shape<Op>::kUnroll);
    ew_vec_kernel<NIN, Op><<<grid, kThreads, 0, as_stream(stream)>>>(op, in0, in1, out, n);
  } else {
    unsigned grid = grid_for(n, kThreads);
    ew_scalar_kernel<NIN, Op><<<grid, kThreads, 0, as_stream(stream)>>>(op, in0, in1, out, n);
  }
  return check_launch(name);
}

}  // namespace
}  // namespace polar_b200

using namespace polar_b200;

extern "C" {

int polar_b200_ffill(float pattern, float* out, uint64_t n, void* stream) {
  return launch_ew<0>("ffill", FillOp{pattern}, nullptr, nullptr, out, n, stream);
}
int polar_b200_fcopy(const float* in, float* out, uint64_t n, void* stream) {
  return launch_ew<1>("fcopy", CopyOp{}, in, nullptr, out, n, stream);
}
int polar_b200_fadd(const float* a, float scaleA, const float* b, float scaleB, float* out,
                    uint64_t n, void* stream) {
  return launch_ew<2>("fadd", AddOp{scaleA, scaleB}, a, b, out, n, stream);
}
int polar_b200_fmul(const float* a, const float* b, float* out, uint64_t n, void* stream) {
  return launch_ew<2>("fmul", MulOp{}, a, b, out, n, stream);
}
int polar_b200_fdivide(const float* numerator, const float* denominator, float* out, uint64_t n,
                       void* stream) {
  return launch_ew<2>("fdivide", DivOp{}, numerator, denominator, out, n, stream);
}
int polar_b200_fsigmoid(const float* in, float* out, uint64_t n, void* stream) {
  return launch_ew<1>("fsigmoid", SigmoidOp<true>{}, in, nullptr, out, n, stream);
}
int polar_b200_fsigmoid_unclamped(const float* in, float* out, uint64_t n, void* stream) {
  return launch_ew<1>("fsigmoid_unclamped", SigmoidOp<false>{}, in, nullptr, out, n, stream);
}
int polar_b200_flogloss(const float* predicted, const float* groundTruth, float* out, uint64_t n,
                        void* stream) {
  if (n >= 4 && predicted && groundTruth && out && n <= (1ull << 40) && aligned16(predicted) &&
      aligned16(groundTruth) && aligned16(out)) {
    clear_error();
    LaunchDeviceScope on(stream, out);
    logloss_vec_kernel<<<tiles_for(n >> 2, kLogLossUnroll), kThreads, 0, as_stream(stream)>>>(predicted, groundTruth,
                                                                                            out, n);
    return check_launch("flogloss");
  }
  return launch_ew<2>("flogloss", LogLossOp{}, predicted, groundTruth, out, n, stream);   // null, empty, unaligned
}

int polar_b200_fsigmoid_grad(const float* gradient, const float* sigmoidOut, float* out, uint64_t n,
                             void* stream) {
  return launch_ew<2>("fsigmoid_grad", SigmoidGradOp{}, gradient, sigmoidOut, out, n, stream);
}

int polar_b200_fsigmoid_logloss_grad(const float* predicted, const float* groundTruth, float* out, uint64_t n,
                                     void* stream) {
  return launch_ew<2>("fsigmoid_logloss_grad", SigmoidLogLossGradOp{}, predicted, groundTruth, out, n, stream);
}

int polar_b200_fmulconcat(const float* gradient, const float* localDerivative, float* out,
                          uint64_t n, void* stream) {
  clear_error();
  if (n == 0) return POLAR_B200_OK;
  if (!gradient || !localDerivative || !out) return fail(POLAR_B200_ERR_INVALID, "null device pointer");
  if (n > (1ull << 40)) return fail(POLAR_B200_ERR_INVALID, "element count too large");
  LaunchDeviceScope on(stream, out);
  if (aligned16(localDerivative) && aligned16(out) && n >= 4) {
    unsigned grid = tiles_for(n >> 2);
    mulconcat_vec_kernel<<<grid, kThreads, 0, as_stream(stream)>>>(gradient, localDerivative, out, n);
  } else {
    unsigned grid = grid_for(n, kThreads);
    mulconcat_scalar_kernel<<<grid, kThreads, 0, as_stream(stream)>>>(gradient, localDerivative, out, n);
  }
  return check_launch("fmulconcat");
}

int polar_b200_fsum(const float* in, double* sum, uint64_t n, void* stream) {
  clear_error();
  if (!sum) return fail(POLAR_B200_ERR_INVALID, "null sum pointer");
  if (n == 0) return POLAR_B200_OK;
  if (!in) return fail(POLAR_B200_ERR_INVALID, "null device pointer");
  LaunchDeviceScope on(stream, in);
  int vec_ok = aligned16(in) && n >= 4;
  unsigned grid = grid_for(vec_ok ? (n >> 2) : n, (uint64_t)kThreads * 8);
  sum_kernel<<<grid, kThreads, 0, as_stream(stream)>>>(in, sum, n, vec_ok);
  return check_launch("fsum");
}

uint64_t polar_b200_fsum_f32_workspace_bytes(uint64_t n) {
  // one double per CTA; the grid depends on n alone (not on the pointer's alignment)
  return (uint64_t)grid_for(n >> 2, (uint64_t)kThreads * 8) * sizeof(double);
}

int polar_b200_fsum_f32(const float* in, float* out, uint64_t n, void* workspace, uint64_t workspace_bytes,
                        void* stream) {
  clear_error();
  if (!out) return fail(POLAR_B200_ERR_INVALID, "null result pointer");
  if (n == 0) return polar_b200_ffill(0.0f, out, 1, stream);
  if (!in) return fail(POLAR_B200_ERR_INVALID, "null device pointer");
  LaunchDeviceScope on(stream, in);
  const int vec_ok = aligned16(in) && n >= 4;
  const unsigned grid = grid_for(n >> 2, (uint64_t)kThreads * 8);
  const uint64_t need = (uint64_t)grid * sizeof(double);
  cudaStream_t st = as_stream(stream);
  double* partials = static_cast<double*>(workspace);
  bool own = false;
  if (!partials) {
    cudaError_t e = cudaMallocAsync(reinterpret_cast<void**>(&partials), need, st);
    if (e != cudaSuccess) return fail(POLAR_B200_ERR_CUDA, "cudaMallocAsync(fsum partial sums)", e);
    own = true;
  } else if (workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 7)) {
    return fail(POLAR_B200_ERR_WORKSPACE, "fsum needs 8-byte aligned workspace of polar_b200_fsum_f32_workspace_bytes");
  }
  sum_partials_kernel<<<grid, kThreads, 0, st>>>(in, partials, n, vec_ok);
  int rc = check_launch("fsum_partials");
  if (rc == POLAR_B200_OK) {
    sum_finish_kernel<<<1, 32, 0, st>>>(partials, grid, out);
    rc = check_launch("fsum");
  }
  if (own) cudaFreeAsync(partials, st);
  return rc;
}

}  // extern "C"
