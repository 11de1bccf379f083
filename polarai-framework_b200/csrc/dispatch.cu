// fmatmul entry points and dispatch by native kernel name.
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace polar_b200 {
int launch_ffma(int tl, int tr, uint64_t m, uint64_t n, uint64_t k, const float* left,
                const float* right, float* out, cudaStream_t stream);
int launch_tc(int tl, int tr, uint64_t m, uint64_t n, uint64_t k, const float* left,
              const float* right, float* out, int bn, int bk, int passes, int write_hi, float* ws,
              uint32_t splits, int epilogue, cudaStream_t stream, uint64_t left_pitch = 0, int mt = 1,
              int swap_ab = 0);
uint32_t tc_default_splits(uint64_t m, uint64_t n, uint64_t k, int mt = 1);
bool tc_tail_in_halves(uint64_t tiles, uint64_t grid);
uint64_t tc_workspace_bytes(uint64_t m, uint64_t n, uint64_t k, uint32_t splits, int mt = 1);
bool tc_shape_ok(int tl, int tr, uint64_t m, uint64_t n, uint64_t k, const float* left,
                 const float* right);
int skinny_kind(int tl, int tr, uint64_t m, uint64_t n, uint64_t k, const float* left,
                const float* right, const float* out);
uint64_t skinny_workspace_bytes(int kind, uint64_t m, uint64_t n, uint64_t k);
int launch_skinny(int kind, int tl, int tr, uint64_t m, uint64_t n, uint64_t k, const float* left,
                  const float* right, float* out, float* ws, cudaStream_t st, const float* sig, int sigmoid_out = 0);
bool dense_grad_ok(uint64_t rows, uint64_t kh, uint64_t n, const float* H, const float* din);
uint64_t dense_grad_workspace_bytes(uint64_t rows, uint64_t kh, uint64_t n);
int launch_dense_grad(const float* H, const float* dz, const float* W, float* din, float* dw, float* ws,
                      uint64_t rows, uint64_t kh, uint64_t n, cudaStream_t st);
uint64_t ragged_rows_workspace_bytes(uint64_t rem, uint64_t n, uint64_t k);
int launch_ragged_rows(const float* left_tail, uint64_t left_pitch, const float* right, float* out_tail,
                       float* ws, uint64_t rem, uint64_t n, uint64_t k, cudaStream_t st);

namespace {

enum Path { kPathTc = 0, kPathSkinny = 1, kPathFfma = 2 };

// Tensor-core tiles are 128 x 256 (or 128 x 128): below one tile in either
// output dimension, or with a k extent shorter than a slab, the CUDA-core
// kernel does less wasted work.
int choose_path(int tl, int tr, uint64_t m, uint64_t n, uint64_t k, const float* left,
                const float* right, const float* out) {
  if (skinny_kind(tl, tr, m, n, k, left, right, out)) return kPathSkinny;
  if (tc_shape_ok(tl, tr, m, n, k, left, right) && m >= 64 && n >= 32 && k >= 32) return kPathTc;
  return kPathFfma;
}

// The tensor-core path with `splits` work units per tile; scratch for the partial
// products comes from the caller's workspace or, without one, from the
// stream-ordered pool.
int run_tc(int tl, int tr, uint64_t m, uint64_t n, uint64_t k, const float* left, const float* right,
           float* out, int bn, int bk, int passes, int write_hi, uint32_t splits, void* workspace,
           uint64_t workspace_bytes, cudaStream_t stream, int epilogue = 0, uint64_t left_pitch = 0,
           int mt = 1, int swap_ab = 0) {
  if (splits == 1)
    return launch_tc(tl, tr, m, n, k, left, right, out, bn, bk, passes, write_hi, nullptr, 1, epilogue, stream,
                     left_pitch, mt, swap_ab);
  // splits == 0 is the stream mode of the 256-column tile configurations
  if (splits == 0 && bn != 256) splits = 1;
  const uint64_t need = splits == 0 ? tc_workspace_bytes(m, n, k, 0, mt) : (uint64_t)splits * m * n * sizeof(float);
  if (need == 0)   // stream mode asked for a shape it does not suit
    return launch_tc(tl, tr, m, n, k, left, right, out, bn, bk, passes, write_hi, nullptr, 1, epilogue, stream,
                     left_pitch, mt, swap_ab);
  if (workspace) {
    if (workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 15))
      return fail(POLAR_B200_ERR_WORKSPACE, "workspace too small or not 16-byte aligned");
    return launch_tc(tl, tr, m, n, k, left, right, out, bn, bk, passes, write_hi, static_cast<float*>(workspace),
                     splits, epilogue, stream, left_pitch, mt, swap_ab);
  }
  void* ws = nullptr;
  cudaError_t e = cudaMallocAsync(&ws, need, stream);
  if (e != cudaSuccess) return fail(POLAR_B200_ERR_CUDA, "cudaMallocAsync(workspace)", e);
  int rc = launch_tc(tl, tr, m, n, k, left, right, out, bn, bk, passes, write_hi, static_cast<float*>(ws), splits,
                     epilogue, stream, left_pitch, mt, swap_ab);
  e = cudaFreeAsync(ws, stream);
  if (rc == POLAR_B200_OK && e != cudaSuccess) return fail(POLAR_B200_ERR_CUDA, "cudaFreeAsync(workspace)", e);
  return rc;
}

// A t_f product whose row count is a few rows past a multiple of the 128-row tile would
// spend a whole tile row of tensor-core work on them (784 rows: 7 tile rows for 6.1 of
// work).  Those rows go to the bandwidth-bound kernel instead, which reads `right` once
// more - on a second stream of the library's own, forked from and joined back into the
// caller's stream, so that the pass runs WHILE the tensor-core kernel computes the whole
// tile rows (the two write disjoint rows of the result and use disjoint halves of the
// scratch).  Run one after the other the extra pass only paid for long sums; overlapped it
// pays whenever the tensor-core part lasts longer than the pass, i.e. from a few thousand k.
// Returns the number of such rows (0: not applicable).
uint64_t ragged_rows(int tl, int tr, uint64_t m, uint64_t n, uint64_t k, const float* right, int fused) {
  const uint64_t rem = m & 127;
  if (!tl || tr || fused != 0 || m <= 128 || rem == 0 || rem > 16) return 0;
  if ((n & 3) != 0 || !aligned16(right) || k < 4096) return 0;
  return rem;
}

// The library's side stream of the current device, with the two events of a fork/join.
// Created on first use (make that use outside stream capture: the warm-up call does).
struct SideStream {
  cudaStream_t stream = nullptr;
  cudaEvent_t fork = nullptr, join = nullptr;
};
SideStream* side_stream() {
  static SideStream per_device[64];
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> g(mu);
  SideStream& s = per_device[dev];
  if (!s.stream) {
    if (cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&s.fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&s.join, cudaEventDisableTiming) != cudaSuccess) {
      cudaGetLastError();
      s = SideStream{};
      return nullptr;
    }
  }
  return &s;
}

inline uint64_t align256(uint64_t b) { return (b + 255) & ~255ull; }

// How the tensor-core path runs one product.
//  mt: row sub-tiles per CTA tile.  256 x 256 tiles (2) fetch a third fewer operand bytes per
//    flop than 128 x 256 (1) and are 12-50 % faster on long sums (8192^3: 285 vs 242 TFLOP/s,
//    t_f 275 vs 180), but pad the tile rows to a multiple of 256, cannot overlap a tile's epilogue
//    with the next tile's k loop (both accumulators belong to one tile), and make half as many
//    tiles, which matters when those fill the last wave badly and k is too short to cut.
//  swap: the operands exchange roles (launch_tc), which turns the epilogue's stores into whole
//    128-byte lines: 2-4 % on sums of a few hundred to a few thousand terms, where the epilogue
//    is a visible share of a tile; needs whole tiles or fixed k cuts, and no row pitch.
//  splits: as tc_default_splits, for the orientation chosen.
// The choice compares padded tile area x relative cost / wave efficiency of the candidates.
struct TcChoice {
  int mt;
  int swap;
  uint32_t splits;
};

TcChoice tc_choose(uint64_t m, uint64_t n, uint64_t k, bool may_swap) {
  const double sms = (double)sm_count();
  TcChoice best{1, 0, 1};
  double best_est = 0.0;
  for (int swap = 0; swap <= (may_swap && k >= 256 && k <= 2048 ? 1 : 0); ++swap) {
    const uint64_t rows_dim = swap ? n : m, cols_dim = swap ? m : n;
    for (int mt = 1; mt <= 2; ++mt) {
      if (mt == 2 && (rows_dim < 256 || k < 512)) continue;
      const uint64_t rows = 128ull * mt;
      const uint64_t tiles_m = (rows_dim + rows - 1) / rows, tiles_n = (cols_dim + 255) / 256, tiles = tiles_m * tiles_n;
      uint32_t splits = tc_default_splits(rows_dim, cols_dim, k, mt);
      if (swap && splits == 0) splits = 1;             // stream mode stores through slots: whole tiles instead
      // with cuts of k the exchanged epilogue only writes partial products; measured better at
      // 2048^3 (206-217 vs 193 TFLOP/s) and worse at 1024^3 (48 vs 58), where stream mode stays
      if (swap && splits > 1 && rows_dim * cols_dim < (4ull << 20)) continue;
      double eff = 1.0;
      const uint64_t units = tiles * (splits ? splits : 1);
      if (splits >= 1 && (double)units < 8 * sms) {    // whole waves of work units (stream mode balances itself)
        double waves = (double)((units + (uint64_t)sms - 1) / (uint64_t)sms);
        // a tail of at most half a wave of whole tiles runs as column halves, which last about 0.6 of a tile
        if (splits == 1 && tc_tail_in_halves(tiles, (uint64_t)sms)) waves -= 0.4;
        eff = (double)units / (waves * sms);
      }
      // measured against the 128-row tile: 0.67-0.85 of its cost from k = 16384 up, 0.83-0.88 at
      // k = 784 ... 8192 (256-bit or line-wide stores in the epilogue)
      double cost = mt == 1 ? 1.0 : (k < 16384 ? 0.85 : 0.75);
      if (swap) cost *= 0.97;
      const double est = (double)(tiles_m * rows) * (double)(tiles_n * 256) * cost / eff;
      if (best_est == 0.0 || est < best_est) {
        best_est = est;
        best = TcChoice{mt, swap, splits};
      }
    }
  }
  return best;
}

int check_mm(int tl, int tr, uint64_t m, uint64_t n, uint64_t k, const float* left,
             const float* right, float* out) {
  if ((tl != 0 && tl != 1) || (tr != 0 && tr != 1))
    return fail(POLAR_B200_ERR_INVALID, "transpose flags must be 0 or 1");
  if (m > (1ull << 31) || n > (1ull << 31) || k > (1ull << 31))
    return fail(POLAR_B200_ERR_INVALID, "matrix dimension too large");
  if (m * n != 0 && !out) return fail(POLAR_B200_ERR_INVALID, "null output pointer");
  if (m * n != 0 && k != 0 && (!left || !right)) return fail(POLAR_B200_ERR_INVALID, "null operand pointer");
  return POLAR_B200_OK;
}

}  // namespace
}  // namespace polar_b200

using namespace polar_b200;

extern "C" {

// Scratch a matmul launch needs; `fused` as in fmatmul_impl below (only the sigmoid epilogue
// of the tensor-core kernel changes the answer: it keeps rows past a tile boundary on the
// tensor cores).
static uint64_t workspace_need(int tl, int tr, uint64_t m, uint64_t n, uint64_t k, int fused, bool pitched = false) {
  const float* al = reinterpret_cast<const float*>(256);   // allocator buffers are 256-byte aligned
  int kind = skinny_kind(tl, tr, m, n, k, al, al, al);
  if (kind) return skinny_workspace_bytes(kind, m, n, k);
  if (choose_path(tl, tr, m, n, k, al, al, al) == kPathTc) {
    const uint64_t rem = ragged_rows(tl, tr, m, n, k, al, fused == 1 ? 1 : 0);
    const uint64_t mm = m - rem;
    const TcChoice c = tc_choose(mm, n, k, rem == 0 && !pitched);
    uint64_t need = c.swap ? tc_workspace_bytes(n, mm, k, c.splits, c.mt) : tc_workspace_bytes(mm, n, k, c.splits, c.mt);
    // the two parts run at the same time: the ragged rows' scratch follows the tiles' scratch
    if (rem) need = align256(need) + ragged_rows_workspace_bytes(rem, n, k);
    return need;
  }
  return 0;
}

uint64_t polar_b200_fmatmul_workspace_bytes(int tl, int tr, uint64_t m, uint64_t n, uint64_t k) {
  return workspace_need(tl, tr, m, n, k, 0);
}

int polar_b200_result_count(const char* name) { return name && !std::strcmp(name, "fdense_grad") ? 2 : 1; }

uint64_t polar_b200_launch_workspace_bytes(const char* name, const polar_b200_arg* a, uint64_t argc) {
  if (name && a && !std::strcmp(name, "fmatmul_t_f_rows") && argc == 5 && a[0].is_tensor && a[1].is_tensor &&
      a[0].tensor.dims == 2 && a[1].tensor.dims == 2 && a[0].tensor.shape && a[1].tensor.shape && !a[3].is_tensor)
    return polar_b200_fmatmul_t_f_rows_workspace_bytes((uint64_t)a[3].scalar, a[1].tensor.shape[1], a[0].tensor.shape[0]);
  if (name && a && !std::strcmp(name, "fdense_grad") && argc == 5 && a[0].is_tensor && a[1].is_tensor &&
      a[0].tensor.dims == 2 && a[1].tensor.dims == 2 && a[0].tensor.shape && a[1].tensor.shape)
    return polar_b200_fdense_grad_workspace_bytes(a[0].tensor.shape[0], a[1].tensor.shape[0], a[0].tensor.shape[1]);
  if (name && a && !std::strcmp(name, "fsum") && argc == 2 && a[0].is_tensor && (!a[0].tensor.dims || a[0].tensor.shape)) {
    uint64_t n = 1;
    for (uint64_t d = 0; d < a[0].tensor.dims; ++d) n *= a[0].tensor.shape[d];
    return polar_b200_fsum_f32_workspace_bytes(n);
  }
  if (!name || !a || std::strncmp(name, "fmatmul_", 8) || std::strlen(name) < 11 || argc < 3) return 0;
  const char* suffix = name + 11;
  const int fused = !*suffix ? 0 : !std::strcmp(suffix, "_sigmoid") ? 1 : !std::strcmp(suffix, "_sigmoid_grad") ? 2 : -1;
  if (fused < 0 || !a[0].is_tensor || !a[1].is_tensor || a[0].tensor.dims != 2 || a[1].tensor.dims != 2) return 0;
  const int tl = name[8] == 't', tr = name[10] == 't';
  const polar_b200_tensor &l = a[0].tensor, &r = a[1].tensor;
  const uint64_t m = tl ? l.shape[1] : l.shape[0], k = tl ? l.shape[0] : l.shape[1];
  const uint64_t n = tr ? r.shape[0] : r.shape[1];
  return workspace_need(tl, tr, m, n, k, fused);
}

int polar_b200_fmatmul_path(int tl, int tr, uint64_t m, uint64_t n, uint64_t k) {
  // Alignment of the operands is assumed (allocator buffers are 256-byte aligned).
  const float* al = reinterpret_cast<const float*>(256);
  return choose_path(tl, tr, m, n, k, al, al, al);
}

void polar_b200_fmatmul_tc_plan(int tl, int tr, uint64_t m, uint64_t n, uint64_t k, int* tile_rows, int* exchanged,
                                int* splits) {
  const float* al = reinterpret_cast<const float*>(256);
  const uint64_t rem = ragged_rows(tl, tr, m, n, k, al, 0);
  const TcChoice c = tc_choose(m - rem, n, k, rem == 0);
  if (tile_rows) *tile_rows = 128 * c.mt;
  if (exchanged) *exchanged = c.swap;
  if (splits) *splits = (int)c.splits;
}

// The tensor-core path of one product: whole tiles on the tcgen05 kernel, rows just past a tile
// boundary of a t_f product beside it on the bandwidth-bound kernel.  `pitch` (t_f only; 0 = m)
// is the number of floats between consecutive k rows of the stored left operand: a value above
// m makes the product one over COLUMNS [0, m) of a wider stored matrix, i.e. over a block of
// rows of the full result.
static int tc_path(int tl, int tr, uint64_t m, uint64_t n, uint64_t k, const float* left, const float* right,
                   float* out, void* workspace, uint64_t workspace_bytes, void* stream, int fused, uint64_t pitch) {
  int rc = POLAR_B200_OK;
  const uint64_t lp = pitch ? pitch : m;
  const uint64_t rem = ragged_rows(tl, tr, m, n, k, right, fused);
  if (rem == 0) {
    const TcChoice c = tc_choose(m, n, k, pitch == 0);
    return run_tc(tl, tr, m, n, k, left, right, out, 256, 16, 3, 0, c.splits, workspace,
                  workspace_bytes, as_stream(stream), fused == 1 ? 1 : 0, pitch, c.mt, c.swap);
  }
  // whole tile rows on the tensor cores (left is stored [k, m]: the first m - rem columns
  // of rows of pitch m), the last `rem` rows on the bandwidth-bound kernel, concurrently
  const uint64_t mm = m - rem;
  const TcChoice c = tc_choose(mm, n, k, false);
  const int mt = c.mt;
  const uint64_t tc_need = align256(tc_workspace_bytes(mm, n, k, c.splits, mt));
  const uint64_t rag_need = ragged_rows_workspace_bytes(rem, n, k);
  cudaStream_t main_stream = as_stream(stream);
  void* own = nullptr;
  char* ws = static_cast<char*>(workspace);
  if (ws) {
    if (workspace_bytes < tc_need + rag_need || (reinterpret_cast<uintptr_t>(workspace) & 15))
      return fail(POLAR_B200_ERR_WORKSPACE, "workspace too small or not 16-byte aligned");
  } else {
    cudaError_t e = cudaMallocAsync(&own, tc_need + rag_need, main_stream);
    if (e != cudaSuccess) return fail(POLAR_B200_ERR_CUDA, "cudaMallocAsync(workspace)", e);
    ws = static_cast<char*>(own);
  }
  // fork: the side stream starts where the caller's stream is now (one fork/join at a time
  // per process: the side stream's two events are shared)
  static std::mutex fork_mutex;
  std::lock_guard<std::mutex> fork_guard(fork_mutex);
  SideStream* side = side_stream();
  cudaStream_t rag_stream = main_stream;
  if (side && cudaEventRecord(side->fork, main_stream) == cudaSuccess &&
      cudaStreamWaitEvent(side->stream, side->fork, 0) == cudaSuccess) {
    rag_stream = side->stream;
  } else {
    cudaGetLastError();   // no side stream: one after the other on the caller's stream
  }
  rc = launch_ragged_rows(left + mm, lp, right, out + mm * n, reinterpret_cast<float*>(ws + tc_need), rem, n, k,
                          rag_stream);
  int rc2 = run_tc(tl, tr, mm, n, k, left, right, out, 256, 16, 3, 0, c.splits,
                   tc_need ? ws : nullptr, tc_need, main_stream, 0, lp, mt);
  // join: whatever follows on the caller's stream waits for the side stream too (also when a
  // launch failed: a fork must never be left open, least of all under stream capture)
  if (rag_stream != main_stream) {
    if (cudaEventRecord(side->join, rag_stream) != cudaSuccess ||
        cudaStreamWaitEvent(main_stream, side->join, 0) != cudaSuccess) {
      cudaError_t e = cudaGetLastError();
      if (!rc && !rc2) rc = fail(POLAR_B200_ERR_CUDA, "joining the side stream", e);
    }
  }
  if (own) {
    cudaError_t e = cudaFreeAsync(own, main_stream);
    if (!rc && !rc2 && e != cudaSuccess) rc = fail(POLAR_B200_ERR_CUDA, "cudaFreeAsync(workspace)", e);
  }
  return rc ? rc : rc2;
}

// fused == 0: out = L.R;  1: out = fsigmoid(L.R);  2: out = (L.R) * ((1 - sig) * sig).
// Where the kernel that serves the shape has no fused form, the builtin that follows
// is launched on the result in place (same bits either way).
static int fmatmul_impl(int tl, int tr, uint64_t m, uint64_t n, uint64_t k, const float* left,
                        const float* right, float* out, void* workspace, uint64_t workspace_bytes,
                        void* stream, int fused, const float* sig) {
  clear_error();
  int rc = check_mm(tl, tr, m, n, k, left, right, out);
  if (rc) return rc;
  if (m == 0 || n == 0) return POLAR_B200_OK;
  if (k == 0) {
    rc = polar_b200_ffill(0.0f, out, m * n, stream);  // empty sum
    if (rc || fused == 0) return rc;
    return fused == 1 ? polar_b200_fsigmoid(out, out, m * n, stream)
                      : polar_b200_fsigmoid_grad(out, sig, out, m * n, stream);
  }
  const int path = choose_path(tl, tr, m, n, k, left, right, out);
  const int kind0 = path == kPathSkinny ? skinny_kind(tl, tr, m, n, k, left, right, out) : 0;
  const bool fused_in_kernel = (fused == 1 && (path == kPathTc || kind0 == 1)) || (fused == 2 && kind0 == 3);
  if (fused != 0 && !fused_in_kernel) {
    rc = fmatmul_impl(tl, tr, m, n, k, left, right, out, workspace, workspace_bytes, stream, 0, nullptr);
    if (rc) return rc;
    return fused == 1 ? polar_b200_fsigmoid(out, out, m * n, stream)
                      : polar_b200_fsigmoid_grad(out, sig, out, m * n, stream);
  }
  switch (path) {
    case kPathTc:
      return tc_path(tl, tr, m, n, k, left, right, out, workspace, workspace_bytes, stream, fused, 0);
    case kPathSkinny: {
      const int kind = skinny_kind(tl, tr, m, n, k, left, right, out);
      const uint64_t need = skinny_workspace_bytes(kind, m, n, k);
      if (need == 0)
        return launch_skinny(kind, tl, tr, m, n, k, left, right, out, nullptr, as_stream(stream),
                             fused == 2 ? sig : nullptr, fused == 1 ? 1 : 0);
      if (workspace) {
        if (workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 15))
          return fail(POLAR_B200_ERR_WORKSPACE, "workspace too small or not 16-byte aligned");
        return launch_skinny(kind, tl, tr, m, n, k, left, right, out, static_cast<float*>(workspace),
                             as_stream(stream), nullptr);
      }
      // No workspace from the caller: take it from the stream-ordered pool.
      void* ws = nullptr;
      cudaError_t e = cudaMallocAsync(&ws, need, as_stream(stream));
      if (e != cudaSuccess) return fail(POLAR_B200_ERR_CUDA, "cudaMallocAsync(workspace)", e);
      rc = launch_skinny(kind, tl, tr, m, n, k, left, right, out, static_cast<float*>(ws), as_stream(stream), nullptr);
      e = cudaFreeAsync(ws, as_stream(stream));
      if (rc == POLAR_B200_OK && e != cudaSuccess) return fail(POLAR_B200_ERR_CUDA, "cudaFreeAsync(workspace)", e);
      return rc;
    }
    default:
      return launch_ffma(tl, tr, m, n, k, left, right, out, as_stream(stream));
  }
}

extern "C" {
int polar_b200_fmatmul(int tl, int tr, uint64_t m, uint64_t n, uint64_t k, const float* left,
                       const float* right, float* out, void* workspace, uint64_t workspace_bytes,
                       void* stream) {
  LaunchDeviceScope on(stream, out);
  return fmatmul_impl(tl, tr, m, n, k, left, right, out, workspace, workspace_bytes, stream, 0, nullptr);
}

uint64_t polar_b200_fmatmul_t_f_rows_workspace_bytes(uint64_t rows, uint64_t n, uint64_t k) {
  // a block that is the whole result runs as the plain builtin, which may choose differently
  const uint64_t a = workspace_need(1, 0, rows, n, k, 0, true), b = workspace_need(1, 0, rows, n, k, 0, false);
  return a > b ? a : b;
}

int polar_b200_fmatmul_t_f_rows(uint64_t m, uint64_t row0, uint64_t rows, uint64_t n, uint64_t k, const float* left,
                                const float* right, float* out, void* workspace, uint64_t workspace_bytes,
                                void* stream) {
  clear_error();
  if (rows == 0) return POLAR_B200_OK;
  if (!left || !right || !out) return fail(POLAR_B200_ERR_INVALID, "null device pointer");
  if (row0 + rows > m || (row0 & 3) || m > (1ull << 31) || n > (1ull << 31) || k > (1ull << 31))
    return fail(POLAR_B200_ERR_INVALID, "fmatmul_t_f_rows: rows outside the result, or row0 not a multiple of 4");
  if (row0 == 0 && rows == m) return polar_b200_fmatmul(1, 0, m, n, k, left, right, out, workspace, workspace_bytes, stream);
  const float* l = left + row0;
  float* o = out + row0 * n;
  if ((m & 3) || !tc_shape_ok(1, 0, rows, n, k, l, right) || rows < 64 || n < 32 || k < 32 ||
      skinny_kind(1, 0, rows, n, k, l, right, o))
    return fail(POLAR_B200_ERR_UNSUPPORTED, "fmatmul_t_f_rows serves blocks of rows that run on the tensor-core path");
  LaunchDeviceScope on(stream, out);
  return tc_path(1, 0, rows, n, k, l, right, o, workspace, workspace_bytes, stream, 0, m);
}

int polar_b200_fmatmul_sigmoid(int tl, int tr, uint64_t m, uint64_t n, uint64_t k, const float* left,
                               const float* right, float* out, void* workspace, uint64_t workspace_bytes,
                               void* stream) {
  LaunchDeviceScope on(stream, out);
  return fmatmul_impl(tl, tr, m, n, k, left, right, out, workspace, workspace_bytes, stream, 1, nullptr);
}

int polar_b200_fmatmul_sigmoid_grad(int tl, int tr, uint64_t m, uint64_t n, uint64_t k, const float* left,
                                    const float* right, const float* sigmoidOut, float* out, void* workspace,
                                    uint64_t workspace_bytes, void* stream) {
  if (m * n != 0 && !sigmoidOut) {
    clear_error();
    return fail(POLAR_B200_ERR_INVALID, "null sigmoid-output pointer");
  }
  LaunchDeviceScope on(stream, out);
  return fmatmul_impl(tl, tr, m, n, k, left, right, out, workspace, workspace_bytes, stream, 2, sigmoidOut);
}
}

uint64_t polar_b200_fdense_grad_workspace_bytes(uint64_t rows, uint64_t kh, uint64_t n) {
  const float* al = reinterpret_cast<const float*>(256);
  if (dense_grad_ok(rows, kh, n, al, al)) return dense_grad_workspace_bytes(rows, kh, n);
  // the two builtins in sequence
  const uint64_t a = workspace_need(1, 0, kh, n, rows, 0), b = workspace_need(0, 1, rows, kh, n, 2);
  return a > b ? a : b;
}

int polar_b200_fdense_grad(uint64_t rows, uint64_t kh, uint64_t n, const float* dz, const float* w,
                           const float* h, float* dw, float* din, void* workspace, uint64_t workspace_bytes,
                           void* stream) {
  clear_error();
  if (rows == 0 || kh == 0 || n == 0) return fail(POLAR_B200_ERR_UNSUPPORTED, "fdense_grad: empty operand");
  if (!dz || !w || !h || !dw || !din) return fail(POLAR_B200_ERR_INVALID, "null device pointer");
  if (rows > (1ull << 31) || kh > (1ull << 31)) return fail(POLAR_B200_ERR_INVALID, "matrix dimension too large");
  LaunchDeviceScope on(stream, din);
  if (!dense_grad_ok(rows, kh, n, h, din)) {
    // shapes the one-pass kernel does not serve: the two builtins it stands for, one after the other
    int rc = polar_b200_fmatmul(1, 0, kh, n, rows, h, dz, dw, workspace, workspace_bytes, stream);
    if (rc) return rc;
    return polar_b200_fmatmul_sigmoid_grad(0, 1, rows, kh, n, dz, w, h, din, workspace, workspace_bytes, stream);
  }
  const uint64_t need = dense_grad_workspace_bytes(rows, kh, n);
  cudaStream_t st = as_stream(stream);
  if (need == 0) return launch_dense_grad(h, dz, w, din, dw, nullptr, rows, kh, n, st);
  if (workspace) {
    if (workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 15))
      return fail(POLAR_B200_ERR_WORKSPACE, "workspace too small or not 16-byte aligned");
    return launch_dense_grad(h, dz, w, din, dw, static_cast<float*>(workspace), rows, kh, n, st);
  }
  void* ws = nullptr;
  cudaError_t e = cudaMallocAsync(&ws, need, st);
  if (e != cudaSuccess) return fail(POLAR_B200_ERR_CUDA, "cudaMallocAsync(workspace)", e);
  int rc = launch_dense_grad(h, dz, w, din, dw, static_cast<float*>(ws), rows, kh, n, st);
  e = cudaFreeAsync(ws, st);
  if (rc == POLAR_B200_OK && e != cudaSuccess) return fail(POLAR_B200_ERR_CUDA, "cudaFreeAsync(workspace)", e);
  return rc;
}

int polar_b200_fmatmul_ffma(int tl, int tr, uint64_t m, uint64_t n, uint64_t k, const float* left,
                            const float* right, float* out, void* stream) {
  clear_error();
  int rc = check_mm(tl, tr, m, n, k, left, right, out);
  if (rc) return rc;
  if (m == 0 || n == 0) return POLAR_B200_OK;
  if (k == 0) return polar_b200_ffill(0.0f, out, m * n, stream);
  LaunchDeviceScope on(stream, out);
  return launch_ffma(tl, tr, m, n, k, left, right, out, as_stream(stream));
}

int polar_b200_fmatmul_tc(int tl, int tr, uint64_t m, uint64_t n, uint64_t k, const float* left,
                          const float* right, float* out, int tile_n, int slab_k, int passes,
                          int write_hi, int splits, void* stream) {
  clear_error();
  int rc = check_mm(tl, tr, m, n, k, left, right, out);
  if (rc) return rc;
  if (m == 0 || n == 0 || k == 0) return fail(POLAR_B200_ERR_UNSUPPORTED, "empty matrix");
  // tile_n + 1000: the operands exchange roles (the transposed product is computed and stored
  // transposed; whole tiles or fixed k cuts only)
  const int swap_ab = tile_n >= 1000 ? 1 : 0;
  if (swap_ab) tile_n -= 1000;
  // tile_n = 512 selects the 256 x 256 tile configuration (256 columns, two row sub-tiles)
  const int mt = tile_n == 512 ? 2 : 1;
  if (mt == 2) tile_n = 256;
  if (tile_n != 128 && tile_n != 256) return fail(POLAR_B200_ERR_INVALID, "tile_n must be 128, 256 or 512");
  if (mt == 2 && slab_k != 16) return fail(POLAR_B200_ERR_INVALID, "256 x 256 tiles need slab_k = 16");
  if (slab_k != 16 && slab_k != 32) return fail(POLAR_B200_ERR_INVALID, "slab_k must be 16 or 32");
  if (passes != 1 && passes != 3 && passes != 13)
    return fail(POLAR_B200_ERR_INVALID, "passes must be 1 or 3 (13: issue-rate diagnostic)");
  if (!tc_shape_ok(tl, tr, m, n, k, left, right))
    return fail(POLAR_B200_ERR_UNSUPPORTED, "operands are not expressible as TMA tensor maps");
  if (swap_ab && (splits == -1 || !tc_shape_ok(tr ? 0 : 1, tl ? 0 : 1, n, m, k, right, left)))
    return fail(POLAR_B200_ERR_UNSUPPORTED, "exchanged operands: not with stream mode, and both roles must suit TMA");
  if (splits < -1 || splits > 64 || (splits > 1 && ((m * n) & 3)))
    return fail(POLAR_B200_ERR_INVALID,
                "splits must be -1 (stream), 0 (automatic) or 1..64, and m*n a multiple of 4 when > 1");
  if (splits == -1 && tile_n != 256) return fail(POLAR_B200_ERR_INVALID, "stream mode needs tile_n = 256");
  LaunchDeviceScope on(stream, out);
  uint32_t s = splits == -1 ? 0u : splits == 0 ? (swap_ab ? tc_default_splits(n, m, k, mt) : tc_default_splits(m, n, k, mt))
                                               : (uint32_t)splits;
  if (swap_ab && s == 0) s = 1;
  return run_tc(tl, tr, m, n, k, left, right, out, tile_n, slab_k, passes, write_hi, s, nullptr, 0, as_stream(stream),
                0, 0, mt, swap_ab);
}

static uint64_t numel(const polar_b200_tensor& t) {
  uint64_t n = 1;
  for (uint64_t d = 0; d < t.dims; ++d) n *= t.shape[d];
  return n;
}

int polar_b200_launch_by_name(const char* name, const polar_b200_arg* a, uint64_t argc,
                              void* workspace, uint64_t workspace_bytes, void* stream) {
  clear_error();
  if (!name || (!a && argc)) return fail(POLAR_B200_ERR_INVALID, "null kernel name or argument list");
  auto pattern = [&](const char* pat) {  // 'T' tensor, 'f' scalar
    if (std::strlen(pat) != argc) return false;
    for (uint64_t i = 0; i < argc; ++i) {
      if ((pat[i] == 'T') != (a[i].is_tensor != 0)) return false;
      if (a[i].is_tensor && a[i].tensor.dims && !a[i].tensor.shape) return false;
    }
    return true;
  };
  auto same = [&](uint64_t i, uint64_t j) { return numel(a[i].tensor) == numel(a[j].tensor); };
  const int bad_args = POLAR_B200_ERR_UNSUPPORTED;
  if (!std::strcmp(name, "ffill")) {
    if (!pattern("fT")) return fail(bad_args, "ffill expects (f32 pattern, T out)");
    return polar_b200_ffill(a[0].scalar, a[1].tensor.data, numel(a[1].tensor), stream);
  }
  if (!std::strcmp(name, "fcopy")) {
    if (!pattern("TT") || !same(0, 1)) return fail(bad_args, "fcopy expects (T in, T out) of equal size");
    return polar_b200_fcopy(a[0].tensor.data, a[1].tensor.data, numel(a[1].tensor), stream);
  }
  if (!std::strcmp(name, "fadd")) {
    if (!pattern("TfTfT") || !same(0, 4) || !same(2, 4))
      return fail(bad_args, "fadd expects (T a, f32 scaleA, T b, f32 scaleB, T out) of equal size");
    return polar_b200_fadd(a[0].tensor.data, a[1].scalar, a[2].tensor.data, a[3].scalar,
                           a[4].tensor.data, numel(a[4].tensor), stream);
  }
  if (!std::strcmp(name, "fmul") || !std::strcmp(name, "fdivide") || !std::strcmp(name, "flogloss")) {
    if (!pattern("TTT") || !same(0, 2) || !same(1, 2))
      return fail(bad_args, "binary builtin expects (T, T, T out) of equal size");
    uint64_t n = numel(a[2].tensor);
    if (name[1] == 'm') return polar_b200_fmul(a[0].tensor.data, a[1].tensor.data, a[2].tensor.data, n, stream);
    if (name[1] == 'd') return polar_b200_fdivide(a[0].tensor.data, a[1].tensor.data, a[2].tensor.data, n, stream);
    return polar_b200_flogloss(a[0].tensor.data, a[1].tensor.data, a[2].tensor.data, n, stream);
  }
  if (!std::strcmp(name, "fsigmoid")) {
    if (!pattern("TT") || !same(0, 1)) return fail(bad_args, "fsigmoid expects (T in, T out) of equal size");
    return polar_b200_fsigmoid(a[0].tensor.data, a[1].tensor.data, numel(a[1].tensor), stream);
  }
  if (!std::strcmp(name, "frelu")) {
    if (!pattern("TT") || !same(0, 1)) return fail(bad_args, "frelu expects (T in, T out) of equal size");
    return polar_b200_frelu(a[0].tensor.data, a[1].tensor.data, numel(a[1].tensor), stream);
  }
  if (!std::strcmp(name, "fsoftmax")) {
    if (!pattern("TT") || !same(0, 1)) return fail(bad_args, "fsoftmax expects (T in, T out) of equal size");
    return polar_b200_fsoftmax(a[0].tensor.data, a[1].tensor.data, numel(a[1].tensor), nullptr, 0, stream);
  }
  if (!std::strcmp(name, "fpool")) {
    if (!pattern("TffffT") || a[0].tensor.dims != 2 || a[5].tensor.dims != 2)
      return fail(bad_args, "fpool expects (T in[h,w], i64 windowH, i64 windowW, i64 strideH, i64 strideW, T out)");
    const uint64_t h = a[0].tensor.shape[0], w = a[0].tensor.shape[1];
    const int64_t wh = a[1].integer, ww = a[2].integer, sh = a[3].integer, sw = a[4].integer;
    if (wh <= 0 || ww <= 0 || sh <= 0 || sw <= 0 || (uint64_t)wh > h || (uint64_t)ww > w ||
        a[5].tensor.shape[0] != (h - wh) / sh + 1 || a[5].tensor.shape[1] != (w - ww) / sw + 1)
      return fail(bad_args, "fpool: window, stride and output shape do not agree");
    return polar_b200_fpool(a[0].tensor.data, h, w, wh, ww, sh, sw, a[5].tensor.data, stream);
  }
  if (!std::strcmp(name, "fconv2d")) {
    if (!pattern("TTT") || a[0].tensor.dims != 2 || a[1].tensor.dims != 2 || a[2].tensor.dims != 2)
      return fail(bad_args, "fconv2d expects (T in[h,w], T kernel[kh,kw], T out)");
    const uint64_t h = a[0].tensor.shape[0], w = a[0].tensor.shape[1];
    const uint64_t kh = a[1].tensor.shape[0], kw = a[1].tensor.shape[1];
    if (kh > h || kw > w || a[2].tensor.shape[0] != h - kh + 1 || a[2].tensor.shape[1] != w - kw + 1)
      return fail(bad_args, "fconv2d: shapes do not agree");
    return polar_b200_fconv2d(a[0].tensor.data, h, w, a[1].tensor.data, kh, kw, a[2].tensor.data, stream);
  }
  if (!std::strcmp(name, "fmatmul_t_f_rows")) {
    // (T left[k,m], T right[k,n], f32 row0, f32 rows, T out[m,n]): rows [row0, row0+rows) of fmatmul_t_f
    if (!pattern("TTffT") || a[0].tensor.dims != 2 || a[1].tensor.dims != 2 || a[4].tensor.dims != 2)
      return fail(bad_args, "fmatmul_t_f_rows expects (T left, T right, f32 row0, f32 rows, T out)");
    const uint64_t k = a[0].tensor.shape[0], m = a[0].tensor.shape[1], n = a[1].tensor.shape[1];
    const float r0 = a[2].scalar, rr = a[3].scalar;
    if (a[1].tensor.shape[0] != k || a[4].tensor.shape[0] != m || a[4].tensor.shape[1] != n || r0 < 0 || rr < 0 ||
        r0 != (float)(uint64_t)r0 || rr != (float)(uint64_t)rr)
      return fail(bad_args, "fmatmul_t_f_rows: shapes do not agree, or a row count that is not a whole number");
    return polar_b200_fmatmul_t_f_rows(m, (uint64_t)r0, (uint64_t)rr, n, k, a[0].tensor.data, a[1].tensor.data,
                                       a[4].tensor.data, workspace, workspace_bytes, stream);
  }
  if (!std::strcmp(name, "fdense_grad")) {
    // (T dZ [rows,n], T W [kh,n], T H [rows,kh], T dW [kh,n], T dIn [rows,kh]): TWO results
    if (!pattern("TTTTT") || a[0].tensor.dims != 2 || a[1].tensor.dims != 2 || a[2].tensor.dims != 2)
      return fail(bad_args, "fdense_grad expects (T dZ[rows,n], T W[kh,n], T H[rows,kh], T dW[kh,n], T dIn[rows,kh])");
    const uint64_t rows = a[0].tensor.shape[0], n = a[0].tensor.shape[1], kh = a[1].tensor.shape[0];
    if (a[1].tensor.shape[1] != n || a[2].tensor.shape[0] != rows || a[2].tensor.shape[1] != kh ||
        numel(a[3].tensor) != kh * n || numel(a[4].tensor) != rows * kh)
      return fail(bad_args, "fdense_grad: shapes do not agree");
    return polar_b200_fdense_grad(rows, kh, n, a[0].tensor.data, a[1].tensor.data, a[2].tensor.data, a[3].tensor.data,
                                  a[4].tensor.data, workspace, workspace_bytes, stream);
  }
  if (!std::strcmp(name, "fsum")) {
    if (!pattern("TT") || numel(a[1].tensor) < 1) return fail(bad_args, "fsum expects (T in, T out[1])");
    return polar_b200_fsum_f32(a[0].tensor.data, a[1].tensor.data, numel(a[0].tensor), workspace, workspace_bytes,
                               stream);
  }
  if (!std::strcmp(name, "ftranspose")) {
    if (!pattern("TT") || a[0].tensor.dims != 2 || a[1].tensor.dims != 2 ||
        a[1].tensor.shape[0] != a[0].tensor.shape[1] || a[1].tensor.shape[1] != a[0].tensor.shape[0])
      return fail(bad_args, "ftranspose expects (T in[r,c], T out[c,r])");
    return polar_b200_ftranspose(a[0].tensor.data, a[0].tensor.shape[0], a[0].tensor.shape[1], a[1].tensor.data, stream);
  }
  if (!std::strcmp(name, "fslice")) {
    if (!pattern("TfT") || a[0].tensor.dims < 1 || a[0].tensor.shape[0] == 0 || a[1].integer < 0 ||
        numel(a[2].tensor) * a[0].tensor.shape[0] != numel(a[0].tensor))
      return fail(bad_args, "fslice expects (T in[d0,...], i64 index, T out[...]) with out one sub-tensor of in");
    return polar_b200_fslice(a[0].tensor.data, a[0].tensor.shape[0], numel(a[2].tensor), (uint64_t)a[1].integer,
                             a[2].tensor.data, stream);
  }
  if (!std::strcmp(name, "fsigmoid_grad")) {
    if (!pattern("TTT") || !same(0, 2) || !same(1, 2))
      return fail(bad_args, "fsigmoid_grad expects (T gradient, T sigmoidOut, T out) of equal size");
    return polar_b200_fsigmoid_grad(a[0].tensor.data, a[1].tensor.data, a[2].tensor.data, numel(a[2].tensor),
                                    stream);
  }
  if (!std::strcmp(name, "fsigmoid_logloss_grad")) {
    if (!pattern("TTT") || !same(0, 2) || !same(1, 2))
      return fail(bad_args, "fsigmoid_logloss_grad expects (T predicted, T groundTruth, T out) of equal size");
    return polar_b200_fsigmoid_logloss_grad(a[0].tensor.data, a[1].tensor.data, a[2].tensor.data,
                                            numel(a[2].tensor), stream);
  }
  if (!std::strcmp(name, "fmulconcat")) {
    if (!pattern("TTT") || !same(1, 2) || numel(a[0].tensor) < 1)
      return fail(bad_args, "fmulconcat expects (T gradient, T localDerivative, T out)");
    return polar_b200_fmulconcat(a[0].tensor.data, a[1].tensor.data, a[2].tensor.data,
                                 numel(a[2].tensor), stream);
  }
  if (!std::strncmp(name, "fmatmul_", 8) && std::strlen(name) >= 11 && name[9] == '_' &&
      (name[8] == 'f' || name[8] == 't') && (name[10] == 'f' || name[10] == 't')) {
    // "fmatmul_x_y", or the extended forms "fmatmul_x_y_sigmoid" (T left, T right, T out)
    // and "fmatmul_x_y_sigmoid_grad" (T left, T right, T sigmoidOut, T out)
    const char* suffix = name + 11;
    const int fused = !*suffix ? 0 : !std::strcmp(suffix, "_sigmoid") ? 1 : !std::strcmp(suffix, "_sigmoid_grad") ? 2 : -1;
    if (fused < 0) return fail(POLAR_B200_ERR_UNSUPPORTED, "unknown native kernel name");
    if (!pattern(fused == 2 ? "TTTT" : "TTT")) return fail(bad_args, "fmatmul expects (T left, T right, [T sigmoidOut,] T out)");
    const polar_b200_tensor &l = a[0].tensor, &r = a[1].tensor, &o = a[fused == 2 ? 3 : 2].tensor;
    if (l.dims != 2 || r.dims != 2 || o.dims != 2) return fail(bad_args, "fmatmul operands must be 2-D");
    int tl = name[8] == 't', tr = name[10] == 't';
    // m = tl ? left.shape[1] : left.shape[0]; n = tr ? right.shape[0] : right.shape[1]
    // (src/operation/internal/MatMulOperationInternal.cpp:39-40 of the reference)
    uint64_t m = tl ? l.shape[1] : l.shape[0], k = tl ? l.shape[0] : l.shape[1];
    uint64_t n = tr ? r.shape[0] : r.shape[1], k2 = tr ? r.shape[1] : r.shape[0];
    if (k != k2 || o.shape[0] != m || o.shape[1] != n) return fail(bad_args, "fmatmul shapes do not agree");
    if (fused == 2 && numel(a[2].tensor) != m * n) return fail(bad_args, "sigmoidOut must have the shape of out");
    if (fused == 1)
      return polar_b200_fmatmul_sigmoid(tl, tr, m, n, k, l.data, r.data, o.data, workspace, workspace_bytes, stream);
    if (fused == 2)
      return polar_b200_fmatmul_sigmoid_grad(tl, tr, m, n, k, l.data, r.data, a[2].tensor.data, o.data, workspace,
                                             workspace_bytes, stream);
    return polar_b200_fmatmul(tl, tr, m, n, k, l.data, r.data, o.data, workspace, workspace_bytes, stream);
  }
  return fail(POLAR_B200_ERR_UNSUPPORTED, "unknown native kernel name");
}

}  // extern "C"
