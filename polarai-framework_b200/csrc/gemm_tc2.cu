// fmatmul on the tensor cores with PAIRS of CTAs (tcgen05 cta_group::2): two CTAs of
// a cluster, one per SM of a TPC, compute one 256 x 256 output tile together.
//
// Why: with one CTA per tile the kernel in gemm_tc.cu is held back by shared-memory
// bandwidth - per 16-wide k slab the three TF32 products fetch 72 KB of operands and
// the split pass moves another 48 KB.  In a pair each CTA stages only ITS 128 rows of
// A and ITS 128 columns of B (16 KB per slab instead of 24 KB), the paired MMA reads
// the other half from the partner's shared memory, and every byte staged feeds twice
// the arithmetic.
//
// Per CTA (both CTAs run the same roles; only the even-ranked "leader" issues MMAs):
//   warp 0      TMA producer for this CTA's halves; completion is signalled on a
//               barrier of this CTA
//   warp 1      tensor-memory allocation (both CTAs, cta_group::2); in the leader: the
//               MMA issuer - tcgen05.mma.cta_group::2 with M = 256, three products per
//               k step, tcgen05.commit multicast to both CTAs' barriers
//   warps 2-9   split warps: wait for this CTA's slab, write the lo part, then one
//               lane per warp arrives on the LEADER's "slab ready" barrier (16 arrivals:
//               8 warps x 2 CTAs), remotely from the partner
//   warps 10-17 epilogue: each CTA drains its own 128 rows of the accumulator from
//               its tensor memory and hands the accumulator back to the leader
// The accumulator is double-buffered (2 x 256 columns), the work list is the same
// (tile, k-split) list as in the one-CTA kernel, walked by cluster index.
// No TMA load here uses cluster-wide delivery: every load lands in the issuing CTA.
//
// All waits are bounded as in gemm_tc.cu; before it exits, every CTA meets its partner
// at a cluster barrier so that no remote arrive can target a CTA that has gone.
#include <cuda.h>
#include <cstdio>
#include <cstdlib>

#include "common.cuh"
#include "tc_ptx.cuh"

namespace polar_b200 {
namespace tc {

int make_map(CUtensorMap* map, const float* base, uint64_t inner, uint64_t outer, uint32_t box_inner,
             uint32_t box_outer, bool mn_major, int bk, uint64_t pitch = 0);
int ensure_status();
extern int* g_status_dev;
int launch_add_splits(const float* ws, float* out, uint64_t m, uint64_t n, uint32_t splits, int epilogue,
                      cudaStream_t stream);

namespace pair {

constexpr int BMH = 128;            // rows of A per CTA (tile M = 256)
constexpr int BNH = 128;            // columns of B per CTA (tile N = 256)
constexpr int BN = 256;
constexpr int BK = 16;
constexpr int kSplitWarps = 8;
constexpr int kEpilogueWarps = 8;
constexpr int kThreads = 32 * (2 + kSplitWarps + kEpilogueWarps);
constexpr int kGroupM = 8;          // raster: 8 row tiles of 256 share their column tiles
constexpr uint32_t kABytes = BMH * BK * 4;              // 8 KB
constexpr uint32_t kBBytes = BNH * BK * 4;              // 8 KB
constexpr uint32_t kRawBytes = kABytes + kBBytes;       // 16 KB
constexpr uint32_t kStageBytes = 2 * kRawBytes;         // raw + lo
constexpr int kStages = 6;
constexpr uint32_t kTileBytes = kStages * kStageBytes;  // 192 KB
constexpr uint32_t kSmemBytes = kTileBytes + 1024 + 512;
constexpr uint32_t kTmemCols = 2 * BN;
constexpr uint32_t kBoxBytes = 32 * BK * 4;

// ---- cluster-scope PTX ----------------------------------------------------

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Address of the same shared-memory offset in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_mma2_tf32(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives, once the MMAs issued so far have completed, on the barrier at this offset
// in both CTAs of the pair.
__device__ __forceinline__ void tc_commit2_both(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"((uint16_t)3)
      : "memory");
}

struct Params {
  uint64_t m, n, k;
  float* out;
  int a_mn_major, b_mn_major;
  int* status;
  uint32_t tiles_m, tiles_n;   // tiles of 256 x 256
  int epilogue;
  uint32_t splits;
  float* partial;
  int diag;   // 1: skip the split pass and issue hi*hi three times (issue-rate diagnostic)
};

__device__ __forceinline__ void tile_coords(uint32_t t, uint32_t tiles_m, uint32_t tiles_n, int* m0, int* n0) {
  const uint32_t per_group = kGroupM * tiles_n;
  const uint32_t g = t / per_group;
  const uint32_t first_m = g * kGroupM;
  const uint32_t rows = (tiles_m - first_m < (uint32_t)kGroupM) ? tiles_m - first_m : (uint32_t)kGroupM;
  const uint32_t r = t - g * per_group;
  *m0 = (int)((first_m + r % rows) * 256);
  *n0 = (int)((r / rows) * 256);
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
fmatmul_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                       const Params p) {
  constexpr int S = kStages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + kTileBytes;
  auto raw_here = [&](int s) { return bar_base + 8u * s; };               // this CTA's slab landed (TMA)
  auto ready = [&](int s) { return bar_base + 8u * (S + s); };            // leader: slab split in both CTAs
  auto empty = [&](int s) { return bar_base + 8u * (2 * S + s); };        // stage free (MMA commit, both CTAs)
  auto acc_full = [&](int a) { return bar_base + 8u * (3 * S + a); };     // accumulator done (both CTAs)
  auto acc_empty = [&](int a) { return bar_base + 8u * (3 * S + 2 + a); };  // leader: accumulator drained
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + kTileBytes + 8 * (3 * S + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0 = leader
  const bool leader = rank == 0;
  const uint32_t cluster_id = blockIdx.x >> 1;
  const uint32_t num_clusters = gridDim.x >> 1;
  const uint32_t num_kb = (uint32_t)((p.k + BK - 1) / BK);
  const uint32_t num_units = p.tiles_m * p.tiles_n * p.splits;
  auto slab_begin = [&](uint32_t u) { return (uint32_t)(((uint64_t)(u % p.splits) * num_kb) / p.splits); };
  auto slab_end = [&](uint32_t u) { return (uint32_t)(((uint64_t)(u % p.splits + 1) * num_kb) / p.splits); };

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(raw_here(s), 1);
      mbar_init(ready(s), 2 * kSplitWarps);      // one arrival per split warp of both CTAs
      mbar_init(empty(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full(a), 1);
      mbar_init(acc_empty(a), 2 * kEpilogueWarps);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc2(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // partner's barriers exist before anything is signalled
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer (this CTA's halves) ----------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (uint32_t u = cluster_id; u < num_units && ok; u += num_clusters) {
        int m0, n0;
        tile_coords(u / p.splits, p.tiles_m, p.tiles_n, &m0, &n0);
        m0 += (int)rank * BMH;
        n0 += (int)rank * BNH;
        for (uint32_t kb = slab_begin(u), kb_end = slab_end(u); kb < kb_end; ++kb, ++it) {
          const int s = it % S;
          const uint32_t ph = (it / S) & 1u;
          if (!mbar_wait(empty(s), ph ^ 1u, abort_flag, p.status, 201)) { ok = false; break; }
          const uint32_t stage = smem_base + s * kStageBytes;
          mbar_expect_tx(raw_here(s), kRawBytes);
          const int k0 = (int)(kb * BK);
          if (!p.a_mn_major) {
            tma_load_2d(stage, &map_a, raw_here(s), k0, m0);                    // box {16 k, 128 m}
          } else {
            for (int c = 0; c < BMH / 32; ++c)                                   // boxes {32 m, 16 k}
              tma_load_2d(stage + c * kBoxBytes, &map_a, raw_here(s), m0 + 32 * c, k0);
          }
          const uint32_t bdst = stage + kABytes;
          if (!p.b_mn_major) {
            tma_load_2d(bdst, &map_b, raw_here(s), k0, n0);                     // box {16 k, 128 n}
          } else {
            for (int c = 0; c < BNH / 32; ++c)                                   // boxes {32 n, 16 k}
              tma_load_2d(bdst + c * kBoxBytes, &map_b, raw_here(s), n0 + 32 * c, k0);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (leader && lane == 0) {
      const uint32_t idesc = make_idesc(256, BN, p.a_mn_major, p.b_mn_major);
      constexpr uint32_t kRowGroup = 8u * BK * 4u;   // 512 B: K-major, 64-byte rows, SWIZZLE_64B (layout 4)
      const uint32_t a_lbo = p.a_mn_major ? kBoxBytes : 16u, a_step = p.a_mn_major ? 1024u : 32u;
      const uint32_t b_lbo = p.b_mn_major ? kBoxBytes : 16u, b_step = p.b_mn_major ? 1024u : 32u;
      const uint32_t a_sbo = p.a_mn_major ? 512u : kRowGroup, a_lt = p.a_mn_major ? 1u : 4u;
      const uint32_t b_sbo = p.b_mn_major ? 512u : kRowGroup, b_lt = p.b_mn_major ? 1u : 4u;
      uint32_t it = 0, unit_iter = 0;
      bool ok = true;
      for (uint32_t u = cluster_id; u < num_units && ok; u += num_clusters, ++unit_iter) {
        const uint32_t as = unit_iter & 1u;
        ok = mbar_wait(acc_empty(as), ((unit_iter >> 1) & 1u) ^ 1u, abort_flag, p.status, 206);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_acc = tmem_base + as * BN;
        const uint32_t kb_first = slab_begin(u);
        for (uint32_t kb = kb_first, kb_end = slab_end(u); kb < kb_end; ++kb, ++it) {
          const int s = it % S;
          const uint32_t ph = (it / S) & 1u;
          ok = mbar_wait(ready(s), ph, abort_flag, p.status, 203);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_hi = smem_base + s * kStageBytes;
          const uint32_t b_hi = a_hi + kABytes;
          const uint32_t a_lo = a_hi + kRawBytes;
          const uint32_t b_lo = b_hi + kRawBytes;
#pragma unroll
          for (int kk = 0; kk < BK / 8; ++kk) {
            const uint64_t da_hi = make_desc(a_hi + kk * a_step, a_lbo, a_sbo, a_lt);
            const uint64_t db_hi = make_desc(b_hi + kk * b_step, b_lbo, b_sbo, b_lt);
            const uint64_t da_lo = make_desc(a_lo + kk * a_step, a_lbo, a_sbo, a_lt);
            const uint64_t db_lo = make_desc(b_lo + kk * b_step, b_lbo, b_sbo, b_lt);
            tc_mma2_tf32(tmem_acc, da_hi, db_hi, idesc, ((kb - kb_first) | (uint32_t)kk) ? 1u : 0u);
            tc_mma2_tf32(tmem_acc, p.diag ? da_hi : da_lo, db_hi, idesc, 1u);
            tc_mma2_tf32(tmem_acc, da_hi, p.diag ? db_hi : db_lo, idesc, 1u);
          }
          tc_commit2_both(empty(s));      // frees the stage in both CTAs
        }
        if (ok) tc_commit2_both(acc_full(as));
      }
    }
  } else if (warp < 2 + kSplitWarps) {
    // ---------------- split warps ----------------
    const int tid = threadIdx.x - 64;
    const uint32_t ready_leader = map_to_cta(ready(0), 0);   // leader's copy of the barrier block
    uint32_t it = 0;
    bool ok = true;
    for (uint32_t u = cluster_id; u < num_units && ok; u += num_clusters) {
      for (uint32_t kb = slab_begin(u), kb_end = slab_end(u); kb < kb_end; ++kb, ++it) {
        const int s = it % S;
        const uint32_t ph = (it / S) & 1u;
        if (!mbar_wait(raw_here(s), ph, abort_flag, p.status, 204)) { ok = false; break; }
        float4* raw = reinterpret_cast<float4*>(smem_gen + s * kStageBytes);
        float4* lo = reinterpret_cast<float4*>(smem_gen + s * kStageBytes + kRawBytes);
        constexpr int kVecs = kRawBytes / 16;
        static_assert(kVecs % (kSplitWarps * 32) == 0, "slab must divide over the split warps");
#pragma unroll
        for (int i = 0; i < (p.diag ? 0 : kVecs / (kSplitWarps * 32)); ++i) {
          const int e = tid + i * kSplitWarps * 32;
          float4 v = raw[e];
          float4 h;
          h.x = __uint_as_float(__float_as_uint(v.x) & 0xFFFFE000u);
          h.y = __uint_as_float(__float_as_uint(v.y) & 0xFFFFE000u);
          h.z = __uint_as_float(__float_as_uint(v.z) & 0xFFFFE000u);
          h.w = __uint_as_float(__float_as_uint(v.w) & 0xFFFFE000u);
          lo[e] = make_float4(v.x - h.x, v.y - h.y, v.z - h.z, v.w - h.w);
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(ready_leader + 8u * s);
      }
    }
  } else {
    // ---------------- epilogue warps: this CTA's 128 rows ----------------
    const int q = warp & 3;
    const int half = (warp - (2 + kSplitWarps)) >> 2;
    const bool vec_ok = ((p.n & 3) == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0) &&
                        ((reinterpret_cast<uintptr_t>(p.partial) & 15) == 0);
    const uint32_t acc_empty_leader = map_to_cta(acc_empty(0), 0);
    uint32_t unit_iter = 0;
    for (uint32_t u = cluster_id; u < num_units; u += num_clusters, ++unit_iter) {
      int m0, n0;
      tile_coords(u / p.splits, p.tiles_m, p.tiles_n, &m0, &n0);
      m0 += (int)rank * BMH;
      float* const out_base = p.splits > 1 ? p.partial + (uint64_t)(u % p.splits) * p.m * p.n : p.out;
      const uint32_t as = unit_iter & 1u;
      if (!mbar_wait(acc_full(as), (unit_iter >> 1) & 1u, abort_flag, p.status, 205)) break;
      tc_fence_after();
      const uint64_t row = (uint64_t)m0 + q * 32 + lane;
      const uint32_t tmem_acc = tmem_base + as * BN + ((uint32_t)(q * 32) << 16);
      for (int c = half * (BN / 2); c < (half + 1) * (BN / 2); c += 32) {
        if ((uint64_t)n0 + c >= p.n) break;
        uint32_t r[32];
        tmem_ld_32x32(tmem_acc + (uint32_t)c, r);
        tmem_ld_wait();
        if (p.epilogue == 1) {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(sigmoid_clamped(__uint_as_float(r[j])));
        }
        if (row < p.m) {
          float* dst = out_base + row * p.n + n0 + c;
          if (vec_ok && (uint64_t)n0 + c + 32 <= p.n) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              *reinterpret_cast<float4*>(dst + j) = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                                                __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if ((uint64_t)n0 + c + j < p.n) dst[j] = __uint_as_float(r[j]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc_empty_leader + 8u * as);
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000ll) { }
  }
  cluster_sync_all();          // no remote arrive may target a CTA that has left
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, kTmemCols);
  }
}

}  // namespace pair

int launch_pair(int tl, int tr, uint64_t m, uint64_t n, uint64_t k, const float* left, const float* right,
                float* out, float* ws, uint32_t splits, int epilogue, cudaStream_t stream) {
  using namespace pair;
  int dev = 0;
  cudaGetDevice(&dev);
  static bool attr_done[64] = {false};
  if (dev >= 0 && dev < 64 && !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(fmatmul_tc_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)kSmemBytes);
    if (e != cudaSuccess) return fail(POLAR_B200_ERR_CUDA, "cudaFuncSetAttribute(smem, pair)", e);
    attr_done[dev] = true;
  }
  int rc = ensure_status();
  if (rc) return rc;
  CUtensorMap map_a, map_b;
  rc = tl ? make_map(&map_a, left, m, k, 32, BK, true, BK) : make_map(&map_a, left, k, m, BK, BMH, false, BK);
  if (rc) return rc;
  rc = tr ? make_map(&map_b, right, k, n, BK, BNH, false, BK) : make_map(&map_b, right, n, k, 32, BK, true, BK);
  if (rc) return rc;
  Params p;
  p.m = m; p.n = n; p.k = k; p.out = out;
  p.a_mn_major = tl ? 1 : 0;
  p.b_mn_major = tr ? 0 : 1;
  p.status = g_status_dev;
  const uint64_t tm = (m + 255) / 256, tn = (n + 255) / 256;
  const uint64_t num_kb = (k + BK - 1) / BK;
  if (splits < 1 || !ws || splits > num_kb) splits = 1;
  p.tiles_m = (uint32_t)tm; p.tiles_n = (uint32_t)tn;
  p.splits = splits;
  p.partial = splits > 1 ? ws : nullptr;
  p.epilogue = splits > 1 ? 0 : (epilogue & 1);
  p.diag = (epilogue & 2) ? 1 : 0;
  const uint64_t units = tm * tn * splits;
  if (units > 0x3fffffffull) return fail(POLAR_B200_ERR_UNSUPPORTED, "too many tiles");
  // How many pairs can be resident at once: not every TPC of a part has both SMs
  // available, and a persistent grid larger than that would run its tail serially.
  static int max_pairs[64] = {0};
  if (dev >= 0 && dev < 64 && max_pairs[dev] == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2u * (unsigned)(sm_count() / 2));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kSmemBytes;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n_clusters = 0;
    cudaError_t e = cudaOccupancyMaxActiveClusters(&n_clusters, fmatmul_tc_pair_kernel, &cfg);
    if (e != cudaSuccess || n_clusters <= 0) {
      cudaGetLastError();
      n_clusters = sm_count() / 2;
    }
    max_pairs[dev] = n_clusters;
    if (std::getenv("POLAR_B200_VERBOSE"))
      std::fprintf(stderr, "[polar_b200] device %d: %d CTA pairs resident at once (%d SMs)\n", dev, n_clusters,
                   sm_count());
  }
  const uint64_t pairs_max = (uint64_t)(dev >= 0 && dev < 64 ? max_pairs[dev] : sm_count() / 2);
  const unsigned grid = 2u * (unsigned)(units < pairs_max ? units : pairs_max);
  fmatmul_tc_pair_kernel<<<grid, kThreads, kSmemBytes, stream>>>(map_a, map_b, p);
  rc = check_launch("fmatmul_tc_pair");
  if (rc || splits == 1) return rc;
  return launch_add_splits(ws, out, m, n, splits, epilogue & 1, stream);
}

}  // namespace tc

int launch_tc_pair(int tl, int tr, uint64_t m, uint64_t n, uint64_t k, const float* left, const float* right,
                   float* out, float* ws, uint32_t splits, int epilogue, cudaStream_t stream) {
  return tc::launch_pair(tl, tr, m, n, k, left, right, out, ws, splits, epilogue, stream);
}

}  // namespace polar_b200
