// fmatmul on the 5th-generation tensor cores of B200 (sm_100a): TMA-staged,
// tcgen05.mma with the accumulator in tensor memory, fp32 accuracy through a
// three-product TF32 split.
//
//   C[128 x BN tile] = sum over k slabs of 32:  Ahi*Bhi + Ahi*Blo + Alo*Bhi
//
// where x_hi is the TF32 the tensor core sees when it reads an fp32 word (the
// top 19 bits) and x_lo = x - x_hi, exact in fp32.  The dropped Alo*Blo term and
// the truncation of x_lo to TF32 are each below 2^-21 relative to |a||b|.
//
// One persistent CTA per SM walks 128 x BN output tiles; two accumulators in
// tensor memory let the epilogue of one tile overlap the k loop of the next.  In
// the 256 x BN configuration (MT = 2, see Cfg) both accumulators belong to one
// tile and every B slab serves two row sub-tiles: a third fewer operand bytes per
// flop, which is what limits the 128-row form (24 KB per slab per SM from L2).
// Warp roles:
//   warp 0     TMA producer: cp.async.bulk.tensor loads of the fp32 A and B
//              slabs into 128-byte-swizzled shared memory (plain per-CTA loads:
//              every CTA fetches its own tiles from this GPU's memory / L2);
//   warp 1     allocates tensor memory, issues tcgen05.mma (one elected lane),
//              commits to mbarriers to free stages and to publish the tile;
//   warps 2-9  split warps: read each landed slab, write the lo part
//              (and, when asked, the masked hi part in place) for the async proxy;
//   warps 10-17 epilogue: tcgen05.ld the finished accumulator (two warps per
//              32-lane quarter, half of the columns each), apply the fused
//              activation if asked, store C rows with bounds checks, then hand the
//              accumulator back.
// The hi*hi product of a slab is issued as soon as TMA has delivered it, so the
// split warps' pass over the slab is hidden behind tensor-core work.
//
// All four transpose forms run natively: a K-contiguous operand is a K-major
// SWIZZLE_128B tile (rows of 32 floats), an M- or N-contiguous one is an
// MN-major tile built from 32x32 boxes in the 128-byte swizzle with 32-byte base
// (the only MN-major layout tcgen05 takes for 32-bit operands); only the shared-memory
// descriptors, the instruction descriptor's major bits and the TMA boxes differ.
//
// Shapes with too few tiles to load every SM evenly (e.g. 784 x 4096 with a k of
// 65536: 112 tiles on 148 SMs) are cut along k, either into up to 8 work units per
// tile whose partial products a second kernel adds in a fixed order, or - stream
// mode, for k up to 32768 - into exactly equal shares per team of CTAs, a team
// being one CTA per row tile working the same column tile and k range in lockstep
// (see Params and PieceWalk).  Every warp role walks the same sequence of pieces.
//
// Every wait on an mbarrier is bounded: after about two seconds of polling the
// waiter records a code in the status word, raises the CTA's abort flag, and
// every role leaves its loop; the CTA then lets copies in flight land, frees its
// tensor memory and returns.
#include <cuda.h>

#include <cstdlib>
#include <mutex>

#include "common.cuh"
#include "tc_plan.hpp"
#include "tc_ptx.cuh"

namespace polar_b200 {
namespace tc {

constexpr int BM = 128;
constexpr int kSplitWarps = 8;                                  // warps 2..9
constexpr int kEpilogueWarps = 8;                               // warps 10..17
constexpr int kThreads = 32 * (2 + kSplitWarps + kEpilogueWarps);
constexpr int kGroupM = kPlanGroupM;                            // tile raster: 16 row tiles share their column tiles

// BN: tile width (256 or 128).  BK: floats per k slab (32 -> 128-byte rows, 16 ->
// 64-byte rows); a shallower slab halves the stage and doubles the pipeline depth.
// MT = row sub-tiles of 128 per CTA tile.  MT = 1: 128 x BN tiles, the two tensor-memory
// accumulators alternate between consecutive tiles so the epilogue of one overlaps the k loop
// of the next.  MT = 2: 256 x BN tiles, both accumulators belong to the current tile; every B
// slab fetched from L2, and its split pass, then serves twice the multiply-adds (operand bytes
// per flop drop by a third), at the price of an epilogue that is not overlapped.
template <int BN, int BK, int MT = 1> struct Cfg {
  static constexpr uint32_t kASubBytes = BM * BK * 4;      // one 128-row sub-tile of A
  static constexpr uint32_t kABytes = MT * kASubBytes;
  static constexpr uint32_t kBBytes = BN * BK * 4;
  static constexpr uint32_t kRawBytes = kABytes + kBBytes;
  static constexpr uint32_t kStageBytes = 2 * kRawBytes;   // raw (hi) + lo
  static constexpr int kStages = (int)((200u * 1024u) / kStageBytes);
  static constexpr uint32_t kTileBytes = kStages * kStageBytes;
  // tile buffers + 1 KB alignment slack + barriers/flags
  static constexpr uint32_t kSmemBytes = kTileBytes + 1024 + 256;
  static constexpr uint32_t kTmemCols = 2 * BN;            // two fp32 accumulators
  static constexpr uint32_t kBoxBytes = 32 * BK * 4;       // one MN-major TMA box {32 m/n, BK k}
  static constexpr int kBBoxRows = BN < 128 ? BN : 128;    // a K-major B slab arrives in boxes of 128 rows
};

struct Params {
  uint64_t m, n, k;
  float* out;
  int a_mn_major;   // left operand stored [k,m]
  int b_mn_major;   // right operand stored [k,n]
  int passes;       // 3 = fp32-accurate split, 1 = plain TF32 (diagnostic)
  int write_hi;     // split warps also store the masked hi part in place
  int* status;      // this device's status word (pinned host memory, device-visible)
  unsigned long long wait_ns;   // bound of every mbarrier wait
  uint32_t tiles_m, tiles_n;
  int epilogue;     // 0: store the product; 1: store fsigmoid(product) (only when splits == 1)
  uint32_t splits;  // work units per tile: the k range is cut into `splits` parts
  float* partial;   // [splits][m][n] partial products when splits > 1
  // Stream mode (share > 0; see PieceWalk in tc_plan.hpp): partial tiles go to `slots`,
  // [slot][tile rows][BN] floats.
  uint32_t share;   // slabs per team
  uint32_t teams;
  float* slots;
  int wide_store;   // 256-bit stores in the epilogue where alignment allows
  // The kernel was given the operands in exchanged roles (it computes the transposed product):
  // a tile's rows are columns of the result, whose row length is m.  See launch_tc.
  int out_t;
  // Whole-tile mode: tiles from this one on are computed as two column halves by two CTAs
  // (halves_from in tc_plan.hpp; kNoHalves = none).  256-column tiles only.
  uint32_t half_from;
};

// Tile raster: groups of kGroupM row tiles walk the column tiles together, so the
// CTAs running at the same time share A row panels and B column panels in L2.
__device__ __forceinline__ void tile_coords(uint32_t t, uint32_t tiles_m, uint32_t tiles_n, int bn,
                                            int* m0, int* n0, int bm = BM) {
  const uint32_t per_group = kGroupM * tiles_n;
  const uint32_t g = t / per_group;
  const uint32_t first_m = g * kGroupM;
  const uint32_t rows = (tiles_m - first_m < (uint32_t)kGroupM) ? tiles_m - first_m : (uint32_t)kGroupM;
  const uint32_t r = t - g * per_group;
  *m0 = (int)((first_m + r % rows) * bm);
  *n0 = (int)((r / rows) * bn);
}

template <int BN, int BK, int MT>
__global__ void __launch_bounds__(kThreads, 1)
fmatmul_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                  const Params p) {
  using C = Cfg<BN, BK, MT>;
  constexpr int kTileM = BM * MT;
  // accumulator columns of row sub-tile h of the tile held in buffer `as`
  auto acc_col = [](uint32_t as, int h) { return (uint32_t)((MT == 1 ? as : (uint32_t)h) * BN); };
  constexpr int S = C::kStages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  // barrier block after the tiles
  const uint32_t bar_base = smem_base + C::kTileBytes;
  auto full_raw = [&](int s) { return bar_base + 8u * s; };
  auto full_lo = [&](int s) { return bar_base + 8u * (S + s); };
  auto empty = [&](int s) { return bar_base + 8u * (2 * S + s); };
  auto acc_full = [&](int a) { return bar_base + 8u * (3 * S + a); };
  auto acc_empty = [&](int a) { return bar_base + 8u * (3 * S + 2 + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + C::kTileBytes + 8 * (3 * S + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t num_kb = (uint32_t)((p.k + BK - 1) / BK);
  // Work comes in pieces (PieceWalk): a (tile, split) unit with a fixed share of the k slabs,
  // or, in stream mode, whatever part of a tile falls into this CTA's share of all slabs.
  auto make_walk = [&]() {
    return PieceWalk(p.tiles_m, p.tiles_n, p.splits, p.share, p.teams, num_kb, blockIdx.x, gridDim.x, p.half_from);
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full_raw(s), 1);
      mbar_init(full_lo(s), kSplitWarps * 32);
      mbar_init(empty(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full(a), 1);
      mbar_init(acc_empty(a), (kEpilogueWarps + (MT == 2 ? kSplitWarps : 0)) * 32);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Drains row sub-tiles [h0, h1) of the finished piece in accumulator buffer `as` for lane
  // quarter q (a warp may only touch tensor-memory lanes [32*(warp%4), +32)) and one half of
  // the columns: to the result, to the piece's partial-product buffer, or to its slot.
  const bool vec_ok = ((p.n & 3) == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0) &&
                      ((reinterpret_cast<uintptr_t>(p.partial) & 15) == 0);
  // A thread owns a row of the tile, so a warp's store instruction touches 32 rows: with 256-bit
  // stores each of them is a whole 32-byte sector instead of half of one.
  const bool wide_ok = p.wide_store && ((p.n & 7) == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 31) == 0) &&
                       ((reinterpret_cast<uintptr_t>(p.partial) & 31) == 0) &&
                       ((reinterpret_cast<uintptr_t>(p.slots) & 31) == 0);
  auto drain = [&](const Piece& pc, uint32_t as, int h0, int h1, int q, int half) {
      int m0, n0;
      tile_coords(pc.tile, p.tiles_m, p.tiles_n, BN, &m0, &n0, kTileM);
      // a column half of a tile: its 128 accumulator columns belong to tile columns [n0, n0 + 128)
      const int width = pc.half ? BN / 2 : BN;
      if (pc.half == 2) n0 += BN / 2;
      const bool to_slot = p.share != 0 && pc.slot != kNoSlot;
      float* const out_base = to_slot ? nullptr
                              : (p.splits > 1 ? p.partial + (uint64_t)pc.slot * p.m * p.n : p.out);
      const bool final_piece = !to_slot && p.splits <= 1;      // this store is the result itself
#pragma unroll 1
      for (int h = h0; h < h1; ++h) {
      const uint32_t tile_row = (uint32_t)(h * BM + q * 32 + lane);
      const uint64_t row = (uint64_t)m0 + tile_row;
      const uint32_t tmem_acc = tmem_base + acc_col(as, h) + ((uint32_t)(q * 32) << 16);
      for (int c = half * (width / 2); c < (half + 1) * (width / 2); c += 32) {
        if ((uint64_t)n0 + c >= p.n) break;               // warp-uniform
        uint32_t r[32];
        tmem_ld_32x32(tmem_acc + (uint32_t)c, r);
        tmem_ld_wait();
        if (p.epilogue == 1 && final_piece) {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(sigmoid_clamped(__uint_as_float(r[j])));
        }
        if (p.write_hi == 2) {
          // diagnostic: the accumulator is drained but nothing is stored
        } else if (to_slot) {
          // a whole tile per slot, padding rows and columns included (they hold zeros)
          float* dst = p.slots + ((uint64_t)pc.slot * kTileM + tile_row) * BN + c;
          if (wide_ok) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) st_global_v8(dst + j, r + j);
          } else
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            float4 v = {__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                        __uint_as_float(r[j + 3])};
            *reinterpret_cast<float4*>(dst + j) = v;
          }
        } else if (p.out_t) {
          // A tensor-memory lane is a COLUMN of the result here: the 32 lanes of a warp write 32
          // consecutive floats of one result row with every store instruction (one 128-byte line),
          // where the plain orientation has each lane writing into a row of its own.
          if (row < p.m) {
            float* dst = out_base + ((uint64_t)n0 + c) * p.m + row;
            if ((uint64_t)n0 + c + 32 <= p.n) {
#pragma unroll
              for (int j = 0; j < 32; ++j, dst += p.m) *dst = __uint_as_float(r[j]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j, dst += p.m)
                if ((uint64_t)n0 + c + j < p.n) *dst = __uint_as_float(r[j]);
            }
          }
        } else if (row < p.m) {
          float* dst = out_base + row * p.n + n0 + c;
          if (wide_ok && (uint64_t)n0 + c + 32 <= p.n) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) st_global_v8(dst + j, r + j);
          } else if (vec_ok && (uint64_t)n0 + c + 32 <= p.n) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              float4 v = {__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                          __uint_as_float(r[j + 3])};
              *reinterpret_cast<float4*>(dst + j) = v;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if ((uint64_t)n0 + c + j < p.n) dst[j] = __uint_as_float(r[j]);
          }
        }
      }
      }   // row sub-tiles
  };

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      uint32_t it = 0;   // k slabs issued so far, over all tiles of this CTA
      bool ok = true;
      PieceWalk walk = make_walk();
      Piece pc;
      while (ok && walk.next(pc)) {
        int m0, n0;
        tile_coords(pc.tile, p.tiles_m, p.tiles_n, BN, &m0, &n0, kTileM);
        // a column half of a tile: half of the B slab, at the start of the stage's B area
        const int bn_now = pc.half ? BN / 2 : BN;
        if (pc.half == 2) n0 += BN / 2;
        for (uint32_t kb = pc.kb0, kb_end = pc.kb1; kb < kb_end; ++kb, ++it) {
          const int s = it % S;
          const uint32_t ph = (it / S) & 1u;
          if (!mbar_wait(empty(s), ph ^ 1u, abort_flag, p.status, 101, p.wait_ns)) { ok = false; break; }
          const uint32_t stage = smem_base + s * C::kStageBytes;
          mbar_expect_tx(full_raw(s), C::kABytes + (pc.half ? C::kBBytes / 2 : C::kBBytes));
          const int k0 = (int)(kb * BK);
          if (!p.a_mn_major) {
            for (int h = 0; h < MT; ++h)                               // boxes {BK k, 128 m}
              tma_load_2d(stage + h * C::kASubBytes, &map_a, full_raw(s), k0, m0 + h * BM);
          } else {
            for (int c = 0; c < kTileM / 32; ++c)                      // boxes {32 m, BK k}
              tma_load_2d(stage + c * C::kBoxBytes, &map_a, full_raw(s), m0 + 32 * c, k0);
          }
          const uint32_t bdst = stage + C::kABytes;
          if (!p.b_mn_major) {
            for (int c = 0; c < bn_now / C::kBBoxRows; ++c)            // boxes {BK k, 128 n}
              tma_load_2d(bdst + c * (C::kBBoxRows * BK * 4), &map_b, full_raw(s), k0, n0 + C::kBBoxRows * c);
          } else {
            for (int c = 0; c < bn_now / 32; ++c)                      // boxes {32 n, BK k}
              tma_load_2d(bdst + c * C::kBoxBytes, &map_b, full_raw(s), n0 + 32 * c, k0);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t idesc_whole = make_idesc(BM, BN, p.a_mn_major, p.b_mn_major);
      const uint32_t idesc_half = make_idesc(BM, BN / 2, p.a_mn_major, p.b_mn_major);
      // K-major: rows of BK floats (128 or 64 bytes, swizzled over that span:
      // layout 2 or 4), 8-row groups 8*BK*4 bytes apart (SBO); a k step of 8 floats
      // is +32 B inside the swizzle span.
      // MN-major (128B swizzle, 32B base: layout 1): rows of 32 m/n-contiguous
      // floats, one row per k; 4-row swizzle atoms 512 B apart along k (SBO);
      // 32-element chunks of m/n one TMA box apart (LBO); a k step of 8 = +1024 B.
      constexpr uint32_t kRowGroup = 8u * BK * 4u;
      constexpr uint32_t kKMajorLayout = (BK == 32) ? 2u : 4u;
      const uint32_t a_lbo = p.a_mn_major ? C::kBoxBytes : 16u, a_step = p.a_mn_major ? 1024u : 32u;
      const uint32_t b_lbo = p.b_mn_major ? C::kBoxBytes : 16u, b_step = p.b_mn_major ? 1024u : 32u;
      const uint32_t a_sbo = p.a_mn_major ? 512u : kRowGroup, a_lt = p.a_mn_major ? 1u : kKMajorLayout;
      const uint32_t b_sbo = p.b_mn_major ? 512u : kRowGroup, b_lt = p.b_mn_major ? 1u : kKMajorLayout;
      uint32_t it = 0, tile_iter = 0;
      bool ok = true;
      PieceWalk walk = make_walk();
      Piece pc;
      for (; ok && walk.next(pc); ++tile_iter) {
        // MT = 1: the two accumulators alternate, the epilogue must have drained this one (two
        // tiles ago).  MT = 2: one buffer of two accumulators, drained after every tile.
        const uint32_t as = MT == 1 ? (tile_iter & 1u) : 0u;
        const uint32_t use = MT == 1 ? (tile_iter >> 1) : tile_iter;   // how often this buffer was used
        ok = mbar_wait(acc_empty(as), (use & 1u) ^ 1u, abort_flag, p.status, 106, p.wait_ns);
        if (!ok) break;
        tc_fence_after();
        const uint32_t idesc = pc.half ? idesc_half : idesc_whole;   // a column half: 128-column MMAs
        const uint32_t kb_first = pc.kb0;
        for (uint32_t kb = kb_first, kb_end = pc.kb1; kb < kb_end; ++kb, ++it) {
          const int s = it % S;
          const uint32_t ph = (it / S) & 1u;
          ok = mbar_wait(full_raw(s), ph, abort_flag, p.status, 102, p.wait_ns);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_hi = smem_base + s * C::kStageBytes;
          const uint32_t b_hi = a_hi + C::kABytes;
          const uint32_t a_lo = a_hi + C::kRawBytes;
          const uint32_t b_lo = b_hi + C::kRawBytes;
          // hi*hi needs only what TMA delivered: issue it while the split warps work
#pragma unroll
          for (int kk = 0; kk < BK / 8; ++kk) {
            const uint64_t db_hi = make_desc(b_hi + kk * b_step, b_lbo, b_sbo, b_lt);
#pragma unroll
            for (int h = 0; h < MT; ++h) {
              const uint64_t da_hi = make_desc(a_hi + h * C::kASubBytes + kk * a_step, a_lbo, a_sbo, a_lt);
              tc_mma_tf32(tmem_base + acc_col(as, h), da_hi, db_hi, idesc,
                          ((kb - kb_first) | (uint32_t)kk) ? 1u : 0u);
            }
          }
          if (p.passes == 3) {
            ok = mbar_wait(full_lo(s), ph, abort_flag, p.status, 103, p.wait_ns);
            if (!ok) break;
            tc_fence_after();
#pragma unroll
            for (int kk = 0; kk < BK / 8; ++kk) {
              const uint64_t db_hi = make_desc(b_hi + kk * b_step, b_lbo, b_sbo, b_lt);
              const uint64_t db_lo = make_desc(b_lo + kk * b_step, b_lbo, b_sbo, b_lt);
#pragma unroll
              for (int h = 0; h < MT; ++h) {
                const uint32_t sub = h * C::kASubBytes + kk * a_step;
                const uint64_t da_hi = make_desc(a_hi + sub, a_lbo, a_sbo, a_lt);
                const uint64_t da_lo = make_desc(a_lo + sub, a_lbo, a_sbo, a_lt);
                tc_mma_tf32(tmem_base + acc_col(as, h), da_lo, db_hi, idesc, 1u);
                tc_mma_tf32(tmem_base + acc_col(as, h), da_hi, db_lo, idesc, 1u);
              }
            }
          }
          if (p.passes == 13) {
            // diagnostic: the issue rate of three products per slab with no split
            // pass at all (the result is 3 x the plain TF32 product)
#pragma unroll
            for (int kk = 0; kk < BK / 8; ++kk) {
              const uint64_t db_hi = make_desc(b_hi + kk * b_step, b_lbo, b_sbo, b_lt);
#pragma unroll
              for (int h = 0; h < MT; ++h) {
                const uint64_t da_hi = make_desc(a_hi + h * C::kASubBytes + kk * a_step, a_lbo, a_sbo, a_lt);
                tc_mma_tf32(tmem_base + acc_col(as, h), da_hi, db_hi, idesc, 1u);
                tc_mma_tf32(tmem_base + acc_col(as, h), da_hi, db_hi, idesc, 1u);
              }
            }
          }
          tc_commit(empty(s));   // frees the stage once these MMAs have read it
        }
        if (ok) tc_commit(acc_full(as));
      }
    }
  } else if (warp < 2 + kSplitWarps) {
    // ---------------- split warps ----------------
    const int tid = threadIdx.x - 64;  // 0..255
    if (p.passes == 3 || MT == 2) {
      uint32_t it = 0, tile_iter = 0;
      bool ok = true;
      PieceWalk walk = make_walk();
      Piece pc;
      for (; ok && walk.next(pc); ++tile_iter) {
        for (uint32_t kb = pc.kb0, kb_end = pc.kb1; p.passes == 3 && kb < kb_end; ++kb, ++it) {
          const int s = it % S;
          const uint32_t ph = (it / S) & 1u;
          if (!mbar_wait(full_raw(s), ph, abort_flag, p.status, 104, p.wait_ns)) { ok = false; break; }
          float4* raw = reinterpret_cast<float4*>(smem_gen + s * C::kStageBytes);
          float4* lo = reinterpret_cast<float4*>(smem_gen + s * C::kStageBytes + C::kRawBytes);
          constexpr int kVecs = C::kRawBytes / 16;
          static_assert(kVecs % (kSplitWarps * 32) == 0, "slab must divide over the split warps");
#pragma unroll
          for (int i = 0; i < kVecs / (kSplitWarps * 32); ++i) {
            const int e = tid + i * kSplitWarps * 32;
            float4 v = raw[e];
            float4 h;
            h.x = __uint_as_float(__float_as_uint(v.x) & 0xFFFFE000u);
            h.y = __uint_as_float(__float_as_uint(v.y) & 0xFFFFE000u);
            h.z = __uint_as_float(__float_as_uint(v.z) & 0xFFFFE000u);
            h.w = __uint_as_float(__float_as_uint(v.w) & 0xFFFFE000u);
            float4 l = {v.x - h.x, v.y - h.y, v.z - h.z, v.w - h.w};
            lo[e] = l;
            if (p.write_hi == 1) raw[e] = h;
          }
          fence_async_smem();
          mbar_arrive(full_lo(s));
        }
        if (MT == 2 && ok) {
          // 256-row tiles: nothing is left to split until this tile is drained, so these
          // warps drain its lower sub-tile while the epilogue warps drain the upper one
          if (!mbar_wait(acc_full(0), tile_iter & 1u, abort_flag, p.status, 107, p.wait_ns)) break;
          tc_fence_after();
          drain(pc, 0, 1, 2, warp & 3, (warp - 2) >> 2);
          tc_fence_before();
          mbar_arrive(acc_empty(0));
        }
      }
    }
  } else {
    // ---------------- epilogue warps ----------------
    // Four consecutive warps cover the 128 rows of a sub-tile; the two warps of a lane quarter
    // take half of the columns each.  With 256-row tiles these warps drain the upper sub-tile
    // and the split warps, idle at that point, the lower one.
    const int q = warp & 3;
    const int half = (warp - (2 + kSplitWarps)) >> 2;
    uint32_t tile_iter = 0;
    PieceWalk walk = make_walk();
    Piece pc;
    for (; walk.next(pc); ++tile_iter) {
      const uint32_t as = MT == 1 ? (tile_iter & 1u) : 0u;
      const uint32_t use = MT == 1 ? (tile_iter >> 1) : tile_iter;
      if (!mbar_wait(acc_full(as), use & 1u, abort_flag, p.status, 105, p.wait_ns)) break;
      tc_fence_after();
      drain(pc, as, 0, 1, q, half);
      tc_fence_before();
      mbar_arrive(acc_empty(as));   // this accumulator may be overwritten
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // let copies and MMAs in flight finish before the tensor memory goes away
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000ll) { }
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// ---- host side --------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// 2-D fp32 tensor map: `inner` contiguous elements per row, `outer` rows.
// `pitch` (floats between consecutive outer rows; 0 = inner) lets a map cover the first
// `inner` columns of a wider stored matrix.
int make_map(CUtensorMap* map, const float* base, uint64_t inner, uint64_t outer,
                    uint32_t box_inner, uint32_t box_outer, bool mn_major, int bk, uint64_t pitch = 0) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return fail(POLAR_B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {(pitch ? pitch : inner) * 4};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                            : (bk == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B),
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(POLAR_B200_ERR_CUDA, "cuTensorMapEncodeTiled failed");
  return POLAR_B200_OK;
}

bool shape_ok(int tl, int tr, uint64_t m, uint64_t n, uint64_t k, const float* left,
              const float* right) {
  // TMA: 16-byte aligned base, row pitch a multiple of 16 bytes.
  if (!aligned16(left) || !aligned16(right)) return false;
  uint64_t a_inner = tl ? m : k, b_inner = tr ? k : n;
  if ((a_inner & 3) || (b_inner & 3)) return false;
  if (m >= (1ull << 31) || n >= (1ull << 31) || k >= (1ull << 31)) return false;
  return m > 0 && n > 0 && k > 0;
}

// out[e] = sum of the splits' partial products, ascending split index (fixed order).  The
// partial products live in 16-byte aligned scratch; `out` is the caller's and may be only
// 4-byte aligned, in which case the four sums are stored one by one.
__global__ void __launch_bounds__(256) add_splits_kernel(const float4* __restrict__ partial, float* __restrict__ out,
                                                         uint64_t nvec, uint32_t splits, int epilogue, int out_vec) {
  const uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= nvec) return;
  float4 s = __ldcs(partial + i);
  for (uint32_t sp = 1; sp < splits; ++sp) {
    float4 v = __ldcs(partial + (uint64_t)sp * nvec + i);
    s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
  }
  if (epilogue == 1) {
    s.x = sigmoid_clamped(s.x); s.y = sigmoid_clamped(s.y); s.z = sigmoid_clamped(s.z); s.w = sigmoid_clamped(s.w);
  }
  if (out_vec) {
    reinterpret_cast<float4*>(out)[i] = s;
  } else {
    float* o = out + 4 * i;
    o[0] = s.x; o[1] = s.y; o[2] = s.z; o[3] = s.w;
  }
}

int launch_add_splits(const float* ws, float* out, uint64_t m, uint64_t n, uint32_t splits, int epilogue,
                      cudaStream_t stream) {
  const uint64_t nvec = m * n / 4;
  add_splits_kernel<<<(unsigned)((nvec + 255) / 256), 256, 0, stream>>>(reinterpret_cast<const float4*>(ws), out, nvec,
                                                                       splits, epilogue, aligned16(out) ? 1 : 0);
  return check_launch("fmatmul_add_splits");
}

// How many ways to cut k so that the persistent grid is evenly loaded: the smallest
// count up to 8 whose last wave is at least 90 % full, else the best one.  Needs
// m*n to be a multiple of 4 for the vectorised sum of the partial products.
// Stream mode: the tiles whose slabs were shared between teams are summed from their slots,
// in ascending team order (a fixed order).  Tiles that one CTA computed whole are in `out` already.
template <int BN, int MT>
__global__ void __launch_bounds__(256) stream_reduce_kernel(const float* __restrict__ slots, float* __restrict__ out,
                                                            uint64_t m, uint64_t n, uint32_t tiles_m, uint32_t tiles_n,
                                                            uint32_t num_kb, uint32_t share, uint32_t teams,
                                                            int epilogue) {
  constexpr uint32_t kVecsPerTile = BM * MT * BN / 4;
  constexpr uint32_t kBlocksPerTile = kVecsPerTile / 256;
  const uint32_t tile = blockIdx.x / kBlocksPerTile;
  const uint32_t v = (blockIdx.x % kBlocksPerTile) * 256 + threadIdx.x;
  const uint32_t trow = tile % tiles_m, col_tile = tile / tiles_m;
  uint32_t t_first, t_last;
  stream_teams_of_column(col_tile, num_kb, share, &t_first, &t_last);
  if (t_first == t_last) return;
  int m0, n0;
  tile_coords(tile, tiles_m, tiles_n, BN, &m0, &n0, BM * MT);
  const uint32_t r = v / (BN / 4), c = (v % (BN / 4)) * 4;
  const uint64_t row = (uint64_t)m0 + r, col = (uint64_t)n0 + c;
  if (row >= m || col >= n) return;
  const uint64_t first_slot = (uint64_t)trow * (teams + tiles_n) + t_first + col_tile;
  const float4* src = reinterpret_cast<const float4*>(slots) + (first_slot * kVecsPerTile + v);
  float4 acc = __ldcg(src);
  for (uint32_t t = t_first + 1; t <= t_last; ++t) {
    src += kVecsPerTile;
    const float4 x = __ldcg(src);
    acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
  }
  if (epilogue == 1) {
    acc.x = sigmoid_clamped(acc.x); acc.y = sigmoid_clamped(acc.y);
    acc.z = sigmoid_clamped(acc.z); acc.w = sigmoid_clamped(acc.w);
  }
  float* dst = out + row * n + col;
  if ((n & 3) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
    *reinterpret_cast<float4*>(dst) = acc;
  } else {
    dst[0] = acc.x;
    if (col + 1 < n) dst[1] = acc.y;
    if (col + 2 < n) dst[2] = acc.z;
    if (col + 3 < n) dst[3] = acc.w;
  }
}

uint32_t choose_splits(uint64_t tiles, uint64_t num_kb, uint64_t m, uint64_t n, int mt = 1) {
  const uint64_t sms = (uint64_t)sm_count();
  if (tiles >= 8 * sms) return 1;
  // last wave at least 95 % full with whole tiles: nothing to gain from cutting k
  if ((double)tiles / (double)(((tiles + sms - 1) / sms) * sms) >= 0.95) return 1;
  // Stream mode (0): teams of CTAs in lockstep with perfectly even shares; taken when it keeps
  // at least 95 % of the SMs busy and every team still gets a decent run of slabs.  Measured in
  // the MLP step (dW1, 784 x 4096 x k) against the fixed cuts below: the step takes 0.714 vs
  // 0.730 ms at k = 8192, 1.317 vs 1.340 ms at 16384, 2.58 vs 2.60 ms at 32768, but 5.21 vs
  // 5.17 ms at 65536, where both balance equally well - so fixed cuts keep the long sums.
  if (num_kb <= 2048) {
    const StreamPlan plan = stream_plan((m + BM * mt - 1) / (BM * mt), (n + 255) / 256, num_kb, 256, mt, sms);
    if (plan.teams && plan.share >= 64 && (double)plan.grid >= 0.95 * (double)sms) return 0;
  }
  if (((m * n) & 3) != 0) return 1;
  double best_eff = 0.0;
  uint32_t best = 1;
  for (uint32_t s = 1; s <= 8; ++s) {
    if (num_kb / s < 32) break;                       // keep at least 32 slabs per unit
    const uint64_t units = tiles * s;
    const double eff = (double)units / (double)(((units + sms - 1) / sms) * sms);
    if (eff >= 0.9) return s;
    if (eff > best_eff + 0.02) { best_eff = eff; best = s; }
  }
  return best;
}

static bool wide_store_enabled() {
  static const bool on = [] {
    const char* e = getenv("POLAR_B200_TC_STORE_BITS");
    return !(e && atoi(e) == 128);
  }();
  return on;
}

static bool halves_enabled() {
  static const bool on = [] {
    const char* e = getenv("POLAR_B200_TC_TAIL_HALVES");
    return !(e && atoi(e) == 0);
  }();
  return on;
}

template <int BN, int BK, int MT = 1>
static int launch_cfg(int tl, int tr, uint64_t m, uint64_t n, uint64_t k, const float* left,
                      const float* right, float* out, int passes, int write_hi, float* ws, uint32_t splits,
                      int epilogue, cudaStream_t stream, uint64_t left_pitch, int out_t) {
  using C = Cfg<BN, BK, MT>;
  static_assert(C::kStages >= 2 && C::kSmemBytes <= 227 * 1024, "stage ring must fit shared memory");
  int dev = 0;
  cudaGetDevice(&dev);
  static bool attr_done[64] = {false};
  if (dev >= 0 && dev < 64 && !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(fmatmul_tc_kernel<BN, BK, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)C::kSmemBytes);
    if (e != cudaSuccess) return fail(POLAR_B200_ERR_CUDA, "cudaFuncSetAttribute(smem)", e);
    attr_done[dev] = true;
  }
  int rc = POLAR_B200_OK;
  int* status_word = device_status_word(&rc);
  if (!status_word) return rc;
  CUtensorMap map_a, map_b;
  // left: stored [m,k] (K-major: inner k, box {BK, 128}) or [k,m] (MN-major: inner m, box {32, BK})
  rc = tl ? make_map(&map_a, left, m, k, 32, BK, true, BK, left_pitch)
          : make_map(&map_a, left, k, m, BK, BM, false, BK, left_pitch);
  if (rc) return rc;
  // right: stored [n,k] when transposed (K-major: inner k, box {BK, BN}) or [k,n] (MN-major)
  rc = tr ? make_map(&map_b, right, k, n, BK, C::kBBoxRows, false, BK) : make_map(&map_b, right, n, k, 32, BK, true, BK);
  if (rc) return rc;
  Params p;
  p.m = m; p.n = n; p.k = k; p.out = out;
  p.a_mn_major = tl ? 1 : 0;
  p.b_mn_major = tr ? 0 : 1;
  p.passes = passes; p.write_hi = write_hi; p.status = status_word;
  p.wait_ns = wait_limit_ns(2000000000ull);
  p.wide_store = wide_store_enabled() ? 1 : 0;
  p.out_t = out_t;
  if (out_t && (splits == 0 || left_pitch))
    return fail(POLAR_B200_ERR_UNSUPPORTED, "exchanged operands: whole tiles or fixed k cuts only, no row pitch");
  uint64_t tm = (m + BM * MT - 1) / (BM * MT), tn = (n + BN - 1) / BN;
  if (tm * tn > 0x7fffffffull) return fail(POLAR_B200_ERR_UNSUPPORTED, "too many tiles");
  p.tiles_m = (uint32_t)tm; p.tiles_n = (uint32_t)tn;
  const uint64_t num_kb = (k + BK - 1) / BK;
  p.share = 0;
  p.slots = nullptr;
  p.teams = 0;
  p.half_from = kNoHalves;
  const StreamPlan plan = (splits == 0 && ws) ? stream_plan(tm, tn, num_kb, BN, MT, (uint64_t)sm_count()) : StreamPlan{0, 0, 0, 0};
  if (plan.teams) {
    // stream mode: equal shares of all slabs, partial tiles through slots, then one summing pass
    p.splits = 1;
    p.partial = nullptr;
    p.epilogue = epilogue;
    p.share = plan.share;
    p.teams = plan.teams;
    p.slots = ws;
    fmatmul_tc_kernel<BN, BK, MT><<<plan.grid, kThreads, C::kSmemBytes, stream>>>(map_a, map_b, p);
    rc = check_launch("fmatmul_tc");
    if (rc) return rc;
    constexpr uint32_t kBlocksPerTile = BM * MT * BN / 4 / 256;
    stream_reduce_kernel<BN, MT><<<(unsigned)(tm * tn * kBlocksPerTile), 256, 0, stream>>>(
        ws, out, m, n, p.tiles_m, p.tiles_n, (uint32_t)num_kb, plan.share, plan.teams, epilogue);
    return check_launch("fmatmul_stream_reduce");
  }
  if (splits < 1 || !ws || splits > num_kb) splits = 1;
  p.splits = splits;
  p.partial = splits > 1 ? ws : nullptr;
  p.epilogue = splits > 1 ? 0 : epilogue;
  uint64_t units = tm * tn * splits;
  if (units > 0x7fffffffull) return fail(POLAR_B200_ERR_UNSUPPORTED, "too many tiles");
  unsigned grid = (unsigned)(units < (uint64_t)sm_count() ? units : (uint64_t)sm_count());   // one CTA per SM
  if (splits == 1 && BN == 256 && halves_enabled()) p.half_from = halves_from(units, grid);
  fmatmul_tc_kernel<BN, BK, MT><<<grid, kThreads, C::kSmemBytes, stream>>>(map_a, map_b, p);
  rc = check_launch("fmatmul_tc");
  if (rc || splits == 1) return rc;
  return launch_add_splits(ws, out, m, n, splits, epilogue, stream);
}

}  // namespace tc

// swap_ab: the operands exchange roles.  out[m,n] = L.R is computed as its transpose
// R'.L' [n,m] - `right` becomes the operand whose rows are tensor-memory lanes - and the epilogue
// stores tile element (lane i, column j) at out[j][i]: consecutive lanes then write consecutive
// floats of a result row.  The products and the order of the sum over k are the same; only the
// two cross terms of the split (lo.hi, hi.lo) are added in exchanged order.  Pays where the
// epilogue is a visible part of a tile's time, i.e. for short sums.
int launch_tc(int tl, int tr, uint64_t m, uint64_t n, uint64_t k, const float* left,
              const float* right, float* out, int bn, int bk, int passes, int write_hi, float* ws,
              uint32_t splits, int epilogue, cudaStream_t stream, uint64_t left_pitch, int mt, int swap_ab) {
  if (swap_ab) {
    // left' = right: stored [k,n] (tr = 0) is "stored [k,m']" (tl' = 1); right' = left: stored
    // [m,k] (tl = 0) is "stored [n',k]" (tr' = 1)
    const int tl2 = tr ? 0 : 1, tr2 = tl ? 0 : 1;
    const float* l2 = right;
    const float* r2 = left;
    const uint64_t m2 = n, n2 = m;
    tl = tl2; tr = tr2; left = l2; right = r2; m = m2; n = n2;
  }
  if (mt == 2)   // 256 x 256 tiles, 16-float slabs
    return tc::launch_cfg<256, 16, 2>(tl, tr, m, n, k, left, right, out, passes, write_hi, ws, splits, epilogue, stream, left_pitch, swap_ab);
  if (bn == 128 && bk == 32)
    return tc::launch_cfg<128, 32>(tl, tr, m, n, k, left, right, out, passes, write_hi, ws, splits, epilogue, stream, left_pitch, swap_ab);
  if (bn == 128)
    return tc::launch_cfg<128, 16>(tl, tr, m, n, k, left, right, out, passes, write_hi, ws, splits, epilogue, stream, left_pitch, swap_ab);
  if (bk == 32)
    return tc::launch_cfg<256, 32>(tl, tr, m, n, k, left, right, out, passes, write_hi, ws, splits, epilogue, stream, left_pitch, swap_ab);
  return tc::launch_cfg<256, 16>(tl, tr, m, n, k, left, right, out, passes, write_hi, ws, splits, epilogue, stream, left_pitch, swap_ab);
}

// Whether a whole-tile launch of `tiles` 256-column tiles on `grid` CTAs cuts its last wave into column halves.
bool tc_tail_in_halves(uint64_t tiles, uint64_t grid) {
  return tc::halves_enabled() && tc::halves_from(tiles, grid) != tc::kNoHalves;
}

// Splits the default configuration (128 x 256 tiles, 16-float slabs) would use.
// mt = row sub-tiles per CTA tile: 1 (128 x 256 tiles) or 2 (256 x 256).
uint32_t tc_default_splits(uint64_t m, uint64_t n, uint64_t k, int mt) {
  const uint64_t rows = 128ull * mt;
  return tc::choose_splits(((m + rows - 1) / rows) * ((n + 255) / 256), (k + 15) / 16, m, n, mt);
}

// Scratch the default configuration needs for `splits` (0 = stream mode) work units per tile.
uint64_t tc_workspace_bytes(uint64_t m, uint64_t n, uint64_t k, uint32_t splits, int mt) {
  const uint64_t rows = 128ull * mt;
  if (splits == 0) return tc::stream_plan((m + rows - 1) / rows, (n + 255) / 256, (k + 15) / 16, 256, mt, (uint64_t)sm_count()).bytes;
  return splits > 1 ? (uint64_t)splits * m * n * sizeof(float) : 0;
}

bool tc_shape_ok(int tl, int tr, uint64_t m, uint64_t n, uint64_t k, const float* left,
                 const float* right) {
  return tc::shape_ok(tl, tr, m, n, k, left, right);
}


}  // namespace polar_b200
