// Work planning of the tensor-core matmul: which slabs of which tiles a CTA computes, in which
// order, and where partial tiles go.  Plain C++ (host and device), so that the arithmetic the
// kernel, the summing kernels and the scratch sizing must agree on can be tested on a CPU.
#pragma once
#include <stdint.h>

#ifdef __CUDACC__
#define POLAR_HD __host__ __device__ __forceinline__
#else
#define POLAR_HD inline
#endif

namespace polar_b200 {
namespace tc {

constexpr int kPlanTileRows = 128;      // rows of one row sub-tile
constexpr int kPlanGroupM = 16;         // tile raster: 16 row tiles share their column tiles
constexpr uint32_t kNoSlot = 0xffffffffu;

// One piece of work: slabs [kb0, kb1) of a tile.  Every warp role walks the same sequence.
// slot: kNoSlot = the piece is the whole tile and is stored as the result; otherwise the index
// of its partial product (fixed cuts: the cut; stream mode: the slot).
// half: 0 = the tile's whole width; 1, 2 = its left, right half of the columns (see PieceWalk).
struct Piece {
  uint32_t tile, kb0, kb1, slot, half;
};

constexpr uint32_t kNoHalves = 0xffffffffu;

// Whole tiles dealt round-robin leave the last wave partly empty: 512 tiles on 148 CTAs are three
// full waves and 68 tiles, and the kernel lasts four tile times.  When that tail is at most half
// a wave its tiles are cut into column halves, one CTA each, and the kernel lasts about 3.6.
// Returns the first tile of the tail (tiles before it stay whole), or kNoHalves.
POLAR_HD uint32_t halves_from(uint64_t tiles, uint64_t grid) {
  if (grid == 0 || tiles < grid) return kNoHalves;
  const uint64_t full = (tiles / grid) * grid, tail = tiles - full;
  return (tail > 0 && 2 * tail <= grid) ? (uint32_t)full : kNoHalves;
}

// Fixed cuts (share == 0): work unit u = (tile u / splits, cut u % splits), units dealt to CTAs
// round-robin.  Stream mode (share > 0): CTAs form teams of tiles_m, one CTA per row tile; the
// teams cut the sequence (column tile 0, all its k slabs), (column tile 1, ...), ... into equal
// shares of `share` slabs; a share may end inside a column and the next team continues it.  The
// CTAs of a team work on the same column and the same k at the same time, so they share the
// column's operand panel in L2.  A piece that is not a whole tile goes to slot
// row * (teams + tiles_n) + team + column: along a row, consecutive pieces advance the team or
// the column, so the slot numbers are distinct.
// Whole-tile mode (splits == 1) with half_from != kNoHalves: units below half_from are whole tiles,
// every tile from half_from on is two units, its left and its right column half.
struct PieceWalk {
  uint32_t num_kb, splits, num_units, unit, stride, half_from;
  uint32_t row, team, tiles_m, slot_base;
  uint64_t g, g_end;
  bool stream;
  POLAR_HD PieceWalk(uint32_t tiles_m_, uint32_t tiles_n, uint32_t splits_, uint32_t share, uint32_t teams,
                     uint32_t nkb, uint32_t cta, uint32_t grid, uint32_t half_from_ = kNoHalves) {
    num_kb = nkb;
    splits = splits_;
    num_units = tiles_m_ * tiles_n * splits_;
    half_from = (share == 0 && splits_ == 1 && half_from_ < num_units) ? half_from_ : kNoHalves;
    if (half_from != kNoHalves) num_units = half_from + 2 * (num_units - half_from);
    unit = cta;
    stride = grid;
    stream = share != 0;
    tiles_m = tiles_m_;
    row = cta % tiles_m_;
    team = cta / tiles_m_;
    slot_base = row * (teams + tiles_n) + team;
    const uint64_t total = (uint64_t)tiles_n * nkb;
    g = (uint64_t)team * share;
    g_end = g + share < total ? g + share : total;
    if (team >= teams) g = g_end = 0;
  }
  POLAR_HD bool next(Piece& pc) {
    if (!stream) {
      if (unit >= num_units) return false;
      if (unit >= half_from) {
        const uint32_t h = unit - half_from;
        pc.tile = half_from + h / 2;
        pc.half = 1 + (h & 1u);
        pc.kb0 = 0;
        pc.kb1 = num_kb;
        pc.slot = kNoSlot;
        unit += stride;
        return true;
      }
      pc.half = 0;
      const uint32_t sp = unit % splits;
      pc.tile = unit / splits;
      pc.kb0 = (uint32_t)(((uint64_t)sp * num_kb) / splits);
      pc.kb1 = (uint32_t)(((uint64_t)(sp + 1) * num_kb) / splits);
      pc.slot = splits > 1 ? sp : kNoSlot;
      unit += stride;
      return true;
    }
    if (g >= g_end) return false;
    pc.half = 0;
    const uint32_t col = (uint32_t)(g / num_kb);
    pc.tile = col * tiles_m + row;        // the tile raster's numbering when tiles_m <= kPlanGroupM
    pc.kb0 = (uint32_t)(g % num_kb);
    const uint64_t left = g_end - g;
    pc.kb1 = (uint64_t)pc.kb0 + left < num_kb ? (uint32_t)(pc.kb0 + left) : num_kb;
    pc.slot = (pc.kb0 == 0 && pc.kb1 == num_kb) ? kNoSlot : slot_base + col;
    g += pc.kb1 - pc.kb0;
    return true;
  }
};

// Stream mode: the teams whose shares touch column tile `col` (inclusive range).  One team:
// that team computed the column's tiles whole.
POLAR_HD void stream_teams_of_column(uint32_t col, uint32_t num_kb, uint32_t share, uint32_t* first,
                                     uint32_t* last) {
  *first = (uint32_t)(((uint64_t)col * num_kb) / share);
  *last = (uint32_t)((((uint64_t)col + 1) * num_kb - 1) / share);
}

// Stream mode geometry: teams of tiles_m CTAs, slabs per team, CTAs in all, scratch.
// teams == 0: the shape does not suit the mode (more row tiles than the raster's group, or
// than SMs).
struct StreamPlan {
  uint32_t grid, share, teams;
  uint64_t bytes;
};
inline StreamPlan stream_plan(uint64_t tiles_m, uint64_t tiles_n, uint64_t num_kb, int bn, int mt, uint64_t sms) {
  if (tiles_m == 0 || tiles_m > (uint64_t)kPlanGroupM || tiles_m > sms) return StreamPlan{0, 0, 0, 0};
  const uint64_t total = tiles_n * num_kb;
  uint64_t teams = sms / tiles_m;
  if (teams > total) teams = total;
  const uint64_t share = (total + teams - 1) / teams;
  teams = (total + share - 1) / share;
  return StreamPlan{(uint32_t)(teams * tiles_m), (uint32_t)share, (uint32_t)teams,
                    tiles_m * (teams + tiles_n) * (uint64_t)(kPlanTileRows * mt) * (uint64_t)bn * sizeof(float)};
}

}  // namespace tc
}  // namespace polar_b200
