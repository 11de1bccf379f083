// Host-side check of the tensor-core matmul's work planning (csrc/tc_plan.hpp): the same code
// the kernels run.  For many shapes and both modes it walks every CTA's pieces and verifies
// that each slab of each tile is computed exactly once, that partial tiles get distinct slots
// inside the planned scratch, and that the summing kernel's view of a tile (which teams
// contributed) matches what the CTAs actually did.
#include <tc_plan.hpp>

#include <cstdio>
#include <map>
#include <set>
#include <vector>

using namespace polar_b200::tc;

static int failures = 0;
#define CHECK(cond, ...)                                   \
  do {                                                     \
    if (!(cond)) {                                         \
      if (failures < 20) { std::printf("FAIL %s: ", #cond); std::printf(__VA_ARGS__); std::printf("\n"); } \
      ++failures;                                          \
    }                                                      \
  } while (0)

static void check_cover(uint32_t tiles_m, uint32_t tiles_n, uint32_t num_kb, uint32_t splits, uint32_t share,
                        uint32_t teams, uint32_t grid, uint64_t slot_capacity, const char* what) {
  const uint32_t tiles = tiles_m * tiles_n;
  std::vector<std::vector<uint8_t>> seen(tiles, std::vector<uint8_t>(num_kb, 0));
  std::set<uint32_t> slots;
  std::map<uint32_t, std::set<uint32_t>> teams_of_tile;   // stream mode: partial pieces per tile
  std::set<uint32_t> whole;
  for (uint32_t cta = 0; cta < grid; ++cta) {
    PieceWalk walk(tiles_m, tiles_n, splits, share, teams, num_kb, cta, grid);
    Piece pc;
    uint32_t prev_tile = 0xffffffffu;
    while (walk.next(pc)) {
      CHECK(pc.tile < tiles && pc.kb0 < pc.kb1 && pc.kb1 <= num_kb, "%s tile %u [%u,%u)", what, pc.tile, pc.kb0, pc.kb1);
      if (pc.tile >= tiles) continue;
      for (uint32_t kb = pc.kb0; kb < pc.kb1 && kb < num_kb; ++kb) {
        CHECK(!seen[pc.tile][kb], "%s slab %u of tile %u twice", what, kb, pc.tile);
        seen[pc.tile][kb] = 1;
      }
      if (share) {
        CHECK(pc.tile % tiles_m == cta % tiles_m, "%s cta %u left its row", what, cta);
        CHECK(pc.tile != prev_tile, "%s cta %u got tile %u twice in a row", what, cta, pc.tile);
        prev_tile = pc.tile;
        if (pc.slot == kNoSlot) {
          CHECK(pc.kb0 == 0 && pc.kb1 == num_kb, "%s whole-tile piece is not whole", what);
          whole.insert(pc.tile);
        } else {
          CHECK(slots.insert(pc.slot).second, "%s slot %u used twice", what, pc.slot);
          CHECK(pc.slot < slot_capacity, "%s slot %u beyond the scratch (%llu)", what, pc.slot,
                (unsigned long long)slot_capacity);
          const uint32_t row = pc.tile % tiles_m, col = pc.tile / tiles_m, team = cta / tiles_m;
          CHECK(pc.slot == row * (teams + tiles_n) + team + col, "%s slot formula", what);
          teams_of_tile[pc.tile].insert(team);
        }
      } else {
        CHECK((splits > 1) == (pc.slot != kNoSlot) && (pc.slot == kNoSlot || pc.slot < splits), "%s cut index", what);
      }
    }
  }
  for (uint32_t t = 0; t < tiles; ++t)
    for (uint32_t kb = 0; kb < num_kb; ++kb) CHECK(seen[t][kb], "%s slab %u of tile %u never computed", what, kb, t);
  if (share) {
    for (uint32_t t = 0; t < tiles; ++t) {
      uint32_t first, last;
      stream_teams_of_column(t / tiles_m, num_kb, share, &first, &last);
      if (first == last) {
        CHECK(whole.count(t) == 1 && teams_of_tile.count(t) == 0, "%s tile %u should be whole", what, t);
      } else {
        const auto& ts = teams_of_tile[t];
        CHECK(whole.count(t) == 0 && ts.size() == last - first + 1 && *ts.begin() == first && *ts.rbegin() == last,
              "%s tile %u: teams %zu, expected %u..%u", what, t, ts.size(), first, last);
      }
    }
  }
}

// Whole-tile mode with the tail wave cut into column halves: every tile before `from` once and
// whole, every tile from `from` on as its two halves, each once, on different CTAs; no CTA gets
// more than ceil(whole tiles / grid) whole tiles plus one half.
static void check_halves(uint32_t tiles_m, uint32_t tiles_n, uint32_t num_kb, uint32_t grid) {
  const uint32_t tiles = tiles_m * tiles_n;
  const uint32_t from = halves_from(tiles, grid);
  if (from == kNoHalves) return;
  CHECK(from % grid == 0 && from < tiles && 2 * (tiles - from) <= grid, "halves_from(%u, %u) = %u", tiles, grid, from);
  std::vector<int> whole(tiles, 0), left(tiles, 0), right(tiles, 0);
  for (uint32_t cta = 0; cta < grid; ++cta) {
    PieceWalk walk(tiles_m, tiles_n, 1, 0, 0, num_kb, cta, grid, from);
    Piece pc;
    uint32_t n_whole = 0, n_half = 0;
    while (walk.next(pc)) {
      CHECK(pc.tile < tiles && pc.kb0 == 0 && pc.kb1 == num_kb && pc.slot == kNoSlot, "halves: piece of tile %u", pc.tile);
      if (pc.tile >= tiles) continue;
      if (pc.half == 0) { ++whole[pc.tile]; ++n_whole; CHECK(pc.tile < from, "halves: tile %u whole in the tail", pc.tile); }
      else { ++(pc.half == 1 ? left : right)[pc.tile]; ++n_half; CHECK(pc.tile >= from, "halves: tile %u halved too early", pc.tile); }
    }
    CHECK(n_whole == from / grid && n_half <= 1, "halves: cta %u got %u whole tiles and %u halves", cta, n_whole, n_half);
  }
  for (uint32_t t = 0; t < tiles; ++t)
    CHECK(t < from ? (whole[t] == 1 && !left[t] && !right[t]) : (!whole[t] && left[t] == 1 && right[t] == 1),
          "halves: tile %u covered %d/%d/%d", t, whole[t], left[t], right[t]);
}

int main() {
  const uint64_t sms = 148;
  int cases = 0;
  // stream mode, as the launcher plans it
  for (uint32_t tiles_m : {1u, 2u, 3u, 4u, 6u, 7u, 9u, 16u})
    for (uint32_t tiles_n : {1u, 2u, 5u, 16u, 33u})
      for (uint32_t num_kb : {1u, 7u, 64u, 512u, 1000u, 2048u})
        for (int mt : {1, 2}) {
          const StreamPlan plan = stream_plan(tiles_m, tiles_n, num_kb, 256, mt, sms);
          CHECK(plan.teams > 0 && plan.grid == plan.teams * tiles_m && plan.grid <= sms, "plan %u %u %u", tiles_m, tiles_n, num_kb);
          CHECK((uint64_t)plan.share * plan.teams >= (uint64_t)tiles_n * num_kb, "shares do not cover the work");
          CHECK((uint64_t)plan.share * (plan.teams - 1) < (uint64_t)tiles_n * num_kb, "an idle team was planned");
          const uint64_t tile_bytes = 128ull * mt * 256 * 4;
          check_cover(tiles_m, tiles_n, num_kb, 1, plan.share, plan.teams, plan.grid, plan.bytes / tile_bytes, "stream");
          ++cases;
        }
  CHECK(stream_plan(17, 4, 100, 256, 1, sms).teams == 0, "17 row tiles exceed the raster group");
  // the two shapes the MLP step runs in this mode
  {
    const StreamPlan p8 = stream_plan(7, 16, 512, 256, 1, sms);      // 784 x 4096 x 8192, 128-row tiles
    CHECK(p8.teams == 21 && p8.grid == 147 && p8.share == 391, "dW1 at k = 8192: %u teams, share %u", p8.teams, p8.share);
    const StreamPlan p4 = stream_plan(3, 16, 1024, 256, 2, sms);     // 768 x 4096 x 16384, 256-row tiles
    CHECK(p4.teams == 49 && p4.grid == 147, "dW1 at k = 16384: %u teams", p4.teams);
  }
  // fixed cuts
  for (uint32_t tiles_m : {1u, 3u, 7u, 20u})
    for (uint32_t tiles_n : {1u, 16u})
      for (uint32_t num_kb : {8u, 100u, 4096u})
        for (uint32_t splits : {1u, 2u, 3u, 5u, 8u}) {
          if (splits > num_kb) continue;
          const uint32_t units = tiles_m * tiles_n * splits;
          const uint32_t grid = units < sms ? units : (uint32_t)sms;
          check_cover(tiles_m, tiles_n, num_kb, splits, 0, 0, grid, 0, "cuts");
          ++cases;
        }
  // the tail wave in column halves: the first layer of the MLP at an eighth of the batch (32 x 16
  // tiles of 256 x 256: three waves and 68 tiles), and a sweep
  CHECK(halves_from(512, 148) == 444, "512 tiles on 148 CTAs: %u", halves_from(512, 148));
  CHECK(halves_from(1024, 148) == kNoHalves && halves_from(4096, 148) == kNoHalves && halves_from(100, 148) == kNoHalves &&
        halves_from(296, 148) == kNoHalves, "tails above half a wave, less than a wave, whole waves: no halves");
  for (uint32_t tiles_m : {1u, 3u, 16u, 32u})
    for (uint32_t tiles_n : {1u, 5u, 16u, 50u}) {
      check_halves(tiles_m, tiles_n, 49, (uint32_t)sms);
      check_halves(tiles_m, tiles_n, 49, 7);
      ++cases;
    }
  std::printf("%d cases, %d failures\n", cases, failures);
  return failures ? 1 : 0;
}
