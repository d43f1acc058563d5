// Host-side check of the GEMM kernel's work decomposition (gemm_sm100.cuh: decode_tile,
// work_begin, work_next): plain integer arithmetic compiled for the host, no GPU needed.
// Reads "tiles_m tiles_n num_kb splits grid sk_units" lines from stdin and prints, per line,
// "ok" or a description of the first violated property:
//   * every (tile, k-block) is visited exactly once over all CTAs;
//   * a tile's segments are numbered 0 .. nseg-1 without gaps, in k order, and every CTA that
//     touches the tile agrees on nseg;
//   * no tile has more segments than the slots the host reserves (sk_max_seg).
#include <cstdio>
#include <vector>

#include "../../warpir_b200/csrc/gemm_sm100.cuh"

int main() {
  int tiles_m, tiles_n, num_kb, splits, grid, sk_units;
  while (std::scanf("%d %d %d %d %d %d", &tiles_m, &tiles_n, &num_kb, &splits, &grid, &sk_units) == 6) {
    wir::GemmParams p{};
    p.tiles_m = tiles_m;
    p.tiles_n = tiles_n;
    p.num_kb = num_kb;
    p.sk_units = sk_units;
    p.kb_per_split = (num_kb + splits - 1) / splits;
    p.splits = sk_units ? 1 : (num_kb + p.kb_per_split - 1) / p.kb_per_split;
    p.sk_max_seg = sk_units ? (num_kb + sk_units - 2) / sk_units + 1 : p.splits;
    const int tiles = tiles_m * tiles_n;
    std::vector<int> seen(static_cast<size_t>(tiles) * num_kb, 0);
    const char* bad = nullptr;
    // CTAs in index order: with stream-K a tile's segments are owned by consecutive CTAs, and with
    // the static split the splits of a tile are consecutive work items
    for (int pass = 0; pass < 1 && !bad; ++pass) {
      std::vector<std::vector<wir::TileCoord>> per_cta(grid);
      for (int cta = 0; cta < grid; ++cta) {
        wir::WorkIter it = wir::work_begin(p, cta, grid);
        wir::TileCoord t;
        while (wir::work_next(it, p, t)) per_cta[cta].push_back(t);
      }
      // replay in k order per tile: sort by (tile, split) via simple bucket pass
      std::vector<std::vector<wir::TileCoord>> per_tile(tiles);
      for (int cta = 0; cta < grid; ++cta)
        for (const wir::TileCoord& t : per_cta[cta]) {
          if (t.tile < 0 || t.tile >= tiles) { bad = "tile index out of range"; break; }
          if (t.m_blk < 0 || t.m_blk >= tiles_m || t.n_blk < 0 || t.n_blk >= tiles_n) { bad = "block coordinates out of range"; break; }
          per_tile[t.tile].push_back(t);
        }
      std::vector<int> coord(static_cast<size_t>(tiles), 0);
      for (int tile = 0; tile < tiles && !bad; ++tile) {
        auto& v = per_tile[tile];
        if (v.empty()) { bad = "a tile is never visited"; break; }
        const int want = v[0].nseg;
        if (static_cast<int>(v.size()) != want) { bad = "segment count differs from nseg"; break; }
        if (want > p.sk_max_seg) { bad = "more segments than reserved slots"; break; }
        std::vector<char> have(want, 0);
        for (const wir::TileCoord& t : v) {
          if (t.nseg != want) { bad = "CTAs disagree on nseg"; break; }
          if (t.split < 0 || t.split >= want || have[t.split]) { bad = "segment ordinals are not a permutation"; break; }
          have[t.split] = 1;
          if (t.kb_begin >= t.kb_end || t.kb_begin < 0 || t.kb_end > num_kb) { bad = "empty or out-of-range k range"; break; }
          for (int kb = t.kb_begin; kb < t.kb_end; ++kb) ++seen[static_cast<size_t>(tile) * num_kb + kb];
          const int c = t.m_blk * tiles_n + t.n_blk;
          if (coord[c] && coord[c] != tile + 1) { bad = "two tiles map to one block"; break; }
          coord[c] = tile + 1;
        }
        // ordinals must follow k order
        for (const wir::TileCoord& a : v)
          for (const wir::TileCoord& b : v)
            if (a.split < b.split && a.kb_begin >= b.kb_begin) bad = "segment ordinals do not follow k order";
      }
      if (!bad)
        for (int v : seen)
          if (v != 1) { bad = "a k-block is covered zero or several times"; break; }
    }
    std::printf("%s\n", bad ? bad : "ok");
  }
  return 0;
}
