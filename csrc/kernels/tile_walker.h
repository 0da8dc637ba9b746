// Tile enumeration of the grouped GEMM kernels, usable from host code (the native self-check walks
// it exhaustively) and from the kernels.
#pragma once

#if defined(__CUDACC__)
#define FASTB_HD __host__ __device__
#else
#define FASTB_HD
#endif

namespace fastb {
namespace gemm {

constexpr int kWalkBK = 64;  // reduction step of the kernels (BK)

struct TileCoord {
  int g, m_idx, n_idx;   // group, tile row inside the group (of the fixed dim for wgrad), tile column
  int row0;              // first row of the group in the grouped matrix
  int red_blocks;        // BK steps of the reduction
};

// Walks the tile space group by group; inside a group, in bands of kBandRows rows: all column tiles
// of a band are visited (m fastest inside the band) before the next band starts. The tiles that
// run at the same time then form a roughly square patch of the output, which minimises the
// operand bytes a wave pulls from DRAM (a wave of p x q tiles reads p A-panels and q B-panels).
// TILE_M is 128 (one CTA) or 256 (CTA pair). `locate` must be called with non-decreasing tile
// indices (each role of a CTA steps its own walker by the grid stride).
constexpr int kDefaultBandRows = 4096;
template <int TILE_M>
struct TileWalker {
  const int* off; int G, tiles_n, fixed_m, red_len; bool wgrad; int band_rows;
  int g = 0, base = 0;
  FASTB_HD bool locate(int tile, TileCoord& c) {
    while (g < G) {
      const int r0 = off[g], r1 = off[g + 1];
      const int mt = wgrad ? fixed_m : (r1 - r0) / TILE_M;
      const int cnt = mt * tiles_n;
      if (tile < base + cnt) {
        const int local = tile - base;
        const int want = (band_rows > 0 ? band_rows : kDefaultBandRows) / TILE_M;
        const int kBand = want > 1 ? want : 1;
        const int band = local / (kBand * tiles_n), rem = local % (kBand * tiles_n);
        const int m0 = band * kBand, left = mt - m0, cur = kBand < left ? kBand : left;
        c.g = g; c.n_idx = rem / cur; c.m_idx = m0 + rem % cur; c.row0 = r0;
        c.red_blocks = wgrad ? (r1 - r0) / kWalkBK : red_len / kWalkBK;
        return true;
      }
      base += cnt; ++g;
    }
    return false;
  }
};

}  // namespace gemm
}  // namespace fastb
