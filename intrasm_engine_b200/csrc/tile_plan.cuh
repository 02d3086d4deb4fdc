// Tile plan of a CSR sparsity pattern: the stored positions regrouped by tile of 128 rows x
// `tile_cols` columns (64 or 128), storage order kept inside a tile.  Pattern-only, built once
// per pattern (like the reference's row_indices) and shared by the tensor-core SDDMM (128-column
// tiles) and SpMM (64-column tiles).  Layout of the plan buffer, each part 16-byte aligned:
//   tile_ptr int32 [ntiles + 1] | dest int32 [nnz] | entry uint16 [nnz] | cells int32 [ntiles * 128]
// tile = band * tiles_per_band + column tile; tile_ptr[tile] .. tile_ptr[tile + 1] index `entry`
// ((row in band << 7) | column in tile) and `dest` (position in storage order); `cells` is
// scratch of the build.
#pragma once
#include <stddef.h>
#include <stdint.h>

namespace iex {
namespace tile_plan {

constexpr int kBandRows = 128;

struct Layout {
  size_t tile_ptr, dest, entry, cells, total;
  int ntiles, tiles_per_band;
};

inline Layout layout(int m, int n, int nnz, int tile_cols) {
  Layout L{};
  const int bands = (m + kBandRows - 1) / kBandRows;
  L.tiles_per_band = (n + tile_cols - 1) / tile_cols;
  L.ntiles = bands * L.tiles_per_band;
  auto up16 = [](size_t x) { return (x + 15) & ~static_cast<size_t>(15); };
  L.tile_ptr = 0;
  L.dest = up16(4 * (static_cast<size_t>(L.ntiles) + 1));
  L.entry = L.dest + up16(4 * static_cast<size_t>(nnz));
  L.cells = L.entry + up16(2 * static_cast<size_t>(nnz));
  L.total = L.cells + up16(4 * static_cast<size_t>(L.ntiles) * kBandRows);
  return L;
}

}  // namespace tile_plan
}  // namespace iex
