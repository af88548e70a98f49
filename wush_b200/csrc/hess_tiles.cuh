// Order of the 256 x 256 lower-triangle tiles of the Hessian, shared by the accumulation kernel (which walks
// the tiles in this order), the cross-GPU reduce and the mirror kernel (which take ranges of the same list).
#pragma once
#include <stdint.h>

namespace wush {
namespace hess {

constexpr int P_BAND = 8;   // row blocks (of 256) per band of the tile order

// Number of tiles of a matrix with `nblk` row blocks of 256: row block b owns column blocks 0..b.
__host__ __device__ inline int64_t pair_tile_count(int64_t nblk) { return nblk * (nblk + 1) / 2; }

// Tile t -> (row block bi, column block bj <= bi), both in units of 256.  The tiles of row blocks
// [first_block, last_block) are ordered in bands of P_BAND row blocks, column block by column block inside a
// band, so the ~74 tiles in flight cover a compact rectangle of H and share their X columns through L2.
// With first_block == 0 the position is computed directly; otherwise by walking the bands.
__host__ __device__ inline void pair_tile_coords(int64_t t, int first_block, int last_block, int& bi, int& bj) {
  for (int lo = first_block; lo < last_block; lo += P_BAND) {
    const int hi = lo + P_BAND < last_block ? lo + P_BAND : last_block;   // row blocks [lo, hi)
    const int h = hi - lo;
    // columns 0..lo are reached by all h row blocks of the band, column c > lo by the hi - c blocks below it
    const int64_t full = (int64_t)(lo + 1) * h;
    const int64_t band_tiles = full + (int64_t)h * (h - 1) / 2;
    if (t < band_tiles) {
      if (t < full) {
        bj = (int)(t / h);
        bi = lo + (int)(t % h);
        return;
      }
      t -= full;
      for (int c = lo + 1; c < hi; ++c) {
        const int cnt = hi - c;
        if (t < cnt) {
          bi = c + (int)t;
          bj = c;
          return;
        }
        t -= cnt;
      }
    }
    t -= band_tiles;
  }
  bi = first_block;   // not reached for t inside the list
  bj = 0;
}

}  // namespace hess
}  // namespace wush
