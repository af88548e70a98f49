// Cross-GPU sum of the Hessian over NVLink peer memory, fused with the 1/N scaling and the mirror.
//
// Every rank holds its raw lower-triangle sum in a buffer that all ranks can address (symmetric
// memory, one process per GPU).  The lower triangle is cut into 32 x 32 tiles dealt round-robin to the
// ranks.  For each tile it owns, a rank reads the tile from every rank's buffer with plain peer loads,
// adds them (a tile is summed by its owner alone, so all ranks end up with bit-identical results), scales by 1 / total
// tokens, and stores the finished tile and its mirror image into every rank's buffer with peer stores.
// A given tile of any buffer is only ever touched by its owner's kernel, so the exchange can run in
// place; the caller brackets the launch with two cross-rank barriers (all partial sums complete before
// / all results delivered after).  One kernel replaces an all-reduce, a scaling pass and a mirror pass;
// per rank it moves (W-1)/W of the triangle in and twice that out over NVSwitch.
// No TMA, no multicast: ordinary 16-byte loads and stores on peer pointers.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/wush_b200.h"
#include "common.cuh"

namespace wush {
namespace peer {

constexpr int kMaxWorld = 16;

struct Params {
  float* const* bufs;            // device array [world]: base of every rank's H buffer
  const long long* const* counts;  // device array [world]: every rank's local token count
  int rank, world;
  int64_t hidden;
  int64_t tiles_per_side;
};

__global__ void __launch_bounds__(256) peer_reduce_kernel(const Params p) {
  __shared__ float tile[32][33];
  __shared__ float* s_bufs[kMaxWorld];
  __shared__ float s_scale;
  if (threadIdx.x < p.world) s_bufs[threadIdx.x] = p.bufs[threadIdx.x];
  if (threadIdx.x == 0) {
    long long total = 0;
    for (int r = 0; r < p.world; ++r) total += *p.counts[r];
    s_scale = 1.0f / (float)(total > 0 ? total : 1);
  }
  __syncthreads();
  const float scale = s_scale;
  const int64_t n_tiles = p.tiles_per_side * (p.tiles_per_side + 1) / 2;
  const int row_in = threadIdx.x >> 3, c4 = (threadIdx.x & 7) * 4;   // this thread's float4 inside a tile
  const bool vec_ok = (p.hidden & 3) == 0;
  (void)vec_ok;

  // tiles owned by this rank: t = rank, rank + world, ...; the CTAs of the grid share them
  for (int64_t k = blockIdx.x;; k += gridDim.x) {
    const int64_t t = (int64_t)p.rank + k * p.world;
    if (t >= n_tiles) break;
    int64_t bi = (int64_t)((sqrt(8.0 * (double)t + 1.0) - 1.0) * 0.5);
    while (bi * (bi + 1) / 2 > t) --bi;
    while ((bi + 1) * (bi + 2) / 2 <= t) ++bi;
    const int64_t bj = t - bi * (bi + 1) / 2;
    const int64_t i = bi * 32 + row_in, j = bj * 32 + c4;

    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    const bool in = i < p.hidden && j < p.hidden;     // hidden % 4 == 0: a float4 never straddles the edge
    if (in) {
      const int64_t off = i * p.hidden + j;
      // start with the own buffer and walk the ring, so that the ranks do not all read from the same GPU at
      // once; a tile is summed by its owner alone, so the order is a fixed function of the tile
#pragma unroll 8
      for (int r = 0; r < p.world; ++r) {
        const float4 v = *reinterpret_cast<const float4*>(s_bufs[(r + p.rank) % p.world] + off);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
    }
    // entries above the diagonal of a diagonal tile are not part of the sums: take them from the mirror
    tile[row_in][c4] = acc.x; tile[row_in][c4 + 1] = acc.y; tile[row_in][c4 + 2] = acc.z; tile[row_in][c4 + 3] = acc.w;
    __syncthreads();
    if (bi == bj) {
      float* e = &acc.x;
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (c4 + u > row_in) e[u] = tile[c4 + u][row_in];
    }
    // transposed element block for the mirror tile: row (bj*32 + row_in), columns (bi*32 + c4 ..)
    float4 tr;
    if (bi == bj) {
      tr = acc;   // the diagonal tile is its own mirror once completed
    } else {
      tr = make_float4(tile[c4][row_in], tile[c4 + 1][row_in], tile[c4 + 2][row_in], tile[c4 + 3][row_in]);
    }
    const int64_t mi = bj * 32 + row_in, mj = bi * 32 + c4;
    const bool min_ok = mi < p.hidden && mj < p.hidden;
#pragma unroll 4
    for (int r = 0; r < p.world; ++r) {
      float* dst = s_bufs[(r + p.rank) % p.world];    // start with the own buffer, spread the peers
      if (in) *reinterpret_cast<float4*>(dst + i * p.hidden + j) = acc;
      if (bi != bj && min_ok) *reinterpret_cast<float4*>(dst + mi * p.hidden + mj) = tr;
    }
    __syncthreads();
  }
}

}  // namespace peer
}  // namespace wush

extern "C" int wush_hessian_peer_reduce(float* const* bufs, const int64_t* const* counts, int rank, int world,
                                        int64_t hidden, void* stream) {
  using namespace wush;
  if (!bufs || !counts) return WUSH_ERR_NULL_POINTER;
  if (world < 1 || world > peer::kMaxWorld || rank < 0 || rank >= world) return WUSH_ERR_BAD_SHAPE;
  if (hidden <= 0 || hidden % 4 != 0) return WUSH_ERR_BAD_SHAPE;
  peer::Params p{bufs, reinterpret_cast<const long long* const*>(counts), rank, world, hidden, (hidden + 31) / 32};
  const int64_t n_tiles = p.tiles_per_side * (p.tiles_per_side + 1) / 2;
  int64_t mine = (n_tiles - rank + world - 1) / world;
  if (mine <= 0) return WUSH_OK;
  int64_t blocks = mine;
  const int64_t cap = (int64_t)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  peer::peer_reduce_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(p);
  return (int)cudaGetLastError();
}
