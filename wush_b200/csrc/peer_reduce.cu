// Cross-GPU sum of the Hessian over NVLink, fused with the 1/N scaling.
//
// Every rank holds its raw lower-triangle sum in a buffer that all ranks can address (symmetric memory, one
// process per GPU).  The kernel takes a range of the 256 x 256 tile list the accumulation kernel walks
// (hess_tiles.cuh), cut into sub-tiles of 8 rows x 128 columns (a warp moves one 512-byte row segment per access:
// long contiguous bursts are what the NVLink packets carry best) that are dealt round-robin to the ranks.  For each sub-tile it
// owns, a rank sums the sub-tile over all ranks, scales by 1 / total tokens and delivers the result to the
// same place of every rank's buffer.  A sub-tile is summed by its owner alone, so all ranks end up with
// bit-identical results, and a given sub-tile of any buffer is only ever touched by its owner's kernel, so
// the exchange runs in place.  Two ways to move the data:
//   plain      peer loads from every rank's buffer (starting with the own one, then round the ring), peer
//              stores into every rank's buffer: (W-1)/W of the range in and out per rank;
//   multimem   one multimem.ld_reduce per 16 bytes (the NVSwitch adds the W copies on the way) and one
//              multimem.st (the switch replicates it): a rank pulls and pushes 1/W of the range, its links
//              carry about half of what the plain exchange needs.
// Only the lower triangle travels; every rank rebuilds the mirror image locally at HBM speed
// (wush_hessian_mirror_tiles).  The launch must be bracketed by two cross-rank barriers (the partial sums of the
// range are complete everywhere before / every rank has delivered after).  Both kernels can run the barrier that
// precedes them themselves (cross_rank_arrive_and_wait below): a separate barrier kernel costs 10-15 us, more
// than the exchange of a small range itself.  Because the kernel works
// on tile ranges, finished ranges can be combined while the accumulation kernel is still busy with later
// tiles: it is small enough (256 threads, 40 registers, 4 KB of shared memory) to be co-resident with it.
// No TMA, no cluster multicast: 16-byte loads and stores on peer or multicast addresses.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/wush_b200.h"
#include "common.cuh"
#include "hess_tiles.cuh"

namespace wush {
namespace peer {

constexpr int kMaxWorld = 16;

// In-kernel barrier across the ranks, run at the start of a kernel.  Every rank owns `kMaxWorld` 32-bit slots in
// peer-addressable memory; slot s of rank r is written only by rank s.  A use of the barrier has a number (`epoch`,
// the same on all ranks, growing by one per use): the first thread of the grid's first block stores it into its
// slot on every rank, and every block waits until all of its own rank's slots have reached it.  What the previous
// kernel of the stream wrote (locally or into peer memory) is complete when this kernel starts, so a rank's arrival
// says "my previous kernel is done".  The wait is bounded; on expiry the status word is set and the kernel goes on.
struct RankBarrier {
  uint32_t* const* slots;          // device array [world]: every rank's slot array (null: the caller synchronises)
  uint32_t epoch;
  int* status;
};

__device__ __forceinline__ void cross_rank_arrive_and_wait(const RankBarrier& b, int rank, int world) {
  if (b.slots == nullptr) return;
  if (blockIdx.x == 0 && threadIdx.x < world) {
    __threadfence_system();
    uint32_t* dst = b.slots[threadIdx.x] + rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(dst), "r"(b.epoch) : "memory");
  }
  if (threadIdx.x < world) {
    const uint32_t* mine = b.slots[rank] + threadIdx.x;
    uint32_t seen = 0;
    for (uint32_t spin = 0; spin < (1u << 22); ++spin) {      // seconds: far beyond any skew between the ranks
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(seen) : "l"(mine) : "memory");
      if ((int32_t)(seen - b.epoch) >= 0) break;
      __nanosleep(64);
    }
    if ((int32_t)(seen - b.epoch) < 0 && b.status) atomicExch(b.status, 1);
  }
  __syncthreads();
}

struct Params {
  float* const* bufs;              // device array [world]: base of every rank's H buffer
  float* mc;                       // multicast address of the same buffer (multimem variant), else null
  const long long* const* counts;  // device array [world]: every rank's local token count
  int rank, world;
  int64_t hidden;
  int nblk;                        // row blocks of 256
  int64_t tile_begin;
  int64_t n_items;                 // (tiles in range) * (sub-tiles per tile owned by this rank)
  int per_tile;                    // sub-tiles of one tile owned by this rank
  RankBarrier barrier;
};

__device__ __forceinline__ float4 multimem_ld_reduce_add(const float* mc_addr) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];\n"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st(float* mc_addr, const float4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};\n" ::"l"(mc_addr), "f"(v.x), "f"(v.y),
               "f"(v.z), "f"(v.w)
               : "memory");
}

template <bool MC>
__global__ void __launch_bounds__(256) peer_reduce_kernel(const Params p) {
  __shared__ float* s_bufs[kMaxWorld];
  __shared__ long long s_counts[kMaxWorld];
  cross_rank_arrive_and_wait(p.barrier, p.rank, p.world);
  if (threadIdx.x < p.world) {
    s_bufs[threadIdx.x] = p.bufs[(threadIdx.x + p.rank) % p.world];   // own buffer first
    s_counts[threadIdx.x] = *p.counts[threadIdx.x];                    // the peers' counts in parallel
  }
  __syncthreads();
  long long total = 0;
  for (int r = 0; r < p.world; ++r) total += s_counts[r];
  const float scale = 1.0f / (float)(total > 0 ? total : 1);
  const int row_in = threadIdx.x >> 5, c4 = (threadIdx.x & 31) * 4;   // this thread's float4 inside an 8 x 128 sub-tile

  for (int64_t k = blockIdx.x; k < p.n_items; k += gridDim.x) {
    int bi, bj;
    hess::pair_tile_coords(p.tile_begin + k / p.per_tile, 0, p.nblk, bi, bj);
    const int sub = p.rank + (int)(k % p.per_tile) * p.world;          // sub-tile (sub / 2, sub % 2): 32 row groups x 2 halves
    const int64_t row0 = (int64_t)bi * 256 + (sub >> 1) * 8, col0 = (int64_t)bj * 256 + (sub & 1) * 128;
    if (col0 > row0 + 7) continue;                                     // entirely above the diagonal: nothing there
    const int64_t i = row0 + row_in, j = col0 + c4;
    if (i >= p.hidden || j >= p.hidden) continue;                      // hidden % 4 == 0: a float4 never straddles the edge
    const int64_t off = i * p.hidden + j;
    float4 acc;
    if (MC) {
      acc = multimem_ld_reduce_add(p.mc + off);
    } else {
      // a sub-tile is summed by its owner alone, so the order is a fixed function of the sub-tile
      acc = *reinterpret_cast<const float4*>(s_bufs[0] + off);
#pragma unroll 8
      for (int r = 1; r < p.world; ++r) {
        const float4 v = *reinterpret_cast<const float4*>(s_bufs[r] + off);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
    }
    acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
    if (MC) {
      multimem_st(p.mc + off, acc);
    } else {
#pragma unroll 8
      for (int r = 0; r < p.world; ++r) *reinterpret_cast<float4*>(s_bufs[r] + off) = acc;
    }
  }
}

}  // namespace peer
}  // namespace wush

extern "C" int wush_hessian_peer_reduce(float* const* bufs, float* mc_buf, const int64_t* const* counts, int rank,
                                        int world, int64_t hidden, int64_t tile_begin, int64_t tile_end,
                                        uint32_t* const* barrier_slots, uint32_t barrier_epoch, int* status,
                                        void* stream) {
  using namespace wush;
  if (!bufs || !counts) return WUSH_ERR_NULL_POINTER;
  if (world < 1 || world > peer::kMaxWorld || rank < 0 || rank >= world) return WUSH_ERR_BAD_SHAPE;
  if (hidden <= 0 || hidden % 4 != 0) return WUSH_ERR_BAD_SHAPE;
  const int nblk = (int)((hidden + 255) / 256);
  if (tile_begin < 0 || tile_end < tile_begin || tile_end > hess::pair_tile_count(nblk)) return WUSH_ERR_BAD_SHAPE;
  if (mc_buf && ((uintptr_t)mc_buf & 15)) return WUSH_ERR_BAD_ALIGNMENT;
  peer::Params p{bufs, mc_buf, reinterpret_cast<const long long* const*>(counts), rank, world, hidden, nblk,
                 tile_begin, 0, 0, {barrier_slots, barrier_epoch, status}};
  p.per_tile = rank < 64 ? (64 - rank + world - 1) / world : 0;
  p.n_items = (tile_end - tile_begin) * p.per_tile;
  if (p.n_items <= 0 && barrier_slots == nullptr) return WUSH_OK;
  int64_t blocks = p.n_items > 0 ? p.n_items : 1;       // an empty range still takes part in the barrier
  const int64_t cap = (int64_t)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (mc_buf)
    peer::peer_reduce_kernel<true><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(p);
  else
    peer::peer_reduce_kernel<false><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(p);
  return (int)cudaGetLastError();
}

// ---- mirror image of a tile range, optionally behind the in-kernel barrier ------------------------------------
namespace wush {
namespace peer {

// A block copies 32 x 32 sub-tiles of the lower triangle to their transposed places.  Sub-tiles above the diagonal
// of a diagonal tile are skipped, diagonal sub-tiles mirror their strictly lower part.
__global__ void __launch_bounds__(256) mirror_tiles_kernel(float* __restrict__ h, int64_t hidden, int nblk, int64_t tile_begin,
                                                           int64_t n_items, int rank, int world, const RankBarrier barrier) {
  __shared__ float tile[32][33];
  cross_rank_arrive_and_wait(barrier, rank, world);
  const int row = threadIdx.x >> 3, c4 = (threadIdx.x & 7) * 4;       // this thread's 16 bytes of a 32 x 32 sub-tile
  for (int64_t k = blockIdx.x; k < n_items; k += gridDim.x) {
    int bi, bj;
    hess::pair_tile_coords(tile_begin + (k >> 6), 0, nblk, bi, bj);
    const int sub = (int)(k & 63);
    const int64_t si = (int64_t)bi * 8 + (sub >> 3), sj = (int64_t)bj * 8 + (sub & 7);   // 32 x 32 sub-tile (si, sj)
    if (sj > si) continue;                                                             // uniform per block
    const int64_t i = si * 32 + row, j = sj * 32 + c4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < hidden && j < hidden) v = *reinterpret_cast<const float4*>(h + i * hidden + j);   // hidden % 4 == 0
    tile[row][c4] = v.x; tile[row][c4 + 1] = v.y; tile[row][c4 + 2] = v.z; tile[row][c4 + 3] = v.w;
    __syncthreads();
    // row `row` of the transposed sub-tile, columns c4 .. c4 + 3: elements (sj*32 + row, si*32 + c4 + u)
    const int64_t jr = sj * 32 + row, ic = si * 32 + c4;
    if (jr < hidden && ic < hidden) {
      if (si != sj) {
        *reinterpret_cast<float4*>(h + jr * hidden + ic) = make_float4(tile[c4][row], tile[c4 + 1][row], tile[c4 + 2][row], tile[c4 + 3][row]);
      } else {
        // diagonal sub-tile: only the strictly upper part is a mirror image
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (jr < ic + u) h[jr * hidden + ic + u] = tile[c4 + u][row];
      }
    }
    __syncthreads();
  }
}

}  // namespace peer
}  // namespace wush

extern "C" int wush_hessian_mirror_tiles(float* h, int64_t hidden, int64_t tile_begin, int64_t tile_end, int rank, int world,
                                         uint32_t* const* barrier_slots, uint32_t barrier_epoch, int* status, void* stream) {
  using namespace wush;
  if (!h) return WUSH_ERR_NULL_POINTER;
  const int nblk = (int)((hidden + 255) / 256);
  if (hidden <= 0 || hidden % 4 != 0 || tile_begin < 0 || tile_end < tile_begin || tile_end > hess::pair_tile_count(nblk))
    return WUSH_ERR_BAD_SHAPE;
  if ((uintptr_t)h & 15) return WUSH_ERR_BAD_ALIGNMENT;
  if (barrier_slots && (world < 1 || world > peer::kMaxWorld || rank < 0 || rank >= world)) return WUSH_ERR_BAD_SHAPE;
  const int64_t items = (tile_end - tile_begin) * 64;
  if (items == 0 && barrier_slots == nullptr) return WUSH_OK;
  int64_t blocks = items > 0 ? items : 1;
  const int64_t cap = (int64_t)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  peer::mirror_tiles_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      h, hidden, nblk, tile_begin, items, rank, world, peer::RankBarrier{barrier_slots, barrier_epoch, status});
  return (int)cudaGetLastError();
}

// ---- one rank's slot of a symmetric buffer delivered to every rank in one launch ------------------------------
namespace wush {
namespace peer {

struct BroadcastParams {
  const uint4* src;              // this rank's data (its slot of its own buffer), 16-byte units
  uint4* mc_dst;                 // the slot's multicast address (the switch replicates every store), or null
  uint4* dst[kMaxWorld];         // else: the slot's address in every other rank's buffer
  int n_dst;
  int64_t units;
};

// With a multicast address every 16 bytes leave this GPU once (multimem.st) and the NVSwitch writes them into all
// ranks' buffers; without, the kernel stores them to each peer in turn.
__global__ void __launch_bounds__(256) peer_broadcast_kernel(const BroadcastParams p) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < p.units; i += (int64_t)gridDim.x * blockDim.x) {
    const uint4 v = p.src[i];
    if (p.mc_dst != nullptr) {
      asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};\n" ::"l"(p.mc_dst + i),
                   "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
                   "f"(__uint_as_float(v.w))
                   : "memory");
    } else {
      for (int r = 0; r < p.n_dst; ++r) p.dst[r][i] = v;
    }
  }
}

}  // namespace peer
}  // namespace wush

extern "C" int wush_peer_broadcast(const void* src, void* mc_dst, void* const* dst, int n_dst, int64_t bytes,
                                   void* stream) {
  using namespace wush;
  if (!src || (!mc_dst && n_dst > 0 && !dst)) return WUSH_ERR_NULL_POINTER;
  if (bytes < 0 || bytes % 16 != 0 || n_dst < 0 || n_dst > peer::kMaxWorld) return WUSH_ERR_BAD_SHAPE;
  if (((uintptr_t)src & 15) || ((uintptr_t)mc_dst & 15)) return WUSH_ERR_BAD_ALIGNMENT;
  if (bytes == 0 || (!mc_dst && n_dst == 0)) return WUSH_OK;
  if (const int rc = require_sm100()) return rc;
  peer::BroadcastParams p{};
  p.src = (const uint4*)src;
  p.mc_dst = (uint4*)mc_dst;
  p.n_dst = mc_dst ? 0 : n_dst;
  for (int r = 0; r < p.n_dst; ++r) {
    if (!dst[r]) return WUSH_ERR_NULL_POINTER;
    if ((uintptr_t)dst[r] & 15) return WUSH_ERR_BAD_ALIGNMENT;
    p.dst[r] = (uint4*)dst[r];
  }
  p.units = bytes / 16;
  int64_t blocks = (p.units + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 4;
  if (blocks > cap) blocks = cap;
  peer::peer_broadcast_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(p);
  return (int)cudaGetLastError();
}
