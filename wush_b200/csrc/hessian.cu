// GPTQ Hessian accumulation  H += X^T X  on the sm_100a tensor cores.
//
// X is [tokens, hidden] bf16 row-major, H is [hidden, hidden] fp32.  Products of bf16 values are
// exact in fp32.  The tensor core's fp32 accumulation truncates, which biases a long chain of
// MMAs (measured: about 1.3e-5 relative after 4096 tokens), so a TMEM accumulator only ever sums
// CHUNK = 512 tokens; the epilogue threads add the chunk results in registers with
// round-to-nearest fp32 adds and update H in global memory once per call and element.
//
// Only tiles touching the lower triangle are computed (as the reference kernel does); each
// lower element is read-modify-written once and, unless the caller wants the lower triangle
// only, mirrored into the upper triangle.
//
// Structure: persistent CTAs (one per SM) walk a static list of 128 x 256 output tiles.
//   warp 0      TMA producer: per 64-token step, 2 + 4 boxes of 64 channels x 64 tokens
//               (128-byte swizzle) for the A (= X^T rows) and B (= X^T columns) operands
//   warp 1      allocates TMEM, issues tcgen05.mma (M=128, N=256, K=16; both operands MN-major,
//               since the contraction runs over tokens, the slow dimension of X)
//   warps 2..9  epilogue: each thread owns one row and 128 columns of the tile in registers;
//               per chunk TMEM -> registers (+=), after the last chunk registers -> H (+ mirror).
//               Two 256-column TMEM accumulators alternate, so chunk c+1 is multiplied while
//               chunk c is drained, and the H update of a tile overlaps the next tile's MMAs
// All mbarrier waits are bounded; on expiry the CTA raises a flag, unwinds, frees its TMEM and
// reports through the status word.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/wush_b200.h"
#include "common.cuh"
#include "hess_tiles.cuh"
#include "sm100.cuh"

namespace wush {
namespace hess {

using namespace sm100;

constexpr int BM = 128, BN = 256;   // output tile
constexpr int STAGES = 4;
// Element-type dependent geometry.  bf16: boxes of 64 channels x 64 tokens, K = 16 per MMA (kind::f16);
// fp32 input: boxes of 32 channels x 32 tokens, K = 8 per MMA (kind::tf32 -- the tensor core uses the top
// 19 bits of each operand, which is what the reference's Triton kernel does with fp32 inputs).  Either way
// a box row is 128 bytes, a stage holds 16 KB of A and 32 KB of B and feeds 4 MMAs.
template <bool F32>
struct Elem {
  static constexpr int BYTES = F32 ? 4 : 2;
  static constexpr int BOXC = 128 / BYTES;        // channels per TMA box
  static constexpr int KT = F32 ? 32 : 64;        // tokens per pipeline stage
  static constexpr int KMMA = F32 ? 8 : 16;       // tokens per MMA
  static constexpr int KSTEP_BYTES = KMMA * 128;  // descriptor advance per MMA
  static constexpr int BOX_BYTES = 128 * KT;      // one box: BOXC channels x KT tokens
  // Shared-memory layout the MMA descriptor names.  16-bit operands: 128-byte swizzle on 16-byte units,
  // repeating every 8 tokens (1024 bytes).  MN-major 32-bit operands are transposed in 32-byte units, so
  // they use the 128-byte swizzle on 32-byte units, which repeats every 4 tokens (512 bytes).
  static constexpr uint64_t DESC_SWIZZLE = F32 ? 1 /*128B, 32-byte base*/ : 2 /*128B*/;
  static constexpr uint32_t SBO = F32 ? 512 : 1024;
};
constexpr int A_BYTES = BM * 64 * 2;          // 16 KB
constexpr int B_BYTES = BN * 64 * 2;          // 32 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr int THREADS = 320;
constexpr int CHUNK_KB = 8;                  // k-blocks summed in one TMEM accumulator: 512 (bf16) / 256 (fp32) tokens
constexpr uint32_t TMEM_COLS = 512;

struct Params {
  float* h;
  int64_t ldh;
  int hidden;
  int tokens;
  int n_tiles;
  int first_block;  // 128-row blocks [first_block, last_block) of this launch (row panels can be launched separately)
  int last_block;
  int ksplit;       // CTAs sharing the token range of one tile (> 1: results are added with atomics)
  int lower_only;   // do not mirror into the upper triangle
  int overwrite;    // H = X^T X: the previous contents are not read (ksplit == 1 only)
  int tile_off;     // CTA-pair kernel: first entry of the tile list handled by this launch
  int* status;      // optional device word, set to 1 when a bounded wait ran out
};

// tile t -> (row block bi of 128, column block bj of 256); row block bi has bi/2 + 1 column blocks.
// Tiles are ordered in bands of 16 row blocks, column block by column block inside a band, so the
// ~148 tiles in flight cover a compact rectangle of H and share their X columns through L2.
constexpr int BAND = 16;
__device__ __forceinline__ void tile_coords(int t, int first_block, int last_block, int& bi, int& bj) {
  for (int lo = first_block;; lo += BAND) {
    const int hi = min(lo + BAND, last_block);          // row blocks [lo, hi)
    for (int c = 0; c <= (hi - 1) >> 1; ++c) {          // column blocks that some row of the band reaches
      const int first = max(lo, 2 * c);                 // rows bi >= 2c own column block c
      const int cnt = hi - first;
      if (t < cnt) {
        bi = first + t;
        bj = c;
        return;
      }
      t -= cnt;
    }
    if (hi >= last_block) break;
  }
  bi = first_block;   // not reached for t < n_tiles
  bj = 0;
}

// work item w -> tile and the k-block range [kb0, kb1) of its token split.  Tile is the fast index:
// CTAs running at the same time then read the same tokens (different channels), so a block of X
// is fetched from HBM once and served to all of them from L2.
__device__ __forceinline__ void work_range(const Params& p, int w, int k_blocks, int& t, int& kb0, int& kb1) {
  const int sp = w / p.n_tiles;
  t = w - sp * p.n_tiles;
  kb0 = (int)((int64_t)sp * k_blocks / p.ksplit);
  kb1 = (int)((int64_t)(sp + 1) * k_blocks / p.ksplit);
}

// Add this thread's 128 accumulated values (row i, columns jh .. jh+127) into H.  `tile_last_row` is the
// last row of the CTA's tile: 32-column chunks that start beyond it lie above the diagonal for every row
// of the tile and are skipped uniformly.
__device__ __forceinline__ void update_h(const Params& p, float (&acc)[128], int i, int jh, int tile_last_row) {
  const bool row_ok = i < p.hidden;
  float* hrow = p.h + (int64_t)i * p.ldh;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int jc = jh + c * 32;
    if (jc > tile_last_row) continue;
    if (p.ksplit > 1) {
      // several CTAs add into the same tile: fire-and-forget vector reductions (lower-only mode)
      if (row_ok && jc + 31 <= i) {
#pragma unroll
        for (int u = 0; u < 8; ++u)
          atomicAdd(reinterpret_cast<float4*>(hrow + jc + 4 * u),
                    make_float4(acc[c * 32 + 4 * u], acc[c * 32 + 4 * u + 1], acc[c * 32 + 4 * u + 2],
                                acc[c * 32 + 4 * u + 3]));
      } else {
#pragma unroll
        for (int u = 0; u < 32; ++u)
          if (row_ok && jc + u <= i) atomicAdd(hrow + jc + u, acc[c * 32 + u]);
      }
      continue;
    }
    if (row_ok && jc + 31 <= i) {
      // chunk entirely in the lower triangle of this row (and inside the matrix)
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
        if (!p.overwrite) o = *reinterpret_cast<const float4*>(hrow + jc + 4 * u);
        o.x += acc[c * 32 + 4 * u];
        o.y += acc[c * 32 + 4 * u + 1];
        o.z += acc[c * 32 + 4 * u + 2];
        o.w += acc[c * 32 + 4 * u + 3];
        *reinterpret_cast<float4*>(hrow + jc + 4 * u) = o;
        acc[c * 32 + 4 * u] = o.x; acc[c * 32 + 4 * u + 1] = o.y;
        acc[c * 32 + 4 * u + 2] = o.z; acc[c * 32 + 4 * u + 3] = o.w;
      }
    } else {
#pragma unroll
      for (int u = 0; u < 32; ++u) {
        if (row_ok && jc + u <= i) {
          if (!p.overwrite) acc[c * 32 + u] += hrow[jc + u];
          hrow[jc + u] = acc[c * 32 + u];
        }
      }
    }
    if (!p.lower_only) {
      // mirror: element (i, j), j < i, also goes to (j, i); lanes hold consecutive i
#pragma unroll
      for (int u = 0; u < 32; ++u) {
        const int j = jc + u;
        if (row_ok && j < i) p.h[(int64_t)j * p.ldh + i] = acc[c * 32 + u];
      }
    }
  }
}

template <bool F32>
__global__ void __launch_bounds__(THREADS, 1) hessian_kernel(const __grid_constant__ CUtensorMap xmap, const Params p) {
  using E = Elem<F32>;
  constexpr int KT = E::KT, BOX_BYTES = E::BOX_BYTES;
  extern __shared__ uint8_t smem_unaligned[];
  // 1024-byte alignment: the 128-byte swizzle pattern repeats every 8 rows of 128 bytes
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  // bars[0..S): full, [S..2S): empty, [2S..2S+2): tmem_full, [2S+2..2S+4): tmem_empty
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_u32(bars);
  auto full_bar = [&](int s) { return bar_base + 8 * s; };
  auto empty_bar = [&](int s) { return bar_base + 8 * (STAGES + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8 * (2 * STAGES + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8 * (2 * STAGES + 2 + b); };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), 8);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int k_blocks = (p.tokens + KT - 1) / KT;
  const int n_work = p.n_tiles * p.ksplit;

  if (warp == 0) {
    // ------------------------------- TMA producer ---------------------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&xmap);
      int s = 0;
      uint32_t round = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x) {
        int t, kbeg, kend, bi, bj;
        work_range(p, w, k_blocks, t, kbeg, kend);
        tile_coords(t, p.first_block, p.last_block, bi, bj);
        for (int kb = kbeg; kb < kend; ++kb) {
          if (!(ok = mbar_wait(empty_bar(s), (round & 1) ^ 1, abort_flag))) break;
          mbar_arrive_expect_tx(full_bar(s), STAGE_BYTES);
          const uint32_t dst = smem_base + s * STAGE_BYTES;
#pragma unroll
          for (int a = 0; a < BM / E::BOXC; ++a)
            tma_load_2d(dst + a * BOX_BYTES, &xmap, bi * BM + E::BOXC * a, kb * KT, full_bar(s));
#pragma unroll
          for (int b = 0; b < BN / E::BOXC; ++b)
            tma_load_2d(dst + A_BYTES + b * BOX_BYTES, &xmap, bj * BN + E::BOXC * b, kb * KT, full_bar(s));
          if (++s == STAGES) { s = 0; ++round; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -----------------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(F32 ? 2 /*tf32*/ : 1 /*bf16*/, 1, 1, BM, BN);
      int s = 0;
      uint32_t round = 0, it = 0;  // it counts chunks: accumulator buffer = it & 1
      bool ok = true, ready = false;   // ready: the probe issued with the previous k-block saw this one complete
      for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x) {
        int t, kbeg, kend;
        work_range(p, w, k_blocks, t, kbeg, kend);
        for (int kb0 = kbeg; kb0 < kend && ok; kb0 += CHUNK_KB, ++it) {
          const uint32_t buf = it & 1, use = it >> 1;
          if (!(ok = mbar_wait(tempty_bar(buf), (use & 1) ^ 1, abort_flag))) break;
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + buf * BN;
          const int kb1 = min(kb0 + CHUNK_KB, kend);
          for (int kb = kb0; kb < kb1; ++kb) {
            if (!ready && !(ok = mbar_wait(full_bar(s), round & 1, abort_flag))) break;
            tc_fence_after();
            const uint32_t a0 = smem_base + s * STAGE_BYTES, b0 = a0 + A_BYTES;
            // MN-major, 128-byte swizzle: channel atoms (128 bytes wide) are BOX_BYTES apart (leading
            // offset), 8- (or 4-) token groups SBO bytes apart (stride offset); one MMA spans KMMA tokens.
            // The four MMAs of the stage go out together with a probe of the next stage's barrier.
            static_assert(KT / E::KMMA == 4, "four MMAs per stage");
            const uint64_t ad = make_smem_desc(a0, BOX_BYTES, E::SBO, E::DESC_SWIZZLE);
            const uint64_t bd = make_smem_desc(b0, BOX_BYTES, E::SBO, E::DESC_SWIZZLE);
            const int sn = (s + 1 == STAGES) ? 0 : s + 1;
            ready = umma_x4_probe<F32, false>(d_tmem, ad, bd, E::KSTEP_BYTES >> 4, idesc, kb > kb0, full_bar(sn),
                                              (sn == 0 ? round + 1 : round) & 1);
            umma_commit(empty_bar(s));  // the stage is free once these MMAs have read it
            if (++s == STAGES) { s = 0; ++round; }
          }
          if (ok) umma_commit(tfull_bar(buf));
        }
      }
    }
  } else {
    // ------------------------------- epilogue ---------------------------------------------------
    const int quarter = warp & 3;        // TMEM lanes this warp may read: 32*quarter .. +31
    const int half = (warp - 2) >> 2;    // which 128 of the tile's 256 columns
    uint32_t it = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x) {
      int t, kbeg, kend, bi, bj;
      work_range(p, w, k_blocks, t, kbeg, kend);
      tile_coords(t, p.first_block, p.last_block, bi, bj);
      float acc[128];
#pragma unroll
      for (int u = 0; u < 128; ++u) acc[u] = 0.0f;
      for (int kb0 = kbeg; kb0 < kend && ok; kb0 += CHUNK_KB, ++it) {
        const uint32_t buf = it & 1, use = it >> 1;
        if (!(ok = mbar_wait(tfull_bar(buf), use & 1, abort_flag))) break;
        tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN + half * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int u = 0; u < 32; ++u) acc[c * 32 + u] += __uint_as_float(r[u]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(buf));
      }
      if (!ok) break;

      update_h(p, acc, bi * BM + quarter * 32 + lane, bj * BN + half * 128, bi * BM + BM - 1);
    }
  }

  // ------------------------------- teardown -------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_flag && p.status) atomicExch(p.status, 1);
}


// ---------------------------------------------------------------------------------------------------
// CTA-pair variant (cta_group::2).  The 1-CTA kernel above is bound by shared-memory bandwidth: per
// MMA the tensor core reads 12 KB of operands while TMA writes another 12 KB (measured: 1430-1600
// TFLOP/s with the loads removed, 1190-1220 with them).  Two CTAs of a cluster compute a 256 x 256 tile
// together: each holds its own 128 rows of A and one half (128 columns) of B, the hardware shares the B
// halves between the two tensor cores, and the traffic per SM drops to 8 KB + 8 KB per MMA.
//   both CTAs   producer (TMA into own shared memory, completion counted on the LEADER's full barrier),
//               epilogue (own 128 rows of the accumulator)
//   leader only MMA issue; commits are multicast to the barriers of both CTAs
// No TMA multicast is used: every CTA fetches its own boxes.
// ---------------------------------------------------------------------------------------------------
constexpr int P_STAGES = 6;
constexpr int P_STAGE_BYTES = A_BYTES + B_BYTES / 2;   // 32 KB per CTA: 128 rows of A, 128 columns of B
constexpr int P_SMEM_BYTES = P_STAGES * P_STAGE_BYTES + 1024 + 256;
template <bool F32>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
hessian_pair_kernel(const __grid_constant__ CUtensorMap xmap, const Params p) {
  using E = Elem<F32>;
  constexpr int KT = E::KT, BOX_BYTES = E::BOX_BYTES;
  extern __shared__ uint8_t smem_unaligned[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + P_STAGES * P_STAGE_BYTES);
  // same layout in both CTAs: [0..S) full (leader's are used), [S..2S) empty, then tmem_full[2], tmem_empty[2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * P_STAGES + 4);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair_id = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_u32(bars);
  auto full_bar = [&](int s) { return bar_base + 8 * s; };
  auto empty_bar = [&](int s) { return bar_base + 8 * (P_STAGES + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8 * (2 * P_STAGES + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8 * (2 * P_STAGES + 2 + b); };

  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; ++s) {
      mbar_init(full_bar(s), 1);    // the leader's expect_tx arrival; bytes of both CTAs
      mbar_init(empty_bar(s), 1);   // multicast commit
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);   // multicast commit
      mbar_init(tempty_bar(b), 16); // 8 epilogue warps of each CTA (leader's barrier is the one waited on)
    }
    *abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // barriers of both CTAs are initialised before anything is signalled remotely
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int k_blocks = (p.tokens + KT - 1) / KT;
  const int n_work = p.n_tiles * p.ksplit;

  if (warp == 0) {
    // ------------------------------- TMA producer (both CTAs) ---------------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&xmap);
      int s = 0;
      uint32_t round = 0;
      bool ok = true;
      for (int w = pair_id; w < n_work && ok; w += n_pairs) {
        int t, kbeg, kend, bi, bj;
        work_range(p, w, k_blocks, t, kbeg, kend);
        pair_tile_coords(t + p.tile_off, p.first_block, p.last_block, bi, bj);
        const int a_col = bi * 256 + (int)rank * 128, b_col = bj * 256 + (int)rank * 128;
        for (int kb = kbeg; kb < kend; ++kb) {
          if (!(ok = mbar_wait(empty_bar(s), (round & 1) ^ 1, abort_flag))) break;
          if (leader) mbar_arrive_expect_tx(full_bar(s), 2 * P_STAGE_BYTES);
          const uint32_t full_leader = map_to_cta(full_bar(s), 0);
          const uint32_t dst = smem_base + s * P_STAGE_BYTES;
#pragma unroll
          for (int a = 0; a < 128 / E::BOXC; ++a)
            tma_load_2d_pair(dst + a * BOX_BYTES, &xmap, a_col + E::BOXC * a, kb * KT, full_leader);
#pragma unroll
          for (int b = 0; b < 128 / E::BOXC; ++b)
            tma_load_2d_pair(dst + A_BYTES + b * BOX_BYTES, &xmap, b_col + E::BOXC * b, kb * KT, full_leader);
          if (++s == P_STAGES) { s = 0; ++round; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer (leader CTA only) -----------------------------------
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = make_idesc_f16(F32 ? 2 /*tf32*/ : 1 /*bf16*/, 1, 1, 256, BN);
      int s = 0;
      uint32_t round = 0, it = 0;
      bool ok = true, ready = false;
      for (int w = pair_id; w < n_work && ok; w += n_pairs) {
        int t, kbeg, kend;
        work_range(p, w, k_blocks, t, kbeg, kend);
        for (int kb0 = kbeg; kb0 < kend && ok; kb0 += CHUNK_KB, ++it) {
          const uint32_t buf = it & 1, use = it >> 1;
          if (!(ok = mbar_wait(tempty_bar(buf), (use & 1) ^ 1, abort_flag))) break;
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + buf * BN;
          const int kb1 = min(kb0 + CHUNK_KB, kend);
          for (int kb = kb0; kb < kb1; ++kb) {
            if (!ready && !(ok = mbar_wait(full_bar(s), round & 1, abort_flag))) break;
            tc_fence_after();
            const uint32_t a0 = smem_base + s * P_STAGE_BYTES, b0 = a0 + A_BYTES;
            const uint64_t ad = make_smem_desc(a0, BOX_BYTES, E::SBO, E::DESC_SWIZZLE);
            const uint64_t bd = make_smem_desc(b0, BOX_BYTES, E::SBO, E::DESC_SWIZZLE);
            const int sn = (s + 1 == P_STAGES) ? 0 : s + 1;
            ready = umma_x4_probe<F32, true>(d_tmem, ad, bd, E::KSTEP_BYTES >> 4, idesc, kb > kb0, full_bar(sn),
                                             (sn == 0 ? round + 1 : round) & 1);
            umma_commit_pair(empty_bar(s), 3);   // frees the stage in both CTAs
            if (++s == P_STAGES) { s = 0; ++round; }
          }
          if (ok) umma_commit_pair(tfull_bar(buf), 3);
        }
      }
    }
  } else {
    // ------------------------------- epilogue (both CTAs, own 128 rows) -----------------------------
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    uint32_t it = 0;
    bool ok = true;
    for (int w = pair_id; w < n_work && ok; w += n_pairs) {
      int t, kbeg, kend, bi, bj;
      work_range(p, w, k_blocks, t, kbeg, kend);
      pair_tile_coords(t + p.tile_off, p.first_block, p.last_block, bi, bj);
      float acc[128];
#pragma unroll
      for (int u = 0; u < 128; ++u) acc[u] = 0.0f;
      for (int kb0 = kbeg; kb0 < kend && ok; kb0 += CHUNK_KB, ++it) {
        const uint32_t buf = it & 1, use = it >> 1;
        if (!(ok = mbar_wait(tfull_bar(buf), use & 1, abort_flag))) break;
        tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN + half * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int u = 0; u < 32; ++u) acc[c * 32 + u] += __uint_as_float(r[u]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          // the accumulator reads are complete (tcgen05.wait::ld) and nothing travels through memory, so the
          // peer's arrival needs no release fence (which costs ~1600 cycles with TMA traffic in flight)
          if (leader) mbar_arrive(tempty_bar(buf));
          else mbar_arrive_cluster_relaxed(map_to_cta(tempty_bar(buf), 0));
        }
      }
      if (!ok) break;
      const int row0 = bi * 256 + (int)rank * 128;
      update_h(p, acc, row0 + quarter * 32 + lane, bj * 256 + half * 128, row0 + 127);
    }
  }

  // ------------------------------- teardown -------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // neither CTA leaves (or frees TMEM) while the other may still signal it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_flag && p.status) atomicExch(p.status, 1);
}

}  // namespace hess
}  // namespace wush

using namespace wush;

// tile_begin < 0: rows [row_begin, row_end) of H; otherwise entries [tile_begin, tile_end) of the 256 x 256 tile list
static int hessian_launch_one(float* h, const void* x, int64_t tokens, int64_t hidden, int64_t row_begin,
                              int64_t row_end, int64_t tile_begin, int64_t tile_end, int flags, int* status,
                              cudaStream_t stream);

// Tokens per kernel launch.  The CTAs of a launch walk the token axis side by side and share the X
// blocks they read through L2; over very long token ranges they drift apart and that sharing is lost
// (measured at hidden 14336: 1230 TFLOP/s with 32768 tokens per launch, 800 with 262144), so long
// inputs are cut into segments.  Earlier segments only update the lower triangle; the mirror image is
// written once, by the last segment.  Only the first segment may overwrite.
constexpr int64_t kSegmentTokens = 32768;

static int hessian_launch(float* h, const void* x, int64_t tokens, int64_t hidden, int64_t row_begin, int64_t row_end,
                          int64_t tile_begin, int64_t tile_end, int flags, int* status, cudaStream_t stream) {
  if (tokens <= kSegmentTokens + kSegmentTokens / 2 || !x || hidden <= 0)
    return hessian_launch_one(h, x, tokens, hidden, row_begin, row_end, tile_begin, tile_end, flags, status, stream);
  const char* xb = static_cast<const char*>(x);
  for (int64_t t0 = 0; t0 < tokens; t0 += kSegmentTokens) {
    const int64_t n = tokens - t0 < kSegmentTokens + kSegmentTokens / 2 ? tokens - t0 : kSegmentTokens;
    const bool last = t0 + n >= tokens;
    int f = last ? flags : (flags | WUSH_HESSIAN_LOWER_ONLY);
    if (t0 > 0) f &= ~WUSH_HESSIAN_OVERWRITE;
    const int rc = hessian_launch_one(h, xb + t0 * hidden * ((flags & WUSH_HESSIAN_INPUT_F32) ? 4 : 2), n, hidden, row_begin,
                                      row_end, tile_begin, tile_end, f, status, stream);
    if (rc != 0) return rc;
    if (last) break;
  }
  return 0;
}

// CTA pairs (clusters of 2) that can be resident at once on the current device; SMs that cannot be paired
// inside their GPC stay idle.  Cached per device.
template <class Kernel>
static int resident_pairs(PerDevice& cache, Kernel pk, int threads, int smem, int units) {
  const int dev = device_slot();
  if (dev >= 0 && cache.get(dev)) return cache.get(dev);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * units);
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, pk, &cfg) != cudaSuccess || n <= 0) n = units;
  if (n > units) n = units;
  if (dev >= 0) cache.set(dev, n);
  return n;
}

static int hessian_pairs_on_device() {
  static PerDevice attr, pairs;
  auto pk = hess::hessian_pair_kernel<false>;
  if (opt_in_smem(attr, pk, hess::P_SMEM_BYTES) != 0) return 0;
  const int sms = sm_count();
  return sms < 2 ? 0 : resident_pairs(pairs, pk, hess::THREADS, hess::P_SMEM_BYTES, sms / 2);
}

static int hessian_launch_one(float* h, const void* x, int64_t tokens, int64_t hidden, int64_t row_begin,
                              int64_t row_end, int64_t tile_begin, int64_t tile_end, int flags, int* status,
                              cudaStream_t stream) {
  if (!h || !x) return WUSH_ERR_NULL_POINTER;
  if (tokens < 0 || hidden <= 0 || hidden % 8 != 0 || tokens > 0x7fffffff || hidden > (1 << 20)) return WUSH_ERR_BAD_SHAPE;
  const bool by_tiles = tile_begin >= 0;
  const int64_t nblk256 = (hidden + 255) / 256;
  if (by_tiles) {
    if (tile_end < tile_begin || tile_end > hess::pair_tile_count(nblk256)) return WUSH_ERR_BAD_SHAPE;
  } else if (row_begin < 0 || row_end > hidden || row_begin > row_end || row_begin % hess::BM != 0 ||
             (row_end % hess::BM != 0 && row_end != hidden)) {
    return WUSH_ERR_BAD_SHAPE;
  }
  if (flags & ~(WUSH_HESSIAN_LOWER_ONLY | WUSH_HESSIAN_INPUT_F32 | WUSH_HESSIAN_OVERWRITE)) return WUSH_ERR_BAD_FLAG;
  const bool f32 = (flags & WUSH_HESSIAN_INPUT_F32) != 0;
  if (((uintptr_t)h & 15) || ((uintptr_t)x & 15)) return WUSH_ERR_BAD_ALIGNMENT;
  if (tokens == 0 || (by_tiles ? tile_begin == tile_end : row_begin == row_end)) return WUSH_OK;
  int rc = require_sm100();
  if (rc != 0) return rc;

  CUtensorMap map;
  rc = f32 ? make_tensor_map_2d(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, x, (uint64_t)tokens, (uint64_t)hidden,
                                (uint64_t)hidden * 4, hess::Elem<true>::BOXC, hess::Elem<true>::KT,
                                CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)
           : make_tensor_map_2d(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, (uint64_t)tokens, (uint64_t)hidden,
                                (uint64_t)hidden * 2, hess::Elem<false>::BOXC, hess::Elem<false>::KT,
                                CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != 0) return rc;

  const int sms = sm_count();
  // CTA-pair kernel: 256 x 256 tiles, needs row panels aligned to 256 and at least one pair of SMs
  static const int use_pair = env_int("WUSH_B200_HESSIAN_PAIR", 1);
  const bool pair = by_tiles || (use_pair && row_begin % 256 == 0 && (row_end % 256 == 0 || row_end == hidden) && sms >= 2);
  if (pair && sms < 2) return WUSH_ERR_BAD_FLAG;
  const int blk = pair ? 256 : hess::BM;
  int b0, b1;
  int64_t n_tiles = 0;
  if (by_tiles) {
    b0 = 0;
    b1 = (int)nblk256;
    n_tiles = tile_end - tile_begin;
  } else {
    b0 = (int)(row_begin / blk);
    b1 = (int)((row_end + blk - 1) / blk);
    // column blocks past the matrix edge never exist: they start at or before their row block
    for (int b = b0; b < b1; ++b) n_tiles += pair ? b + 1 : (b >> 1) + 1;
  }
  const int units = pair ? sms / 2 : sms;   // CTAs (or CTA pairs) working side by side

  // Token splits: only in lower-only mode (the mirror needs final values) and not when overwriting (the
  // splits add into H with atomics).  Pick the split count that wastes the least of the last wave, keeping
  // at least 1024 tokens per split.
  int ksplit = 1;
  if ((flags & WUSH_HESSIAN_LOWER_ONLY) && !(flags & WUSH_HESSIAN_OVERWRITE)) {
    const int max_split = (int)(tokens / 1024 < 1 ? 1 : (tokens / 1024 > 16 ? 16 : tokens / 1024));
    double best = 1e30;
    for (int ks = 1; ks <= max_split; ++ks) {
      const double work = (double)n_tiles * ks, waves = (double)((int64_t)(work + units - 1) / units);
      const double cost = waves * units / work + 0.02 * ks;   // relative time, penalty per extra pass of atomics over H
      if (cost < best - 1e-9) { best = cost; ksplit = ks; }
    }
  }
  hess::Params p{h, hidden, (int)hidden, (int)tokens, (int)n_tiles, b0, b1, ksplit,
                 (flags & WUSH_HESSIAN_LOWER_ONLY) ? 1 : 0, (flags & WUSH_HESSIAN_OVERWRITE) ? 1 : 0,
                 by_tiles ? (int)tile_begin : 0, status};

  if (pair) {
    auto pk = f32 ? hess::hessian_pair_kernel<true> : hess::hessian_pair_kernel<false>;
    static PerDevice attr_pair[2], max_pairs[2];
    rc = opt_in_smem(attr_pair[f32], pk, hess::P_SMEM_BYTES);
    if (rc != 0) return rc;
    int64_t pairs = resident_pairs(max_pairs[f32], pk, hess::THREADS, hess::P_SMEM_BYTES, units);
    if (pairs > n_tiles * ksplit) pairs = n_tiles * ksplit;
    pk<<<(unsigned)(2 * pairs), hess::THREADS, hess::P_SMEM_BYTES, stream>>>(map, p);
    return (int)cudaGetLastError();
  }

  auto k1 = f32 ? hess::hessian_kernel<true> : hess::hessian_kernel<false>;
  static PerDevice attr_one[2];
  rc = opt_in_smem(attr_one[f32], k1, hess::SMEM_BYTES);
  if (rc != 0) return rc;
  int grid = sms;
  if (grid > n_tiles * ksplit) grid = (int)(n_tiles * ksplit);
  k1<<<grid, hess::THREADS, hess::SMEM_BYTES, stream>>>(map, p);
  return (int)cudaGetLastError();
}

namespace wush {
namespace hess {
// Lower triangle (already summed) -> scaled lower triangle and its mirror image, 32 x 32 tiles:
// a block reads tile (bi, bj), bj <= bi, scales it in place and writes its transpose to (bj, bi)
// through shared memory, so both the reads and the mirrored writes are coalesced.  With scale == 1
// the lower triangle is left alone (mirror only).
__global__ void finalize_kernel(float* __restrict__ h, int64_t hidden, float scale, const long long* __restrict__ count,
                                int64_t tiles_per_side) {
  __shared__ float tile[32][33];
  if (count) scale = 1.0f / (float)(*count > 0 ? *count : 1);   // token count produced on the device (all-reduce)
  const bool rescale = scale != 1.0f;
  const int64_t n_tiles = tiles_per_side * (tiles_per_side + 1) / 2;
  for (int64_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
    // t -> (bi, bj) with bj <= bi
    int64_t bi = (int64_t)((sqrt(8.0 * (double)t + 1.0) - 1.0) * 0.5);
    while (bi * (bi + 1) / 2 > t) --bi;
    while ((bi + 1) * (bi + 2) / 2 <= t) ++bi;
    const int64_t bj = t - bi * (bi + 1) / 2;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 256 threads: 8 rows per pass
#pragma unroll
    for (int r = ty; r < 32; r += 8) {
      const int64_t i = bi * 32 + r, j = bj * 32 + tx;
      float v = 0.0f;
      if (i < hidden && j < hidden && j <= i) {
        v = h[i * hidden + j] * scale;
        if (rescale) h[i * hidden + j] = v;
      }
      tile[r][tx] = v;
    }
    __syncthreads();
#pragma unroll
    for (int r = ty; r < 32; r += 8) {
      // element (j_row, i_col) of the mirrored tile = tile[tx][r]
      const int64_t jr = bj * 32 + r, ic = bi * 32 + tx;
      if (jr < hidden && ic < hidden && jr < ic) h[jr * hidden + ic] = tile[tx][r];
    }
    __syncthreads();
  }
}

}  // namespace hess
}  // namespace wush

extern "C" int wush_hessian_accumulate(float* h, const void* x, int64_t tokens, int64_t hidden, int flags, int* status,
                                       void* stream) {
  return hessian_launch(h, x, tokens, hidden, 0, hidden, -1, -1, flags, status, (cudaStream_t)stream);
}

extern "C" int wush_hessian_accumulate_rows(float* h, const void* x, int64_t tokens, int64_t hidden, int64_t row_begin,
                                            int64_t row_end, int flags, int* status, void* stream) {
  return hessian_launch(h, x, tokens, hidden, row_begin, row_end, -1, -1, flags, status, (cudaStream_t)stream);
}

extern "C" int64_t wush_hessian_tile_count(int64_t hidden) {
  return hidden <= 0 ? 0 : hess::pair_tile_count((hidden + 255) / 256);
}

extern "C" int wush_hessian_tiles_per_wave(void) { return hessian_pairs_on_device(); }

extern "C" int wush_hessian_tile_coords(int64_t hidden, int64_t tile, int* row_block, int* col_block) {
  if (!row_block || !col_block) return WUSH_ERR_NULL_POINTER;
  if (hidden <= 0 || tile < 0 || tile >= wush_hessian_tile_count(hidden)) return WUSH_ERR_BAD_SHAPE;
  hess::pair_tile_coords(tile, 0, (int)((hidden + 255) / 256), *row_block, *col_block);
  return WUSH_OK;
}

extern "C" int wush_hessian_accumulate_tiles(float* h, const void* x, int64_t tokens, int64_t hidden, int64_t tile_begin,
                                             int64_t tile_end, int flags, int* status, void* stream) {
  if (tile_begin < 0) return WUSH_ERR_BAD_SHAPE;
  return hessian_launch(h, x, tokens, hidden, 0, hidden, tile_begin, tile_end, flags, status, (cudaStream_t)stream);
}

static int hessian_finalize(float* h, int64_t hidden, float scale, const long long* count, void* stream);

extern "C" int wush_hessian_finalize(float* h, int64_t hidden, float scale, void* stream) {
  return hessian_finalize(h, hidden, scale, nullptr, stream);
}

extern "C" int wush_hessian_finalize_count(float* h, int64_t hidden, const int64_t* count, void* stream) {
  if (!count) return WUSH_ERR_NULL_POINTER;
  return hessian_finalize(h, hidden, 0.0f, reinterpret_cast<const long long*>(count), stream);
}

static int hessian_finalize(float* h, int64_t hidden, float scale, const long long* count, void* stream) {
  if (!h) return WUSH_ERR_NULL_POINTER;
  if (hidden <= 0 || hidden % 4 != 0) return WUSH_ERR_BAD_SHAPE;
  if ((uintptr_t)h & 15) return WUSH_ERR_BAD_ALIGNMENT;
  const int64_t side = (hidden + 31) / 32;
  int64_t blocks = side * (side + 1) / 2;
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  hess::finalize_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(h, hidden, scale, count, side);
  return (int)cudaGetLastError();
}
