// Block-scaled FP4 GEMM  Y[M,N] (bf16) = alpha * (A . sfa) (B . sfb)^T  for sm_100a.
//
// A is [M, K/2] and B is [N, K/2] packed E2M1 (two codes per byte, K contiguous: "TN");
// the per-group scales arrive in the 128x4 blocked layout: E8M0 per 32 elements (MXFP4) or
// E4M3 per 16 elements (NVFP4).  The products run on tcgen05.mma kind::mxf4 /
// kind::mxf4nvf4 with block scaling: 128 x 256 output tile per CTA, K = 64 per instruction,
// fp32 accumulation in TMEM.  Scale tiles travel global -> shared memory with the operands (bulk
// copies on the same mbarrier) and shared memory -> registers -> TMEM through four feeder warps
// (tcgen05.st).  tcgen05.cp copies issued between the MMAs were measured to cost a quarter of the
// run time -- they execute in the MMA pipe -- and feeding from global memory directly made the
// feeders latency-bound.
//
// Persistent CTAs, one per SM:
//   warp 0      producer: per 256-element k-block one TMA box each for A (128 rows x 128 B) and
//               B (256 rows x 128 B), 128-byte swizzle, plus bulk copies of the scale tiles
//   warp 1      allocates TMEM; per k-block issues 4 MMAs
//   warps 10..13 scale feeders, one per TMEM lane quarter: shared memory -> registers -> TMEM
//   warps 2..9  epilogue: each thread drains one row x 128 columns of the accumulator, scaling and
//               packing to bf16 as it goes (64 registers), releases TMEM (the next tile's MMAs
//               start) and only then stores.  When the K range is split across CTAs it writes fp32
//               partial tiles instead and a second kernel reduces them
// TMEM columns: [0,256) accumulator; from 256 on, one 48-column scale region per pipeline stage
// (16 for A, 32 for B), so the feeders can run ahead of the MMAs.
// All mbarrier waits are bounded (see sm100.cuh).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "../../include/wush_b200.h"
#include "common.cuh"
#include "fp4_gemv.cuh"
#include "sm100.cuh"

namespace wush {
namespace gemm {

using namespace sm100;

constexpr int BM = 128, BN = 256, BK = 256;   // BK in elements = 128 bytes per row
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK / 2;          // 16 KB
constexpr int B_BYTES = BN * BK / 2;          // 32 KB
constexpr int SFA_BYTES = 2048;               // up to 4 atoms of 512 B (NVFP4); MXFP4 uses 2
constexpr int SFB_BYTES = 4096;               // two 128-row blocks
constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 512;
constexpr int THREADS = 480;                  // 15 warps: producer, MMA, 8 epilogue, 4 scale feeders, scale producer
constexpr int EPI_WARP0 = 2, SF_WARP0 = 10, SFP_WARP = 14;
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t SF_COL0 = 256, SF_STAGE_COLS = 48, SFB_OFF = 16;

constexpr int MAX_PEERS = 8;
// Split K inside a thread-block cluster: the CTAs of a cluster share one output tile, each taking a slice of K;
// their fp32 partial tiles meet in shared memory (see splitk_cluster_finish).
constexpr int MAX_CLUSTER_SPLITS = 8;          // portable cluster size
constexpr int CL_ROW_FLOATS = BN + 4;          // padded row of the staged partial tile

struct Params {
  const uint8_t* sfa;   // blocked scales of A: ceil(M/128) row blocks x sf_atoms_k atoms of 512 B
  const uint8_t* sfb;
  const float* alpha;   // device scalar
  __nv_bfloat16* y;     // [M, N] (row stride ldy); with column-sharded weights: this GPU's copy of the full output
  // Column-sharded weights: the tile is also stored into the same place of the other GPUs' output buffers
  // (peer-addressable memory, plain stores over NVLink), which is the all-gather of the output columns.
  __nv_bfloat16* y_peer[MAX_PEERS];
  int n_peers;          // entries of y_peer (0: single GPU)
  int64_t ldy;          // row stride of the output buffers in elements (N, or the unsharded N)
  int64_t ycol0;        // first output column of this GPU's shard inside them
  float* partial;       // [splits, M, N] when splits > 1
  int cluster_splits;   // splits > 1: 1 = the CTAs of a cluster reduce through shared memory, 0 = fp32 partial tiles
                        // in global memory and a second kernel
  // optional epilogue terms, applied in the reference's order with its roundings (linear_fns.py:514-525):
  // y = bf16(alpha * acc); y = bf16(y + bias[col]); y = bf16(y + residual[row, col])
  const __nv_bfloat16* bias;       // [N] or null
  const __nv_bfloat16* residual;   // [M, ldr] or null (may alias y)
  int64_t ldr;
  int m, n, k;
  int m_blocks, n_blocks, k_blocks;   // k_blocks of BK elements (the last may be half)
  int splits;           // CTAs sharing the K range of one tile
  int sf_atoms_k;       // 512-byte atoms per 128-row block = ceil(K/group/4)
  // A given as K shards stacked one after the other (each [a_shard_rows, K/shards/2] codes with its own blocked
  // scale tensor): the layout in which column shards quantized on different GPUs arrive.  a_kbs = 0: plain A.
  int a_kbs;            // k-blocks per shard
  int a_shard_rows;     // rows of the tensor map between two shards
  int a_sf_atoms;       // 512-byte scale atoms per 128-row block inside one shard
  int64_t a_sf_shard_bytes;   // bytes between the scale tensors of two shards
  int sfb_row_blocks;   // 128-row blocks present in sfb
  int* status;
};

__device__ __forceinline__ void bulk_load(uint32_t smem_dst, const void* gsrc, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
      ::"r"(smem_dst), "l"(gsrc), "r"(bytes), "r"(bar)
      : "memory");
}

// registers -> TMEM: 32 lanes (this warp's quarter) x N consecutive 32-bit columns
__device__ __forceinline__ void tmem_st_x8(uint32_t taddr, const uint4& a, const uint4& b) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};\n"
               ::"r"(taddr), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w)
               : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

template <bool NV>
__device__ __forceinline__ void umma_fp4_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                              uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  if (NV) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
  } else {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::mxf4.block_scale.block32 [%0], %1, %2, %3, [%5], [%6], p;\n}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
  }
}

template <bool NV>
__device__ __forceinline__ void umma_fp4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  if (NV) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
  } else {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.block32 [%0], %1, %2, %3, [%5], [%6], p;\n}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
  }
}

// The four MMAs of a full k-block in one instruction sequence, preceded by non-blocking tests of the two
// barriers the NEXT k-block depends on (operands landed, scales in tensor memory).  A barrier test costs the
// issuing thread ~200 cycles even when the phase is complete, and the MMA queue is shallow: with the tests
// between two k-blocks the tensor pipe ran dry for that long in every k-block.  Placed here their latency
// overlaps the issue of the MMAs; only the results are consumed afterwards.  Returns whether both probed
// phases are complete.
template <bool NV, bool PAIR>
__device__ __forceinline__ bool umma_fp4_x4_probe(uint32_t d_tmem, uint64_t ad, uint64_t bd, uint32_t idesc_even,
                                                  uint32_t idesc_odd, uint32_t sfa_col, uint32_t sfb_col,
                                                  uint32_t accumulate, uint32_t probe_bar, uint32_t probe_bar2,
                                                  uint32_t probe_parity) {
  // k-step ks: operands advance 32 bytes (2 descriptor units); MXFP4 uses scale bytes (ks & 1) * 2 of atom
  // ks >> 1, NVFP4 all four bytes of atom ks
  const uint32_t a1 = NV ? 1 : 0, a2 = NV ? 2 : 1, a3 = NV ? 3 : 1;
  uint32_t ready;
#define WUSH_MMA4(GROUP, KIND)                                                                                     \
  asm volatile(                                                                                                    \
      "{\n.reg .pred p, q, q2, t;\n"                                                                               \
      "mbarrier.test_wait.parity.shared::cta.b64 q, [%21], %22;\n"                                                 \
      "mbarrier.test_wait.parity.shared::cta.b64 q2, [%23], %22;\n"                                                \
      "setp.ne.b32 p, %20, 0;\n"                                                                                   \
      "setp.eq.b32 t, 0, 0;\n"                                                                                     \
      "tcgen05.mma.cta_group::" GROUP ".kind::" KIND " [%1], %2, %6, %10, [%12], [%16], p;\n"                      \
      "tcgen05.mma.cta_group::" GROUP ".kind::" KIND " [%1], %3, %7, %11, [%13], [%17], t;\n"                      \
      "tcgen05.mma.cta_group::" GROUP ".kind::" KIND " [%1], %4, %8, %10, [%14], [%18], t;\n"                      \
      "tcgen05.mma.cta_group::" GROUP ".kind::" KIND " [%1], %5, %9, %11, [%15], [%19], t;\n"                      \
      "and.pred q, q, q2;\n"                                                                                       \
      "selp.u32 %0, 1, 0, q;\n}\n"                                                                                 \
      : "=r"(ready)                                                                                                \
      : "r"(d_tmem), "l"(ad), "l"(ad + 2), "l"(ad + 4), "l"(ad + 6), "l"(bd), "l"(bd + 2), "l"(bd + 4),            \
        "l"(bd + 6), "r"(idesc_even), "r"(idesc_odd), "r"(sfa_col), "r"(sfa_col + 4 * a1), "r"(sfa_col + 4 * a2),  \
        "r"(sfa_col + 4 * a3), "r"(sfb_col), "r"(sfb_col + 8 * a1), "r"(sfb_col + 8 * a2), "r"(sfb_col + 8 * a3),  \
        "r"(accumulate), "r"(probe_bar), "r"(probe_parity), "r"(probe_bar2)                                        \
      : "memory")
  if (NV) {
    if (PAIR) WUSH_MMA4("2", "mxf4nvf4.block_scale.block16");
    else WUSH_MMA4("1", "mxf4nvf4.block_scale.block16");
  } else {
    if (PAIR) WUSH_MMA4("2", "mxf4.block_scale.block32");
    else WUSH_MMA4("1", "mxf4.block_scale.block32");
  }
#undef WUSH_MMA4
  return ready != 0;
}

// Block-scaled instruction descriptor: E2M1 operands (format 1), both K-major, scale format
// E8M0 (1) or E4M3 (0), K = 64, scale-factor byte offsets (0..3) inside the TMEM columns.
__device__ __forceinline__ uint32_t make_idesc_fp4(bool nv, uint32_t sf_id, uint32_t m = BM) {
  return (sf_id << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((nv ? 0u : 1u) << 23) |
         ((m >> 4) << 24) | (sf_id << 29);
}

// Where k-block kb of the A rows starting at `row` lives: tensor-map coordinates and scale-atom address.
__device__ __forceinline__ void a_coords(const Params& p, int kb, int row, int& x, int& y) {
  if (p.a_kbs == 0) {
    x = kb * (BK / 2);
    y = row;
  } else {
    const int sh = kb / p.a_kbs;
    x = (kb - sh * p.a_kbs) * (BK / 2);
    y = sh * p.a_shard_rows + row;
  }
}
__device__ __forceinline__ const uint8_t* a_scale_atoms(const Params& p, int kb, int row_block, int atoms_per_kb) {
  if (p.a_kbs == 0) return p.sfa + ((int64_t)row_block * p.sf_atoms_k + kb * atoms_per_kb) * 512;
  const int sh = kb / p.a_kbs;
  return p.sfa + sh * p.a_sf_shard_bytes + ((int64_t)row_block * p.a_sf_atoms + (kb - sh * p.a_kbs) * atoms_per_kb) * 512;
}

// work item -> (m block, n block, split); m fastest so neighbouring CTAs share a weight panel
__device__ __forceinline__ void work_coords(const Params& p, int w, int& mb, int& nb, int& sp) {
  sp = w % p.splits;
  const int tile = w / p.splits;
  mb = tile % p.m_blocks;
  nb = tile / p.m_blocks;
}

__device__ __forceinline__ void split_range(const Params& p, int sp, int& kb0, int& kb1) {
  kb0 = (int)((int64_t)sp * p.k_blocks / p.splits);
  kb1 = (int)((int64_t)(sp + 1) * p.k_blocks / p.splits);
}

// 8 x 8 transposition of 16-byte chunks inside every group of 8 lanes: three butterfly stages that swap bit b
// of the lane index with bit b of the chunk index.  Chunk slot 8h+i of lane (g, j) ends up holding chunk 8h+j
// of lane (g, i), so that the 8 lanes of a group own one whole 128-byte line per slot.
__device__ __forceinline__ void transpose_chunks_8x8(uint32_t (&v)[64], int lane) {
#pragma unroll
  for (int b = 0; b < 3; ++b) {
    const int m = 1 << b;
    const bool upper = (lane & m) != 0;
#pragma unroll
    for (int c = 0; c < 16; ++c) {
      if (c & m) continue;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        uint32_t& lo = v[4 * c + w];
        uint32_t& hi = v[4 * (c | m) + w];
        const uint32_t recv = __shfl_xor_sync(0xffffffffu, upper ? lo : hi, m);
        if (upper) lo = recv; else hi = recv;
      }
    }
  }
}

// 8 packed bf16 values += 8 packed bf16 values, each sum rounded to bf16 (what `y += bias` does on bf16 tensors)
__device__ __forceinline__ uint4 add_bf16x8(const uint4& a, const uint4& b) {
  uint4 o;
  const uint32_t* pa = &a.x;
  const uint32_t* pb = &b.x;
  uint32_t* po = &o.x;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 fa = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pa[i]));
    const float2 fb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pb[i]));
    const __nv_bfloat162 r = __floats2bfloat162_rn(fa.x + fb.x, fa.y + fb.y);
    po[i] = *reinterpret_cast<const uint32_t*>(&r);
  }
  return o;
}

// Epilogue of one warp: every lane drains its row x 128 accumulator columns as packed bf16 (scaled by alpha)
// and the accumulator is released through `release` (after a warp sync).  A lane-per-row store would touch 32
// different lines per instruction (4096 L1 wavefronts per tile, which was measured to stall the scale feeders
// and the next tile's first loads behind it), so the chunks are transposed among groups of 8 lanes first:
// every store instruction then writes 4 rows x 128 contiguous bytes.  `row0` is the row of lane 0.
template <class Release>
__device__ __forceinline__ void drain_and_store(const Params& p, uint32_t taddr, float alpha, int row0, int col0,
                                                int lane, Release release) {
  uint32_t packed[64];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint32_t r[32];
    tmem_ld_32x32(taddr + c * 32, r);
    tmem_ld_wait();
#pragma unroll
    for (int v = 0; v < 16; ++v) {
      const __nv_bfloat162 h =
          __floats2bfloat162_rn(__uint_as_float(r[2 * v]) * alpha, __uint_as_float(r[2 * v + 1]) * alpha);
      packed[c * 16 + v] = *reinterpret_cast<const uint32_t*>(&h);
    }
  }
  tc_fence_before();
  __syncwarp();
  release();
  transpose_chunks_8x8(packed, lane);
  const int j = lane & 7, rbase = row0 + (lane & ~7);
  // bias and residual are added to the bf16 values after the transposition: their loads are then whole lines too
  if (p.bias != nullptr || p.residual != nullptr) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int col = col0 + (8 * h + j) * 8;
      if (col >= p.n) continue;
      uint4 bv = make_uint4(0, 0, 0, 0);
      if (p.bias != nullptr) bv = *reinterpret_cast<const uint4*>(p.bias + col);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int row = rbase + i, slot = 8 * h + i;
        if (row >= p.m) continue;
        uint4 v = make_uint4(packed[4 * slot], packed[4 * slot + 1], packed[4 * slot + 2], packed[4 * slot + 3]);
        if (p.bias != nullptr) v = add_bf16x8(v, bv);
        if (p.residual != nullptr)
          v = add_bf16x8(v, *reinterpret_cast<const uint4*>(p.residual + (int64_t)row * p.ldr + col));
        packed[4 * slot] = v.x; packed[4 * slot + 1] = v.y; packed[4 * slot + 2] = v.z; packed[4 * slot + 3] = v.w;
      }
    }
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int col = col0 + (8 * h + j) * 8;          // n % 8 == 0: a chunk never straddles the edge
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int row = rbase + i, slot = 8 * h + i;
      if (row < p.m && col < p.n)
        *reinterpret_cast<uint4*>(p.y + (int64_t)row * p.ldy + p.ycol0 + col) =
            make_uint4(packed[4 * slot], packed[4 * slot + 1], packed[4 * slot + 2], packed[4 * slot + 3]);
    }
  }
  // the same lines to every other GPU's buffer: whole 128-byte lines, so the NVLink packets are full
  const int first = p.n_peers > 0 ? (int)((blockIdx.x + (threadIdx.x >> 5)) % p.n_peers) : 0;   // spread the warps over the peers
  for (int pi = 0; pi < p.n_peers; ++pi) {
    __nv_bfloat16* yp = p.y_peer[(first + pi) % p.n_peers];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int col = col0 + (8 * h + j) * 8;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int row = rbase + i, slot = 8 * h + i;
        if (row < p.m && col < p.n)
          *reinterpret_cast<uint4*>(yp + (int64_t)row * p.ldy + p.ycol0 + col) =
              make_uint4(packed[4 * slot], packed[4 * slot + 1], packed[4 * slot + 2], packed[4 * slot + 3]);
      }
    }
  }
}

// bf16(alpha * acc) (+ bias) (+ residual) for 4 consecutive columns, with the roundings of the separate steps.
__device__ __forceinline__ uint2 finish_f4(const Params& p, float4 acc, float alpha, int row, int col) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x * alpha, acc.y * alpha);
  __nv_bfloat162 hi = __floats2bfloat162_rn(acc.z * alpha, acc.w * alpha);
  if (p.bias != nullptr) {
    const uint2 bv = *reinterpret_cast<const uint2*>(p.bias + col);
    const float2 b01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&bv.x));
    const float2 b23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&bv.y));
    const float2 l = __bfloat1622float2(lo), h = __bfloat1622float2(hi);
    lo = __floats2bfloat162_rn(l.x + b01.x, l.y + b01.y);
    hi = __floats2bfloat162_rn(h.x + b23.x, h.y + b23.y);
  }
  if (p.residual != nullptr) {
    const uint2 rv = *reinterpret_cast<const uint2*>(p.residual + (int64_t)row * p.ldr + col);
    const float2 r01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&rv.x));
    const float2 r23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&rv.y));
    const float2 l = __bfloat1622float2(lo), h = __bfloat1622float2(hi);
    lo = __floats2bfloat162_rn(l.x + r01.x, l.y + r01.y);
    hi = __floats2bfloat162_rn(h.x + r23.x, h.y + r23.y);
  }
  uint2 o;
  o.x = *reinterpret_cast<const uint32_t*>(&lo);
  o.y = *reinterpret_cast<const uint32_t*>(&hi);
  return o;
}

__device__ __forceinline__ float4 ld_dsmem_f4(uint32_t cluster_addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];\n"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(cluster_addr)
               : "memory");
  return v;
}

// Split K inside a cluster, second half: every CTA of the cluster has staged the valid rows of its fp32 partial
// tile in its own shared memory (row stride CL_ROW_FLOATS) and the cluster has synchronised.  CTA `rank` of the
// `splits` CTAs finishes the column slice [rank, rank + 1) * BN / splits of the tile: it adds the partials of all
// CTAs in rank order through distributed shared memory and writes the bf16 output.  Called by the 256 epilogue threads.
__device__ __forceinline__ void splitk_cluster_finish(const Params& p, uint32_t stage_smem, int rank, int splits,
                                                      int row0, int col0, float alpha, int tid) {
  const int rows = min(BM, p.m - row0);
  const int slice = BN / splits;                 // columns per CTA: 32 .. 128, a multiple of 4
  const int f4_per_row = slice / 4;
  const int items = rows * f4_per_row;
  for (int it = tid; it < items; it += 256) {
    const int r = it / f4_per_row, c = rank * slice + (it % f4_per_row) * 4;
    if (col0 + c >= p.n) continue;               // n % 8 == 0: groups of 4 never straddle the edge
    const uint32_t off = stage_smem + (uint32_t)(r * CL_ROW_FLOATS + c) * 4u;
    float4 v[MAX_CLUSTER_SPLITS];
#pragma unroll
    for (int s = 0; s < MAX_CLUSTER_SPLITS; ++s)       // all loads in flight before the first add
      if (s < splits) v[s] = ld_dsmem_f4(map_to_cta(off, (uint32_t)s));
    float4 acc = v[0];
#pragma unroll
    for (int s = 1; s < MAX_CLUSTER_SPLITS; ++s)
      if (s < splits) { acc.x += v[s].x; acc.y += v[s].y; acc.z += v[s].z; acc.w += v[s].w; }
    *reinterpret_cast<uint2*>(p.y + (int64_t)(row0 + r) * p.ldy + p.ycol0 + col0 + c) =
        finish_f4(p, acc, alpha, row0 + r, col0 + c);
  }
}

// CLUSTER: launched as clusters of p.splits CTAs with exactly one work item per CTA (grid = tiles * splits); the
// CTAs of a cluster reduce their partial tiles through distributed shared memory.
template <bool NV, bool CLUSTER>
__global__ void __launch_bounds__(THREADS, 1)
fp4_gemm_kernel(const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap bmap, const Params p) {
  constexpr int GROUP = NV ? 16 : 32;
  constexpr int ATOMS = BK / GROUP / 4;            // scale atoms (128 rows x 4 scales) per k-block: 2 or 4
  extern __shared__ uint8_t smem_unaligned[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  // bars[0..S): full (operands), [S..2S): empty, [2S]: tmem_full, [2S+1]: tmem_empty, [2S+2..3S+2): scales
  // in TMEM, [3S+2..4S+2): sffull (scale tiles in shared memory)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4 * STAGES + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_u32(bars);
  auto full_bar = [&](int s) { return bar_base + 8 * s; };
  auto empty_bar = [&](int s) { return bar_base + 8 * (STAGES + s); };
  const uint32_t tfull_bar = bar_base + 8 * (2 * STAGES), tempty_bar = bar_base + 8 * (2 * STAGES + 1);
  auto sf_bar = [&](int s) { return bar_base + 8 * (2 * STAGES + 2 + s); };
  auto sffull_bar = [&](int s) { return bar_base + 8 * (3 * STAGES + 2 + s); };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
      mbar_init(sffull_bar(s), 1);
      mbar_init(sf_bar(s), 4);   // one arrival per feeder warp
    }
    mbar_init(tfull_bar, 1);
    mbar_init(tempty_bar, 8);
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
  const int n_work = p.m_blocks * p.n_blocks * p.splits;

  if (warp == 0) {
    // ------------------------------- producer -------------------------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&amap);
      tma_prefetch_desc(&bmap);
      int s = 0;
      uint32_t round = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x) {
        int mb, nb, sp, kb0, kb1;
        work_coords(p, w, mb, nb, sp);
        split_range(p, sp, kb0, kb1);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!(ok = mbar_wait(empty_bar(s), (round & 1) ^ 1, abort_flag))) break;
          mbar_arrive_expect_tx(full_bar(s), A_BYTES + B_BYTES);
          const uint32_t dst = smem_base + s * STAGE_BYTES;
          int ax, ay;
          a_coords(p, kb, mb * BM, ax, ay);
          tma_load_2d(dst, &amap, ax, ay, full_bar(s));
          tma_load_2d(dst + A_BYTES, &bmap, kb * (BK / 2), nb * BN, full_bar(s));
          if (++s == STAGES) { s = 0; ++round; }
        }
      }
    }
  } else if (warp == SFP_WARP) {
    // ------------------------------- scale producer -------------------------------------------------
    // The three small copies per k-block have a thread of their own: issued by the operand producer they
    // made its loop (a barrier wait and seven asynchronous operations per k-block) the slowest stage of
    // the pipeline.  The scale tiles use their own barrier, so the feeders can start before the operands land.
    if (lane == 0) {
      int s = 0;
      uint32_t round = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x) {
        int mb, nb, sp, kb0, kb1;
        work_coords(p, w, mb, nb, sp);
        split_range(p, sp, kb0, kb1);
        const int b_blocks = min(2, p.sfb_row_blocks - nb * 2);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!(ok = mbar_wait(empty_bar(s), (round & 1) ^ 1, abort_flag))) break;
          // scale atoms really present in this k-block (the last block may hold fewer)
          const int atoms = min(ATOMS, p.sf_atoms_k - kb * ATOMS);
          const uint32_t sf_bytes = (uint32_t)atoms * 512u;
          mbar_arrive_expect_tx(sffull_bar(s), sf_bytes * (1 + b_blocks));
          const uint32_t dst = smem_base + s * STAGE_BYTES + A_BYTES + B_BYTES;
          bulk_load(dst, a_scale_atoms(p, kb, mb, ATOMS), sf_bytes, sffull_bar(s));
          for (int r = 0; r < b_blocks; ++r)
            bulk_load(dst + SFA_BYTES + r * (SFB_BYTES / 2),
                      p.sfb + ((int64_t)(nb * 2 + r) * p.sf_atoms_k + kb * ATOMS) * 512, sf_bytes, sffull_bar(s));
          if (++s == STAGES) { s = 0; ++round; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -----------------------------------------------
    if (lane == 0) {
      int s = 0;
      uint32_t round = 0, it = 0;
      bool ok = true, ready = false;   // ready: the probe issued with the previous k-block saw this one complete
      for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x, ++it) {
        int mb, nb, sp, kb0, kb1;
        work_coords(p, w, mb, nb, sp);
        split_range(p, sp, kb0, kb1);
        if (!(ok = mbar_wait(tempty_bar, (it & 1) ^ 1, abort_flag))) break;
        tc_fence_after();
        for (int kb = kb0; kb < kb1; ++kb) {
          // fast path: the probe issued with the previous k-block saw both barriers of this one complete
          if (!ready) {
            if (!(ok = mbar_wait(full_bar(s), round & 1, abort_flag))) break;     // operands landed
            if (!(ok = mbar_wait(sf_bar(s), round & 1, abort_flag))) break;       // scales are in TMEM
          }
          tc_fence_after();
          const uint32_t a0 = smem_base + s * STAGE_BYTES, b0 = a0 + A_BYTES;
          const int atoms = min(ATOMS, p.sf_atoms_k - kb * ATOMS);
          // atom a of A sits in columns sfa_col + 4a, of B (two 128-row blocks) in sfb_col + 8a + 4r
          const uint32_t sfa_col = tmem_base + SF_COL0 + s * SF_STAGE_COLS, sfb_col = sfa_col + SFB_OFF;
          // K-major, 128-byte swizzle: 8-row groups 1024 bytes apart; 64 elements = 32 bytes
          const uint64_t ad = make_smem_desc(a0, 16, 1024, kSwizzle128B);
          const uint64_t bd = make_smem_desc(b0, 16, 1024, kSwizzle128B);
          const int sn = (s + 1 == STAGES) ? 0 : s + 1;
          const uint32_t parity_n = (sn == 0 ? round + 1 : round) & 1;
          if (atoms == ATOMS) {
            ready = umma_fp4_x4_probe<NV, false>(tmem_base, ad, bd, make_idesc_fp4(NV, 0), make_idesc_fp4(NV, NV ? 0 : 2),
                                                 sfa_col, sfb_col, kb > kb0, full_bar(sn), sf_bar(sn), parity_n);
          } else {
            const int ksteps = atoms * (NV ? 1 : 2);   // MMAs of K = 64 in a short last k-block
            for (int ks = 0; ks < ksteps; ++ks) {
              const int atom = NV ? ks : (ks >> 1);
              const uint32_t sf_id = NV ? 0u : (uint32_t)(ks & 1) * 2u;
              umma_fp4<NV>(tmem_base, ad + 2 * ks, bd + 2 * ks, make_idesc_fp4(NV, sf_id), sfa_col + 4 * atom,
                           sfb_col + 8 * atom, (kb > kb0) || (ks != 0));
            }
            ready = false;
          }
          umma_commit(empty_bar(s));
          if (++s == STAGES) { s = 0; ++round; }
        }
        if (ok) umma_commit(tfull_bar);
      }
    }
  } else if (warp >= SF_WARP0 && warp < SFP_WARP) {
    // ------------------------------- scale feeders ------------------------------------------------
    // Lane l of every feeder reads row l of each 128 x 4 scale atom from shared memory (16 bytes =
    // 4 columns: one per 32-row group, 4 consecutive k-scales per column) and stores it to its own
    // TMEM lane quarter.  A full stage implies that its TMEM scale region is free: the producer only
    // refills a stage after the MMAs that read it (and its scales) have completed.
    const int quarter = warp & 3;
    int s = 0;
    uint32_t round = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x) {
      int mb, nb, sp, kb0, kb1;
      work_coords(p, w, mb, nb, sp);
      split_range(p, sp, kb0, kb1);
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!(ok = mbar_wait(sffull_bar(s), round & 1, abort_flag))) break;
        const uint8_t* sfa = smem + s * STAGE_BYTES + A_BYTES + B_BYTES + lane * 16;
        const uint8_t* sfb = sfa + SFA_BYTES;
        uint4 va[ATOMS], vb[ATOMS][2];
#pragma unroll
        for (int a = 0; a < ATOMS; ++a) {
          va[a] = *reinterpret_cast<const uint4*>(sfa + a * 512);
          vb[a][0] = *reinterpret_cast<const uint4*>(sfb + a * 512);
          vb[a][1] = *reinterpret_cast<const uint4*>(sfb + SFB_BYTES / 2 + a * 512);
        }
        const uint32_t sfa_col = tmem_base + ((uint32_t)(quarter * 32) << 16) + SF_COL0 + s * SF_STAGE_COLS;
#pragma unroll
        for (int a = 0; a < ATOMS; a += 2) tmem_st_x8(sfa_col + 4 * a, va[a], va[a + 1]);
#pragma unroll
        for (int a = 0; a < ATOMS; ++a) tmem_st_x8(sfa_col + SFB_OFF + 8 * a, vb[a][0], vb[a][1]);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(sf_bar(s));
        if (++s == STAGES) { s = 0; ++round; }
      }
    }
  } else if (warp >= EPI_WARP0) {
    // ------------------------------- epilogue ---------------------------------------------------
    const int quarter = warp & 3;        // TMEM lanes this warp may read: 32*quarter .. +31
    const int half = (warp - EPI_WARP0) >> 2;    // which 128 of the tile's 256 columns
    const float alpha = *p.alpha;
    uint32_t it = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x, ++it) {
      int mb, nb, sp;
      work_coords(p, w, mb, nb, sp);
      if (!(ok = mbar_wait(tfull_bar, it & 1, abort_flag))) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + half * 128;
      const int row = mb * BM + quarter * 32 + lane;
      const int col0 = nb * BN + half * 128;
      if (p.splits == 1) {
        drain_and_store(p, taddr, alpha, row - lane, col0, lane, [&] {
          if (lane == 0) mbar_arrive(tempty_bar);
        });
      } else if (CLUSTER) {
        // split K inside a cluster: the valid rows of the fp32 partial tile go to this CTA's shared memory (the
        // pipeline stages are free: every MMA has completed, so every load has landed and been read)
        float* dst = reinterpret_cast<float*>(smem) + (quarter * 32 + lane) * CL_ROW_FLOATS + half * 128;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait();
          if (row < p.m) {
#pragma unroll
            for (int u = 0; u < 8; ++u)
              *reinterpret_cast<float4*>(dst + c * 32 + 4 * u) =
                  make_float4(__uint_as_float(r[4 * u]), __uint_as_float(r[4 * u + 1]),
                              __uint_as_float(r[4 * u + 2]), __uint_as_float(r[4 * u + 3]));
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar);
      } else {
        // split K through global memory: fp32 partial tile, stored chunk by chunk; a second kernel adds the splits
        float* dst = p.partial + ((int64_t)sp * p.m + row) * p.n + col0;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait();
          if (row < p.m) {
#pragma unroll
            for (int u = 0; u < 8; ++u)     // n % 8 == 0: groups of 4 never straddle the edge
              if (col0 + c * 32 + 4 * u < p.n)
                *reinterpret_cast<float4*>(dst + c * 32 + 4 * u) =
                    make_float4(__uint_as_float(r[4 * u]), __uint_as_float(r[4 * u + 1]),
                                __uint_as_float(r[4 * u + 2]), __uint_as_float(r[4 * u + 3]));
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar);
      }
    }
  }

  if (CLUSTER) {
    // every thread of every CTA of the cluster gets here, whatever its role and even after a wait that ran out
    cluster_sync_all();                 // the partial tiles of all CTAs are staged
    if (warp >= EPI_WARP0 && warp < SF_WARP0) {
      int mb, nb, sp;
      work_coords(p, blockIdx.x, mb, nb, sp);
      splitk_cluster_finish(p, smem_base, sp, p.splits, mb * BM, nb * BN, *p.alpha, threadIdx.x - EPI_WARP0 * 32);
    }
    cluster_sync_all();                 // nobody leaves while its shared memory may still be read
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_flag && p.status) atomicExch(p.status, 1);
}


// ---------------------------------------------------------------------------------------------------
// CTA-pair kernel (cta_group::2), the default for M > 128: two CTAs of a cluster compute a 256 x 256 tile.
// Each holds its own 128 rows of A (and their scales), one half (128 rows) of B, and the scales of all 256
// columns of B.  Per k-block every SM now receives 32 KB of operands instead of 48: the 1-CTA kernel is bound
// by the L2 -> SM feed (about 15 TB/s over 148 SMs), this one is not.  No TMA multicast: every CTA fetches its
// own boxes.  Barriers: operand loads of both CTAs count on the leader's `full`; scale copies count on a local
// `sffull`; the leader's feeders arrive on its `sfready` (after `full`), the peer's on a local barrier that one
// relay thread forwards with a relaxed cluster-scope arrival (a releasing remote arrival costs ~1600 cycles
// with TMA traffic in flight and had made this kernel half as fast as the 1-CTA one); commits are multicast to
// both CTAs.  WUSH_B200_GEMM_PAIR=0 selects the 1-CTA kernel for every shape.
// ---------------------------------------------------------------------------------------------------
constexpr int P_B_BYTES = B_BYTES / 2;                                   // 128 rows of B
// Stage geometry by format: MXFP4 has half the scale bytes of NVFP4 per k-block, which buys a sixth stage.
template <bool NV>
struct PairGeom {
  static constexpr int SFA_B = NV ? 2048 : 1024;                 // scale tile of A: 4 / 2 atoms of 512 B
  static constexpr int SFB_B = NV ? 4096 : 2048;                 // two 128-row blocks of B scales
  static constexpr int STAGES = NV ? 5 : 6;
  static constexpr int STAGE_BYTES = A_BYTES + P_B_BYTES + SFA_B + SFB_B;      // 38 KB / 35 KB
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + 512;               // barriers: 5 * STAGES + 2 words
  static constexpr uint32_t SF_COLS = NV ? 48 : 24;              // TMEM columns of one stage's scales
  static constexpr uint32_t SFB_COL = NV ? 16 : 8;               // where the B scales start inside them
};

template <bool NV>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
fp4_gemm_pair_kernel(const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap bmap, const Params p) {
  constexpr int GROUP = NV ? 16 : 32;
  constexpr int ATOMS = BK / GROUP / 4;
  using G = PairGeom<NV>;
  constexpr int P_STAGES = G::STAGES, P_STAGE_BYTES = G::STAGE_BYTES;
  extern __shared__ uint8_t smem_unaligned[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + P_STAGES * P_STAGE_BYTES);
  // [0,S) full (leader's used)  [S,2S) sffull (local)  [2S,3S) empty  [3S,4S) sfready (leader's used)
  // [4S] tmem_full  [4S+1] tmem_empty (leader's used)  [4S+2,5S+2) sflocal (peer's used)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5 * P_STAGES + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair_id = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_u32(bars);
  auto full_bar = [&](int s) { return bar_base + 8 * s; };
  auto sffull_bar = [&](int s) { return bar_base + 8 * (P_STAGES + s); };
  auto empty_bar = [&](int s) { return bar_base + 8 * (2 * P_STAGES + s); };
  auto sfready_bar = [&](int s) { return bar_base + 8 * (3 * P_STAGES + s); };
  const uint32_t tfull_bar = bar_base + 8 * (4 * P_STAGES), tempty_bar = bar_base + 8 * (4 * P_STAGES + 1);
  auto sflocal_bar = [&](int s) { return bar_base + 8 * (4 * P_STAGES + 2 + s); };

  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(sffull_bar(s), 1);
      mbar_init(empty_bar(s), 1);
      mbar_init(sfready_bar(s), 5);   // the leader's 4 feeder warps + one relayed arrival for the peer's four
      mbar_init(sflocal_bar(s), 4);   // peer CTA: its feeder warps; a relay thread forwards the completion
    }
    mbar_init(tfull_bar, 1);
    mbar_init(tempty_bar, 16);        // 8 epilogue warps of each CTA
    *abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int m_blocks2 = (p.m + 255) / 256;
  const int n_work = m_blocks2 * p.n_blocks;
  const int sfa_row_blocks = (p.m + 127) / 128;

  if (warp == 0) {
    // ------------------------------- producer (both CTAs) -------------------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&amap);
      tma_prefetch_desc(&bmap);
      int s = 0;
      uint32_t round = 0;
      bool ok = true;
      for (int w = pair_id; w < n_work && ok; w += n_pairs) {
        const int mb2 = w % m_blocks2, nb = w / m_blocks2;
        const int a_blk = mb2 * 2 + (int)rank;                    // this CTA's 128-row block of A
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!(ok = mbar_wait(empty_bar(s), (round & 1) ^ 1, abort_flag))) break;
          if (leader) mbar_arrive_expect_tx(full_bar(s), 2 * (A_BYTES + P_B_BYTES));
          const uint32_t full_leader = map_to_cta(full_bar(s), 0);
          const uint32_t dst = smem_base + s * P_STAGE_BYTES;
          int ax, ay;
          a_coords(p, kb, a_blk * 128, ax, ay);
          tma_load_2d_pair(dst, &amap, ax, ay, full_leader);
          tma_load_2d_pair(dst + A_BYTES, &bmap, kb * (BK / 2), nb * BN + (int)rank * 128, full_leader);
          if (++s == P_STAGES) { s = 0; ++round; }
        }
      }
    }
  } else if (warp == SFP_WARP) {
    // ------------------------------- scale producer (both CTAs) -------------------------------------
    if (lane == 0) {
      int s = 0;
      uint32_t round = 0;
      bool ok = true;
      for (int w = pair_id; w < n_work && ok; w += n_pairs) {
        const int mb2 = w % m_blocks2, nb = w / m_blocks2;
        const int a_blk = mb2 * 2 + (int)rank;
        const bool a_sf = a_blk < sfa_row_blocks;                 // rows past M have no scales (and zero data)
        const int b_blocks = min(2, p.sfb_row_blocks - nb * 2);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!(ok = mbar_wait(empty_bar(s), (round & 1) ^ 1, abort_flag))) break;
          const int atoms = min(ATOMS, p.sf_atoms_k - kb * ATOMS);
          const uint32_t sf_bytes = (uint32_t)atoms * 512u;
          mbar_arrive_expect_tx(sffull_bar(s), sf_bytes * ((a_sf ? 1 : 0) + b_blocks));
          const uint32_t dst = smem_base + s * P_STAGE_BYTES + A_BYTES + P_B_BYTES;
          if (a_sf)
            bulk_load(dst, a_scale_atoms(p, kb, a_blk, ATOMS), sf_bytes, sffull_bar(s));
          for (int r = 0; r < b_blocks; ++r)
            bulk_load(dst + G::SFA_B + r * (G::SFB_B / 2),
                      p.sfb + ((int64_t)(nb * 2 + r) * p.sf_atoms_k + kb * ATOMS) * 512, sf_bytes, sffull_bar(s));
          if (++s == P_STAGES) { s = 0; ++round; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer (leader only) ---------------------------------------
    if (lane == 0 && leader) {
      int s = 0;
      uint32_t round = 0, it = 0;
      bool ok = true, ready = false;
      for (int w = pair_id; w < n_work && ok; w += n_pairs, ++it) {
        if (!(ok = mbar_wait(tempty_bar, (it & 1) ^ 1, abort_flag))) break;
        tc_fence_after();
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!ready) {
            if (!(ok = mbar_wait(full_bar(s), round & 1, abort_flag))) break;      // operands of both CTAs landed
            if (!(ok = mbar_wait(sfready_bar(s), round & 1, abort_flag))) break;   // scales of both CTAs in TMEM
          }
          tc_fence_after();
          const uint32_t a0 = smem_base + s * P_STAGE_BYTES, b0 = a0 + A_BYTES;
          const int atoms = min(ATOMS, p.sf_atoms_k - kb * ATOMS);
          const uint32_t sfa_col = tmem_base + SF_COL0 + s * G::SF_COLS, sfb_col = sfa_col + G::SFB_COL;
          const uint64_t ad = make_smem_desc(a0, 16, 1024, kSwizzle128B);
          const uint64_t bd = make_smem_desc(b0, 16, 1024, kSwizzle128B);
          const int sn = (s + 1 == P_STAGES) ? 0 : s + 1;
          const uint32_t parity_n = (sn == 0 ? round + 1 : round) & 1;
          if (atoms == ATOMS) {
            ready = umma_fp4_x4_probe<NV, true>(tmem_base, ad, bd, make_idesc_fp4(NV, 0, 256),
                                                make_idesc_fp4(NV, NV ? 0 : 2, 256), sfa_col, sfb_col, kb > 0,
                                                full_bar(sn), sfready_bar(sn), parity_n);
          } else {
            const int ksteps = atoms * (NV ? 1 : 2);
            for (int ks = 0; ks < ksteps; ++ks) {
              const int atom = NV ? ks : (ks >> 1);
              const uint32_t sf_id = NV ? 0u : (uint32_t)(ks & 1) * 2u;
              umma_fp4_pair<NV>(tmem_base, ad + 2 * ks, bd + 2 * ks, make_idesc_fp4(NV, sf_id, 256), sfa_col + 4 * atom,
                                sfb_col + 8 * atom, (kb > 0) || (ks != 0));
            }
            ready = false;
          }
          umma_commit_pair(empty_bar(s), 3);
          if (++s == P_STAGES) { s = 0; ++round; }
        }
        if (ok) umma_commit_pair(tfull_bar, 3);
      }
    } else if (lane == 0) {
      // peer CTA: this otherwise idle thread relays "the peer's scales are in TMEM" to the leader with ONE
      // cluster-scope arrival per stage (remote arrivals are expensive; the feeders arrive locally)
      int s = 0;
      uint32_t round = 0;
      bool ok = true;
      for (int w = pair_id; w < n_work && ok; w += n_pairs) {
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!(ok = mbar_wait(sflocal_bar(s), round & 1, abort_flag))) break;
          mbar_arrive_cluster_relaxed(map_to_cta(sfready_bar(s), 0));
          if (++s == P_STAGES) { s = 0; ++round; }
        }
      }
    }
  } else if (warp >= SF_WARP0 && warp < SFP_WARP) {
    // ------------------------------- scale feeders (both CTAs) --------------------------------------
    const int quarter = warp & 3;
    int s = 0;
    uint32_t round = 0;
    bool ok = true;
    for (int w = pair_id; w < n_work && ok; w += n_pairs) {
      for (int kb = 0; kb < p.k_blocks; ++kb) {
        if (!(ok = mbar_wait(sffull_bar(s), round & 1, abort_flag))) break;
        const uint8_t* sfa = smem + s * P_STAGE_BYTES + A_BYTES + P_B_BYTES + lane * 16;
        const uint8_t* sfb = sfa + G::SFA_B;
        uint4 va[ATOMS], vb[ATOMS][2];
#pragma unroll
        for (int a = 0; a < ATOMS; ++a) {
          va[a] = *reinterpret_cast<const uint4*>(sfa + a * 512);
          vb[a][0] = *reinterpret_cast<const uint4*>(sfb + a * 512);
          vb[a][1] = *reinterpret_cast<const uint4*>(sfb + G::SFB_B / 2 + a * 512);
        }
        const uint32_t sfa_col = tmem_base + ((uint32_t)(quarter * 32) << 16) + SF_COL0 + s * G::SF_COLS;
#pragma unroll
        for (int a = 0; a < ATOMS; a += 2) tmem_st_x8(sfa_col + 4 * a, va[a], va[a + 1]);
#pragma unroll
        for (int a = 0; a < ATOMS; ++a) tmem_st_x8(sfa_col + G::SFB_COL + 8 * a, vb[a][0], vb[a][1]);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(leader ? sfready_bar(s) : sflocal_bar(s));
        if (++s == P_STAGES) { s = 0; ++round; }
      }
    }
  } else if (warp >= EPI_WARP0) {
    // ------------------------------- epilogue (both CTAs, own 128 rows) -----------------------------
    const int quarter = warp & 3;
    const int half = (warp - EPI_WARP0) >> 2;
    const float alpha = *p.alpha;
    uint32_t it = 0;
    bool ok = true;
    for (int w = pair_id; w < n_work && ok; w += n_pairs, ++it) {
      const int mb2 = w % m_blocks2, nb = w / m_blocks2;
      if (!(ok = mbar_wait(tfull_bar, it & 1, abort_flag))) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + half * 128;
      const int row = mb2 * 256 + (int)rank * 128 + quarter * 32 + lane;
      drain_and_store(p, taddr, alpha, row - lane, nb * BN + half * 128, lane, [&] {
        if (lane == 0) {
          // the accumulator reads are complete (tcgen05.wait::ld), nothing travels through memory: the
          // relaxed remote arrival avoids the ~1600-cycle release fence
          if (leader) mbar_arrive(tempty_bar);
          else mbar_arrive_cluster_relaxed(map_to_cta(tempty_bar, 0));
        }
      });
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_flag && p.status) atomicExch(p.status, 1);
}

// Split K through global memory, second kernel: add the per-split fp32 partial tiles, scale, add the optional
// epilogue terms, round to bf16.
__global__ void splitk_reduce_kernel(const Params p) {
  const float a = *p.alpha;
  const int64_t mn = (int64_t)p.m * p.n;
  for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < mn; i += (int64_t)gridDim.x * blockDim.x * 4) {
    float4 acc = *reinterpret_cast<const float4*>(p.partial + i);
    for (int s = 1; s < p.splits; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(p.partial + (int64_t)s * mn + i);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    const int row = (int)(i / p.n), col = (int)(i - (int64_t)row * p.n);     // n % 8 == 0: 4 values share a row
    *reinterpret_cast<uint2*>(p.y + (int64_t)row * p.ldy + p.ycol0 + col) = finish_f4(p, acc, a, row, col);
  }
}

// K splits for a problem: enough CTAs to occupy the machine when there are few output tiles
// (small M: the GEMM streams the weights once and is HBM-bound), at least 2 k-blocks per split.
static int choose_splits(int64_t tiles, int k_blocks, int sms, int cap) {
  if (tiles >= sms) return 1;
  int64_t s = sms / tiles;
  if (s > k_blocks / 2) s = k_blocks / 2;
  if (s > cap) s = cap;
  return s < 1 ? 1 : (int)s;
}

struct Shard {               // column-sharded output: where this GPU's columns go, here and on the other GPUs
  void* const* y_all = nullptr;   // HOST array of `world` device pointers, entry `rank` being this GPU's buffer
  int world = 1, rank = 0;
  int64_t ldy = 0, col0 = 0;
};

struct Epilogue {            // optional terms added to the output, its row stride, and a K-sharded A operand
  const void* bias = nullptr;
  const void* residual = nullptr;
  int64_t ldr = 0;
  int64_t ldy = 0;           // 0: n
  int a_shards = 1;          // > 1: A is `a_shards` stacked [a_shard_rows, k / a_shards / 2] matrices
  int64_t a_shard_rows = 0;
  int64_t a_sf_shard_bytes = 0;   // bytes between the scale tensors of two shards (0: densely stacked)
};

// Tensor maps are pure functions of (base pointer, shape, box), and encoding one costs about a microsecond
// of host time; a decode-size GEMM runs for a few microseconds.  The last maps are kept in a small
// direct-mapped cache guarded by a mutex.
struct MapKey {
  const void* base;
  uint64_t rows, cols;
  uint32_t box_rows;
  bool operator==(const MapKey& o) const { return base == o.base && rows == o.rows && cols == o.cols && box_rows == o.box_rows; }
};
static int cached_operand_map(CUtensorMap* out, const void* base, uint64_t rows, uint64_t k_bytes, uint32_t box_rows) {
  constexpr int kSlots = 64;
  static MapKey keys[kSlots];
  static CUtensorMap maps[kSlots];
  static bool used[kSlots];
  static std::mutex mu;
  const MapKey key{base, rows, k_bytes, box_rows};
  const size_t hsh = ((uintptr_t)base >> 8) * 0x9E3779B97F4A7C15ull ^ (rows * 31 + k_bytes * 131 + box_rows);
  const int slot = (int)((hsh >> 20) % kSlots);
  {
    std::lock_guard<std::mutex> lock(mu);
    if (used[slot] && keys[slot] == key) {
      *out = maps[slot];
      return 0;
    }
  }
  const int rc = make_tensor_map_2d(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, base, rows, k_bytes, k_bytes, BK / 2, box_rows,
                                    CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != 0) return rc;
  std::lock_guard<std::mutex> lock(mu);
  keys[slot] = key;
  maps[slot] = *out;
  used[slot] = true;
  return 0;
}

// Clusters of `splits` CTAs of the split-K kernel that can be resident at once on the current device (each CTA
// fills an SM; a cluster must fit into one GPC).  Also opts the kernel into its shared memory.  Cached per device.
static int cluster_capacity(bool nv, int splits) {
  static PerDevice attr[2], cap[2][4];     // cap[..][log2(splits)]: capacity + 1 (0 = not asked yet)
  auto ck = nv ? fp4_gemm_kernel<true, true> : fp4_gemm_kernel<false, true>;
  if (opt_in_smem(attr[nv], ck, SMEM_BYTES) != 0) return 0;
  int lg = 0;
  while ((1 << lg) < splits) ++lg;
  if (lg > 3 || (1 << lg) != splits) return 0;
  const int dev = device_slot();
  int state = dev >= 0 ? cap[nv][lg].get(dev) : 0;
  if (!state) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(splits * (sm_count() / splits)));
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cudaLaunchAttribute a;
    a.id = cudaLaunchAttributeClusterDimension;
    a.val.clusterDim.x = (unsigned)splits;
    a.val.clusterDim.y = 1;
    a.val.clusterDim.z = 1;
    cfg.attrs = &a;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, ck, &cfg) != cudaSuccess || n < 0) n = 0;
    state = n + 1;
    if (dev >= 0) cap[nv][lg].set(dev, state);
  }
  return state - 1;
}

static int gemm_launch(bool nv, const uint8_t* a, const uint8_t* b, const uint8_t* sfa, const uint8_t* sfb,
                       const float* alpha, void* y, int64_t m, int64_t n, int64_t k, float* partial,
                       size_t partial_bytes, int force_splits, int* status, cudaStream_t stream,
                       const Shard* shard = nullptr, const Epilogue* epi = nullptr) {
  if (!a || !b || !sfa || !sfb || !alpha || !y) return WUSH_ERR_NULL_POINTER;
  if (m < 0 || n <= 0 || k <= 0 || k % 128 != 0 || n % 8 != 0 || m > 0x7fffffff || n > 0x7fffffff || k > 0x7fffffff)
    return WUSH_ERR_BAD_SHAPE;
  if (((uintptr_t)a & 15) || ((uintptr_t)b & 15) || ((uintptr_t)sfa & 15) || ((uintptr_t)sfb & 15) || ((uintptr_t)y & 15))
    return WUSH_ERR_BAD_ALIGNMENT;
  if (m == 0) return WUSH_OK;
  int rc = require_sm100();
  if (rc != 0) return rc;
  const int group = nv ? 16 : 32;
  Params p{};
  p.sfa = sfa; p.sfb = sfb; p.alpha = alpha; p.y = (__nv_bfloat16*)y;
  p.m = (int)m; p.n = (int)n; p.k = (int)k;
  p.ldy = n;
  if (epi) {
    if (epi->ldy) p.ldy = epi->ldy;
    p.bias = (const __nv_bfloat16*)epi->bias;
    p.residual = (const __nv_bfloat16*)epi->residual;
    p.ldr = epi->ldr ? epi->ldr : n;
    if (p.ldy < n || p.ldy % 8 || p.ldr < n || p.ldr % 8) return WUSH_ERR_BAD_SHAPE;
    if (((uintptr_t)p.bias & 15) || ((uintptr_t)p.residual & 15)) return WUSH_ERR_BAD_ALIGNMENT;
  }
  if (shard) {
    p.ldy = shard->ldy;
    p.ycol0 = shard->col0;
    // every rank starts with its right-hand neighbour, so that the ranks do not all write to the same GPU at once
    for (int i = 1; i < shard->world; ++i)
      p.y_peer[p.n_peers++] = (__nv_bfloat16*)shard->y_all[(shard->rank + i) % shard->world];
    force_splits = 1;      // partial tiles have no peer path: the sharded GEMM always runs unsplit
  }
  // decode: with a handful of activation rows the product is one pass over the weight bytes, done by the
  // matrix-vector kernel (no K splits, tensor maps or tensor memory); callers that force a split count, shard the
  // output or stack K shards keep the tensor-core path
  if (force_splits <= 0 && !shard && !(epi && epi->a_shards > 1) && m <= gemv::max_rows() && k <= gemv::max_k())
    return gemv::launch(nv, a, b, sfa, sfb, alpha, p.bias, p.residual, p.ldr ? p.ldr : n, y, p.ldy, (int)m, (int)n, (int)k,
                        stream);
  p.m_blocks = (int)((m + BM - 1) / BM);
  p.n_blocks = (int)((n + BN - 1) / BN);
  p.k_blocks = (int)((k + BK - 1) / BK);
  p.sf_atoms_k = (int)((k / group + 3) / 4);
  p.sfb_row_blocks = (int)((n + 127) / 128);
  p.status = status;
  const int sms = sm_count();
  const int64_t tiles = (int64_t)p.m_blocks * p.n_blocks;
  // K splits.  Automatic: a power of two up to 8, the CTAs of a split forming a cluster that reduces through
  // shared memory (no scratch).  Forced by the caller: any count, fp32 partial tiles in the caller's workspace
  // and a second kernel.
  int splits = 1;
  bool cluster = false;
  if (force_splits > 0) {
    splits = force_splits > p.k_blocks ? p.k_blocks : force_splits;
    const size_t need = splits > 1 ? (size_t)splits * m * n * sizeof(float) : 0;
    if (need > partial_bytes || (need && !partial)) return WUSH_ERR_WORKSPACE_TOO_SMALL;
    if (splits > 1 && ((uintptr_t)partial & 15)) return WUSH_ERR_BAD_ALIGNMENT;
  } else {
    // the largest cluster size whose clusters (one per tile) are all resident at once: a second wave of
    // clusters would double the run time of a launch that is a few microseconds long
    static const int cap_env = env_int("WUSH_B200_GEMM_MAX_SPLITS", MAX_CLUSTER_SPLITS);
    const int want = choose_splits(tiles, p.k_blocks, sms, cap_env < MAX_CLUSTER_SPLITS ? cap_env : MAX_CLUSTER_SPLITS);
    while (splits * 2 <= want) splits *= 2;
    while (splits > 1 && cluster_capacity(nv, splits) < tiles) splits /= 2;
    cluster = splits > 1;
  }
  p.splits = splits;
  p.cluster_splits = cluster ? 1 : 0;
  p.partial = partial;

  CUtensorMap amap, bmap;
  if (epi && epi->a_shards > 1) {
    const int64_t ks = k / epi->a_shards;
    if (k % epi->a_shards || ks % BK || epi->a_shard_rows < m) return WUSH_ERR_BAD_SHAPE;
    p.a_kbs = (int)(ks / BK);
    p.a_shard_rows = (int)epi->a_shard_rows;
    p.a_sf_atoms = (int)(ks / group / 4);
    p.a_sf_shard_bytes = epi->a_sf_shard_bytes ? epi->a_sf_shard_bytes
                                               : (int64_t)((epi->a_shard_rows + 127) / 128) * p.a_sf_atoms * 512;
    if (p.a_sf_shard_bytes % 16) return WUSH_ERR_BAD_ALIGNMENT;
    rc = cached_operand_map(&amap, a, (uint64_t)epi->a_shard_rows * epi->a_shards, (uint64_t)ks / 2, BM);
  } else {
    rc = cached_operand_map(&amap, a, (uint64_t)m, (uint64_t)k / 2, BM);
  }
  if (rc != 0) return rc;

  // large M, unsplit: 256 x 256 tiles on CTA pairs
  static const int use_pair = env_int("WUSH_B200_GEMM_PAIR", 1);
  if (use_pair && splits == 1 && m > 128 && sms >= 2) {
    rc = cached_operand_map(&bmap, b, (uint64_t)n, (uint64_t)k / 2, 128);
    if (rc != 0) return rc;
    auto pk = nv ? fp4_gemm_pair_kernel<true> : fp4_gemm_pair_kernel<false>;
    const int psmem = nv ? PairGeom<true>::SMEM : PairGeom<false>::SMEM;
    static PerDevice pair_attr[2], max_pairs[2];
    rc = opt_in_smem(pair_attr[nv], pk, psmem);
    if (rc != 0) return rc;
    const int dev = device_slot();
    int nmax = dev >= 0 ? max_pairs[nv].get(dev) : 0;
    if (nmax == 0) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(2 * (sms / 2));
      cfg.blockDim = dim3(THREADS);
      cfg.dynamicSmemBytes = psmem;
      cudaLaunchAttribute attr;
      attr.id = cudaLaunchAttributeClusterDimension;
      attr.val.clusterDim.x = 2;
      attr.val.clusterDim.y = 1;
      attr.val.clusterDim.z = 1;
      cfg.attrs = &attr;
      cfg.numAttrs = 1;
      if (cudaOccupancyMaxActiveClusters(&nmax, pk, &cfg) != cudaSuccess || nmax <= 0) nmax = sms / 2;
      if (dev >= 0) max_pairs[nv].set(dev, nmax);
    }
    const int64_t ptiles = ((m + 255) / 256) * (int64_t)p.n_blocks;
    int64_t pairs = nmax < sms / 2 ? nmax : sms / 2;
    if (pairs > ptiles) pairs = ptiles;
    pk<<<(unsigned)(2 * pairs), THREADS, psmem, stream>>>(amap, bmap, p);
    return (int)cudaGetLastError();
  }

  rc = cached_operand_map(&bmap, b, (uint64_t)n, (uint64_t)k / 2, BN);
  if (rc != 0) return rc;
  if (cluster) {
    auto ck = nv ? fp4_gemm_kernel<true, true> : fp4_gemm_kernel<false, true>;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(tiles * splits));     // one work item per CTA; cluster c = tile c, rank = split
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = (unsigned)splits;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&cfg, ck, amap, bmap, p);
  }
  auto kern = nv ? fp4_gemm_kernel<true, false> : fp4_gemm_kernel<false, false>;
  static PerDevice attr_one[2];
  rc = opt_in_smem(attr_one[nv], kern, SMEM_BYTES);
  if (rc != 0) return rc;
  int64_t work = tiles * splits;
  int grid = (int)(work < sms ? work : sms);
  kern<<<grid, THREADS, SMEM_BYTES, stream>>>(amap, bmap, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  if (splits > 1) {
    const int64_t mn = m * n;   // n % 8 == 0, so mn % 4 == 0
    int64_t blocks = (mn / 4 + 255) / 256;
    if (blocks > (int64_t)sms * 8) blocks = (int64_t)sms * 8;
    splitk_reduce_kernel<<<(unsigned)blocks, 256, 0, stream>>>(p);
    e = cudaGetLastError();
  }
  return (int)e;
}

static int gemm_with_workspace(bool nv, const uint8_t* a, const uint8_t* b, const uint8_t* sfa, const uint8_t* sfb,
                               const float* alpha, void* y, int64_t m, int64_t n, int64_t k, void* workspace,
                               size_t workspace_bytes, int splits, int* status, void* stream, const Epilogue* epi) {
  return gemm_launch(nv, a, b, sfa, sfb, alpha, y, m, n, k, static_cast<float*>(workspace), workspace ? workspace_bytes : 0,
                     splits, status, (cudaStream_t)stream, nullptr, epi);
}

}  // namespace gemm
}  // namespace wush

extern "C" int wush_gemm_mxf4_bf16_tn(const uint8_t* a, const uint8_t* b, const uint8_t* sfa, const uint8_t* sfb,
                                      const float* alpha, void* y, int64_t m, int64_t n, int64_t k, void* workspace,
                                      size_t workspace_bytes, int splits, int* status, void* stream) {
  return wush::gemm::gemm_with_workspace(false, a, b, sfa, sfb, alpha, y, m, n, k, workspace, workspace_bytes, splits,
                                         status, stream, nullptr);
}

extern "C" int wush_gemm_nvf4_bf16_tn(const uint8_t* a, const uint8_t* b, const uint8_t* sfa, const uint8_t* sfb,
                                      const float* alpha, void* y, int64_t m, int64_t n, int64_t k, void* workspace,
                                      size_t workspace_bytes, int splits, int* status, void* stream) {
  return wush::gemm::gemm_with_workspace(true, a, b, sfa, sfb, alpha, y, m, n, k, workspace, workspace_bytes, splits,
                                         status, stream, nullptr);
}

extern "C" int wush_gemm_fp4_bf16_tn_fused(int format, const uint8_t* a, int a_shards, int64_t a_shard_rows,
                                           int64_t a_sf_shard_bytes, const uint8_t* b, const uint8_t* sfa,
                                           const uint8_t* sfb, const float* alpha,
                                           const void* bias, const void* residual, int64_t ldr, void* y, int64_t ldy,
                                           int64_t m, int64_t n, int64_t k, void* workspace, size_t workspace_bytes,
                                           int splits, int* status, void* stream) {
  if (format != WUSH_FORMAT_MXFP4 && format != WUSH_FORMAT_NVFP4) return WUSH_ERR_BAD_FLAG;
  if (a_shards < 1 || a_shards > 64) return WUSH_ERR_BAD_SHAPE;
  wush::gemm::Epilogue epi;
  epi.bias = bias; epi.residual = residual; epi.ldr = ldr; epi.ldy = ldy;
  epi.a_shards = a_shards; epi.a_shard_rows = a_shard_rows; epi.a_sf_shard_bytes = a_sf_shard_bytes;
  return wush::gemm::gemm_with_workspace(format == WUSH_FORMAT_NVFP4, a, b, sfa, sfb, alpha, y, m, n, k, workspace,
                                         workspace_bytes, splits, status, stream, &epi);
}

extern "C" int wush_gemm_fp4_bf16_tn_sharded(int format, const uint8_t* a, const uint8_t* b, const uint8_t* sfa,
                                             const uint8_t* sfb, const float* alpha, void* const* y_all, int world,
                                             int rank, int64_t ldy, int64_t col0, int64_t m, int64_t n, int64_t k,
                                             int* status, void* stream) {
  using namespace wush::gemm;
  if (format != WUSH_FORMAT_MXFP4 && format != WUSH_FORMAT_NVFP4) return WUSH_ERR_BAD_FLAG;
  if (!y_all) return WUSH_ERR_NULL_POINTER;
  if (world < 1 || world > MAX_PEERS || rank < 0 || rank >= world) return WUSH_ERR_BAD_SHAPE;
  if (ldy < col0 + n || col0 < 0 || col0 % 8 || ldy % 8) return WUSH_ERR_BAD_SHAPE;
  for (int r = 0; r < world; ++r) {
    if (!y_all[r]) return WUSH_ERR_NULL_POINTER;
    if ((uintptr_t)y_all[r] & 15) return WUSH_ERR_BAD_ALIGNMENT;
  }
  Shard sh;
  sh.y_all = y_all; sh.world = world; sh.rank = rank; sh.ldy = ldy; sh.col0 = col0;
  return gemm_launch(format == WUSH_FORMAT_NVFP4, a, b, sfa, sfb, alpha, y_all[rank], m, n, k, nullptr, 0, 1, status,
                     (cudaStream_t)stream, &sh);
}

// ---------------------------------------------------------------------------------------------
// Split-K MXFP4 GEMM whose partial tiles live in a fixed device array instead of a caller-supplied
// workspace.  See the declaration in wush_b200.h for who needs this and for the rules.
// ---------------------------------------------------------------------------------------------
namespace wush {
namespace gemm {

constexpr size_t kStaticScratchFloats = WUSH_GEMM_STATIC_SCRATCH_BYTES / sizeof(float);
static __device__ __align__(256) float g_splitk_scratch[kStaticScratchFloats];

// Device address of g_splitk_scratch on the current device.  In host code the array's name is only a
// handle for the runtime, never a pointer a kernel could use, so the address is looked up once per
// device (with that device current) and cached.
static int static_scratch_address(float** out) {
  static float* cache[kMaxDevices] = {};
  static std::mutex mu;
  const int dev = device_slot();
  if (dev < 0) {
    int d = 0;
    const cudaError_t e = cudaGetDevice(&d);
    return e != cudaSuccess ? (int)e : WUSH_ERR_BAD_SHAPE;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (!cache[dev]) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_splitk_scratch);
    if (e != cudaSuccess) return (int)e;
    cache[dev] = static_cast<float*>(p);
  }
  *out = cache[dev];
  return WUSH_OK;
}

}  // namespace gemm
}  // namespace wush

extern "C" int wush_gemm_mxf4_bf16_tn_noalloc(const uint8_t* a, const uint8_t* b, const uint8_t* sfa, const uint8_t* sfb,
                                              const float* alpha, void* y, int64_t m, int64_t n, int64_t k, int splits,
                                              int* status, void* stream) {
  using namespace wush::gemm;
  if (m < 0 || n <= 0 || k <= 0) return WUSH_ERR_BAD_SHAPE;
  if (splits < 0) return WUSH_ERR_BAD_FLAG;
  const int k_blocks = (int)((k + BK - 1) / BK);
  const int64_t tiles = ((m + BM - 1) / BM) * ((n + BN - 1) / BN);
  if (splits == 0) {
    splits = choose_splits(tiles, k_blocks, wush::sm_count(), 16);
    // keep the partial tiles inside the fixed array, but stay a split-K launch
    while (splits > 2 && (size_t)splits * m * n > kStaticScratchFloats) --splits;
    if (splits < 2) splits = 2;
  }
  if (splits < 2 || splits > k_blocks) return WUSH_ERR_BAD_FLAG;   // K too short to split, or a forced value out of range
  if ((size_t)splits * (size_t)m * (size_t)n > kStaticScratchFloats) return WUSH_ERR_TOO_LARGE;
  float* scratch = nullptr;
  const int rc = static_scratch_address(&scratch);
  if (rc != WUSH_OK) return rc;
  return gemm_launch(false, a, b, sfa, sfb, alpha, y, m, n, k, scratch, WUSH_GEMM_STATIC_SCRATCH_BYTES, splits, status,
                     (cudaStream_t)stream);
}

extern "C" size_t wush_gemm_workspace_bytes(int64_t m, int64_t n, int64_t k, int splits) {
  if (m <= 0 || n <= 0 || k <= 0 || splits <= 1) return 0;
  return (size_t)splits * m * n * sizeof(float);
}

extern "C" int wush_gemm_cluster_capacity(int format, int splits) {
  if (format != WUSH_FORMAT_MXFP4 && format != WUSH_FORMAT_NVFP4) return WUSH_ERR_BAD_FLAG;
  if (wush::require_sm100() != 0) return 0;
  return wush::gemm::cluster_capacity(format == WUSH_FORMAT_NVFP4, splits);
}
