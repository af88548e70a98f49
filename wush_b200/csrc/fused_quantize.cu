// Fused per-group transform + FP4 quantization for sm_100a.
//
// One pass over the activations: x (bf16) is read once with 128-bit loads, each 32-channel
// chunk is multiplied by its own 32x32 (MXFP4) or block-diagonal 2x(16x16) (NVFP4) matrix on
// the tensor cores, and the fp32 results are reduced to a group scale and packed E2M1 codes
// without leaving registers.  HBM traffic is the algorithmic minimum: 2 B/element in,
// 0.5 B/element + 1 scale byte per group out, plus the matrix once per CTA from L2.
//
// The contraction needs 2*32 flop per element (about 165 TFLOP/s at HBM speed), which is
// beyond the fp32 pipes but a small fraction of the tensor pipes, so the kernel uses
// warp-level bf16 MMAs.  Activations travel global -> shared (16-byte cp.async) -> registers
// (ldmatrix); the matrix fragments stay in registers.  One index permutation keeps the packing
// cheap: column 2q+i of n-tile j is assigned to output channel 8q+2j+i, so lane q (= lane % 4)
// ends up owning output channels 8q..8q+7 of the chunk -- 4 packed bytes, and the 4 lanes of a
// row own the chunk's 16 contiguous bytes.
//
// Work split: a CTA owns a slab of 8 chunks (256 channels, 512 B per row) and a range of
// rows; warp w owns chunk w and keeps that chunk's matrix fragments in 16 registers for the
// CTA's lifetime.  Packed codes and scale bytes of a 32-row tile are staged in shared memory
// and written out as full 128-byte lines (scattered 4-byte stores saturate the L1 data pipe).  Rows are walked 32 at a time; the activation loads run kStages-1 tiles ahead
// of the math into a warp-private shared-memory ring, which keeps ~100 KB per SM in flight without holding
// registers: one bulk tensor copy (TMA) per warp and tile in the production kernels, 16-byte cp.async copies
// per lane in the other variants (each lane then reads back exactly the bytes it requested, so that ring needs
// no barrier).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

#include "../../include/wush_b200.h"
#include "common.cuh"
#include "sm100.cuh"

namespace wush {

constexpr int kChunk = 32;          // channels per warp-chunk
constexpr int kWarps = 8;           // chunks per CTA slab
constexpr int kSlab = kChunk * kWarps;
constexpr int kTileRows = 32;       // rows per loop iteration

struct QuantParams {
  const __nv_bfloat16* x;
  const __nv_bfloat16* mat;
  int64_t mat_cols;                 // == cols (per-group) or == transform size (shared)
  const float* global_scale;        // NVFP4 only
  uint8_t* q;
  uint8_t* sf;
  float* transformed;               // debug variant only
  int64_t sf_cols;
  int sf_layout;
  int64_t ldx;                      // row stride of x in elements
  int64_t ldq;                      // row stride of q in bytes
  int64_t sf_group0;                // index of this call's first scale group inside the rows of sf (multiple of 4)
  int64_t rows, cols;
  int row_splits;                   // grid.y: CTAs sharing the rows of one slab
  int round_bf16;
  // optional prologue: x is replaced by bf16(bf16(x * row_scale[row]) * col_scale[col]) before the transform --
  // RMSNorm applied on the fly (row_scale = 1 / rms of the row, col_scale = the norm's weight), with the roundings
  // of the separate bf16 steps
  const float* row_scale;           // fp32 [rows] or null
  const __nv_bfloat16* col_scale;   // bf16 [cols] or null (both or none)
  uint8_t* clip_mask;               // quest only, optional: [rows, cols / 8], bit i of byte b = element 8b + i not clipped
};

__device__ __forceinline__ void mma_bf16_16816_zero(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                    uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%10,%10,%10,%10};\n"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 8 floats -> 8 E2M1 codes in one 32-bit word, v[0] in the lowest nibble.  Round to nearest
// even, saturating; NaN becomes +6 (code 7).
__device__ __forceinline__ uint32_t pack_e2m1x8(const float (&v)[8]) {
  uint32_t out;
  asm("{\n"
      ".reg .b8 b0, b1, b2, b3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n"
      "mov.b32 %0, {b0, b1, b2, b3};\n"
      "}\n"
      : "=r"(out)
      : "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]));
  return out;
}

__device__ __forceinline__ uint32_t e4m3_byte(float v) {
  uint16_t h;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;\n" : "=h"(h) : "f"(0.0f), "f"(v));
  return h & 0xFFu;
}

__device__ __forceinline__ float e4m3_value(uint32_t byte) {
  // exact decode of a non-negative E4M3 byte
  const uint32_t e = (byte >> 3) & 0xF, m = byte & 0x7;
  return e == 0 ? (float)m * 0.001953125f : __uint_as_float(((e + 120u) << 23) | (m << 20));
}

__device__ __forceinline__ float bf16_round(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}

__device__ __forceinline__ int64_t sf_offset(int layout, int64_t sf_cols, int64_t row, int64_t g) {
  if (layout == WUSH_SF_ROW_MAJOR) return row * sf_cols + g;
  return ((row >> 7) * (sf_cols >> 2) + (g >> 2)) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4 + (g & 3);
}

// Quantize the 8 values this lane holds for one row of one 32-channel chunk.
//   MX: the 4 lanes of the row share one scale.  NV: lanes {0,1} and {2,3} form two groups.
template <bool NV>
__device__ __forceinline__ void quantize_row(float (&v)[8], float gs, float gs6, uint32_t& packed,
                                             uint32_t& scale_byte) {
  float amax = fmaxf(fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3]))),
                     fmaxf(fmaxf(fabsf(v[4]), fabsf(v[5])), fmaxf(fabsf(v[6]), fabsf(v[7]))));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  if (!NV) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  float mul;
  if (!NV) {
    // E8M0 byte of RN(0.75 * amax): the fp32 exponent field for normal amax (0.75*m with m in
    // [1,2) rounds to 1 both ways), byte 1 for a subnormal strictly above 2^-127, else 0.
    uint32_t e = __float_as_uint(amax) >> 23;
    // multiplier 3 * 2^(127-e) = 1.5 * 2^(128-e); exact for e in 1..254
    mul = __uint_as_float(((255u - e) << 23) | 0x400000u);
    if (__builtin_expect(e - 1u >= 254u, 0)) {
      // e == 0 (zero / subnormal absmax): 3 * 2^127 overflows fp32, apply it in two exact steps;
      // e == 255: inf/NaN input poisons the group as in the reference
      if (e == 0) e = (amax * 0.75f > 5.877471754111438e-39f) ? 1u : 0u;
      const float pre = (e == 0) ? 1.8446744073709552e19f : (e == 1 ? 1.0f : 0.0f);  // 2^64
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] *= pre;
      mul = (e == 0) ? 2.7670116110564327e19f                                         // 3 * 2^63
                     : (e == 1 ? __uint_as_float((254u << 23) | 0x400000u) : __uint_as_float(0x7fc00000u));
    }
    scale_byte = e;
  } else {
    // gs6 = global_scale / 6 rounded once; the product differs from the oracle's float64
    // absmax * gs / 6 by one fp32 rounding, which can move the E4M3 byte only within ~1e-7
    // (relative) of a rounding boundary
    scale_byte = e4m3_byte(amax * gs6);
    // the oracle divides (x * gs / s); multiplying by the approximate quotient differs by two
    // ulp at most.  A zero scale gives inf, hence +-6 / NaN codes, as the oracle's division does.
    mul = __fdividef(gs, e4m3_value(scale_byte));
  }
  // packed fp32 multiplies: two products per instruction (each product is rounded on its own)
  const float2 m2 = make_float2(mul, mul);
#pragma unroll
  for (int i = 0; i < 8; i += 2) {
    const float2 pr = __fmul2_rn(make_float2(v[i], v[i + 1]), m2);
    v[i] = pr.x;
    v[i + 1] = pr.y;
  }
  packed = pack_e2m1x8(v);
  if (!NV && amax == 0.0f) packed = 0x88888888u;  // the reference encodes an all-zero group as -0
}

// "quest" scaling of one MXFP4 group (the 4 lanes of the row hold its 32 values): the shared exponent comes from
// the group's standard deviation, 2^floor(log2(c * std + 1e-8)) with c = 2.92247856 / 6, and values beyond +-6
// saturate.  Each fp32 operation is rounded on its own, in the order of the reference's Triton kernel
// (inference_lib/src/fp_quant/module/triton/mxfp4.py:64-74); only the order of the two 32-term sums differs.
// keep: bit i set when |v[i] / 2^e| < 6 (the reference's clip mask, ibid. :119-124).
constexpr float kQuestScale = (float)(2.92247856 / 6.0);
__device__ __forceinline__ void quantize_row_quest(float (&v)[8], uint32_t& packed, uint32_t& scale_byte,
                                                   uint32_t& keep) {
  float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    s1 = __fadd_rn(s1, v[i]);
    s2 = __fadd_rn(s2, __fmul_rn(v[i], v[i]));
  }
  s1 = __fadd_rn(s1, __shfl_xor_sync(0xffffffffu, s1, 1));
  s2 = __fadd_rn(s2, __shfl_xor_sync(0xffffffffu, s2, 1));
  s1 = __fadd_rn(s1, __shfl_xor_sync(0xffffffffu, s1, 2));
  s2 = __fadd_rn(s2, __shfl_xor_sync(0xffffffffu, s2, 2));
  const float mean = __fmul_rn(s1, 0.03125f), mean_sq = __fmul_rn(s2, 0.03125f);
  const float sd = __fsqrt_rn(__fsub_rn(mean_sq, __fmul_rn(mean, mean)));
  const float scale = __fadd_rn(__fmul_rn(kQuestScale, sd), 1e-8f);   // >= 1e-8: a normal number, or NaN / inf
  const uint32_t e = (__float_as_uint(scale) >> 23) & 0xFFu;          // biased floor(log2(scale)); 255 for NaN / inf
  scale_byte = e;
  // 2^(127 - e), exact for e <= 253; a NaN / inf scale poisons the group as the reference's division does
  const float mul = e >= 254u ? __uint_as_float(0x7fc00000u) : __uint_as_float((254u - e) << 23);
  keep = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    v[i] *= mul;
    keep |= (fabsf(v[i]) < 6.0f ? 1u : 0u) << i;
  }
  packed = pack_e2m1x8(v);
}

__device__ __forceinline__ void cp_async_16(uint32_t smem_addr, const void* gptr) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_addr), "l"(gptr) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

#ifndef WUSH_Q_STAGES
#define WUSH_Q_STAGES 3
#endif
#ifndef WUSH_Q_MINBLOCKS
#define WUSH_Q_MINBLOCKS 3
#endif
constexpr int kStages = WUSH_Q_STAGES;  // depth of the asynchronous activation ring (tiles)
constexpr int kStageBytes = 4 * kWarps * 32 * 16;
constexpr int kRingBytes = kStages * kStageBytes;
constexpr int kMatStride = kSlab + 8;           // bf16 elements per staged matrix row (528 B: odd multiple of 16 B)
constexpr int kMatBytes = 32 * kMatStride * 2;
constexpr int kOutRow = 144;                    // bytes per staged output row: 128 B of codes, stride keeps STS conflict-free
constexpr int kOutBytes = kTileRows * kOutRow;  // codes of one 32-row tile of the slab
constexpr int kSfRow = 16;                      // staged scale bytes per row (8 MX / 16 NV used)
constexpr int kSfBytes = kTileRows * kSfRow;
constexpr int kQuantSmem = kRingBytes + kMatBytes + 2 * (kOutBytes + kSfBytes);

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t smem_addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_addr));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t smem_addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_addr));
}

// set when a bounded wait on a bulk-copy barrier ran out (TMA variant); read and cleared by wush_fused_quantize_status
__device__ int g_quant_timeout = 0;

// RB: round transformed values to bf16 first.  BL: blocked scale layout.  DEBUG: also store
// the transformed values.  PRO: scale the activations by row_scale / col_scale first (see QuantParams).
// QUEST (MXFP4 only): standard-deviation scale with clipping instead of the absolute-maximum scale.
// W = 0: the transform is as wide as the quantization group (per-group or shared matrix).  W = 1, 2, 4: one dense
// square matrix of 32 W channels shared by every block of 32 W channels (Hadamard sizes 64 and 128, and 32 for
// NVFP4): the W warps of a block each contract all W chunks of the block, reading the other warps' activation tiles
// from the ring (one more block barrier per tile) and keeping W times the matrix fragments in registers.
// TMA: the activation tiles are fetched by one elected lane per warp with cp.async.bulk.tensor (a 32 x 32 box of
// the warp's chunk, 64-byte swizzle = the ring's layout) onto a per-warp, per-stage mbarrier, instead of by four
// cp.async per lane.
template <bool NV, bool DEBUG, bool RB, bool BL, bool PRO = false, bool QUEST = false, int W = 0, bool TMA = false>
__global__ void __launch_bounds__(kWarps * 32, W ? 1 : WUSH_Q_MINBLOCKS)
fused_quantize_kernel(const __grid_constant__ CUtensorMap xmap, const QuantParams p) {
  constexpr int TD = NV ? 16 : 32;       // quantization group (and transform size when W == 0)
  constexpr int GPC = kChunk / TD;       // scale groups per chunk
  constexpr int KC = W ? W : 1;          // chunks contracted per output chunk
  constexpr int kMatRows = W ? 32 * W : 32;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // [0, kRingBytes)   activation ring: per stage and warp a 32-row x 64-byte tile of the warp's chunk, the
  //                   16-byte pieces of a row XOR-swizzled by (row/2)%4 so ldmatrix reads without conflicts
  // then              the slab's matrices as 32 rows x (kSlab + 8) bf16, rows and columns permuted
  //                   into MMA fragment order (see below); NVFP4 chunks are block-diagonal 32x32
  // then              two staging buffers for a tile's packed codes and scale bytes
  __nv_bfloat16* smat = reinterpret_cast<__nv_bfloat16*>(smem_raw + kRingBytes);
  uint8_t* sout = smem_raw + kRingBytes + kMatRows * kMatStride * 2;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, q4 = lane & 3;
  const int64_t slab_col0 = (int64_t)blockIdx.x * kSlab;
  const int64_t col0 = slab_col0 + warp * kChunk;
  const bool shared_mat = W == 0 && p.mat_cols == TD;

  // even split of the 32-row tiles over the row splits (every split gets at least one tile)
  const int tiles_total = (int)((p.rows + kTileRows - 1) / kTileRows);
  const int tile_begin = (int)((int64_t)blockIdx.y * tiles_total / p.row_splits);
  const int tile_end = (int)((int64_t)(blockIdx.y + 1) * tiles_total / p.row_splits);
  const int row_begin = tile_begin * kTileRows;
  const int row_end = min(tile_end * kTileRows, (int)p.rows);
  const int last_row = (int)p.rows - 1;
  const int n_tiles = tile_end - tile_begin;
  const bool active = col0 < p.cols;     // warps past the last chunk of a partial slab only help with stores

  // ---- start the activation pipeline before touching the matrix ------------------------
  const __nv_bfloat16* xcol = p.x + col0 + 8 * q4;
  const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem_raw);
  // this lane copies piece q4 of rows g, g+8, g+16, g+24 of every tile
  const uint32_t ring_wr = smem_base + warp * (kStageBytes / kWarps) + g * 64 + ((q4 ^ ((g >> 1) & 3)) << 4);
  // Tiles are issued strictly in order, so the producer side keeps a running stage offset, a running
  // row and a running source pointer instead of multiplying per tile.
  uint32_t issue_stage_off = 0;
  int issue_row = row_begin + g;                                   // first of this lane's 4 rows of the next tile
  const __nv_bfloat16* issue_ptr = xcol + (int64_t)issue_row * p.ldx;
  const int64_t row8 = 8 * p.ldx, row32 = 32 * p.ldx;             // element strides of 8 and 32 rows
  // TMA variant: barriers [stage][warp] behind the staging buffers, then the CTA's abort word
  constexpr int kTailOff = kRingBytes + kMatRows * kMatStride * 2 + 2 * (kOutBytes + kSfBytes);
  const uint32_t bar0 = smem_base + kTailOff + warp * 8;
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem_raw + kTailOff + kStages * kWarps * 8);
  if (TMA) {
    // the swizzle of a bulk tensor copy follows the shared-memory address bits (period 512 bytes): the ring must
    // start on such a boundary for the copies to land in the layout the ldmatrix offsets assume
    if (smem_base & 511u) {
      if (threadIdx.x == 0) atomicExch(&g_quant_timeout, 2);
      return;
    }
    if (threadIdx.x == 0) *abort_flag = 0;
    if (lane == 0) {
#pragma unroll
      for (int st = 0; st < kStages; ++st) sm100::mbar_init(bar0 + st * kWarps * 8, 1);
      sm100::mbar_init_fence();
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      sm100::tma_prefetch_desc(&xmap);
    }
    __syncwarp();
  }
  int issue_stage = 0;
  auto issue_tile = [&](int t) {
    if (TMA) {
      if (active && t < n_tiles && lane == 0) {
        const uint32_t bar = bar0 + issue_stage * kWarps * 8;
        sm100::mbar_arrive_expect_tx(bar, kStageBytes / kWarps);
        sm100::tma_load_2d(smem_base + issue_stage * kStageBytes + warp * (kStageBytes / kWarps), &xmap, (int)col0,
                           row_begin + t * kTileRows, bar);
      }
      issue_stage = issue_stage + 1 == kStages ? 0 : issue_stage + 1;
      return;
    }
    if (active && t < n_tiles) {
      const uint32_t dst = ring_wr + issue_stage_off;
      if (issue_row + 24 <= last_row) {
#pragma unroll
        for (int i = 0; i < 4; ++i) cp_async_16(dst + i * (8 * 64), issue_ptr + i * row8);
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int r = min(issue_row + 8 * i, last_row);  // clamp: rows past the end are discarded later
          cp_async_16(dst + i * (8 * 64), xcol + (int64_t)r * p.ldx);
        }
      }
      issue_row += kTileRows;
      issue_ptr += row32;
      issue_stage_off = issue_stage_off + kStageBytes == kRingBytes ? 0u : issue_stage_off + kStageBytes;
    }
    cp_async_commit();
  };
#pragma unroll
  for (int t = 0; t < kStages - 1; ++t) issue_tile(t);

  // ---- stage the slab's matrices in fragment order ---------------------------------------
  // Matrix element M[k][n] of a chunk (k: input channel, n: output channel, both 0..31) goes to
  // smem row k and column 8j + 2b + c for n = 8b + 2j + c.  An 8x8 tile (rows 16ks + 8h ..,
  // columns 8j ..) read with ldmatrix.trans then hands lane (g, q) the pair
  // M[16ks+8h+2q+{0,1}][8(g/2)+2j+(g%2)]: the B fragment of the column-permuted MMA described at
  // the top of this file.
  if (W) {
    // dense (32 W) x (32 W) matrix: every 32 x 32 sub-block goes into the same permuted layout
    constexpr int n = 32 * KC, vec_per_row = n / 8;
    for (int idx = threadIdx.x; idx < n * vec_per_row; idx += blockDim.x) {
      const int km = idx / vec_per_row, n8 = (idx % vec_per_row) * 8;
      const uint4 v = *reinterpret_cast<const uint4*>(p.mat + (int64_t)km * n + n8);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j)
        *reinterpret_cast<uint32_t*>(&smat[km * kMatStride + (n8 & ~31) + 8 * j + 2 * ((n8 & 31) >> 3)]) = w[j];
    }
  } else {
    const int ncols = shared_mat ? TD : kSlab;
    const int vec_per_row = ncols / 8;
    for (int idx = threadIdx.x; idx < TD * vec_per_row; idx += blockDim.x) {
      const int km = idx / vec_per_row;          // row of the given matrix
      const int n8 = (idx % vec_per_row) * 8;    // first of 8 consecutive columns
      uint4 v = make_uint4(0, 0, 0, 0);
      if (shared_mat || slab_col0 + n8 < p.cols)
        v = *reinterpret_cast<const uint4*>(p.mat + (int64_t)km * p.mat_cols + (shared_mat ? 0 : slab_col0) + n8);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
      // NVFP4: the 16x16 block of output group (n8/16) sits on the diagonal of the 32x32 chunk matrix
      const int half = NV ? ((n8 >> 4) & 1) : 0;
      const int k = km + 16 * half;
      const int srow = k;
      const int chunk_col0 = NV && shared_mat ? 0 : (n8 & ~31);  // column base of the chunk inside smat
      const int nb = NV && shared_mat ? n8 : (n8 & 31);          // first n inside the chunk (0, 8, 16, 24)
#pragma unroll
      for (int j = 0; j < 4; ++j) {              // w[j] holds n = nb + 2j + {0,1}
        const int scol = chunk_col0 + 8 * j + 2 * (nb >> 3);
        if (NV && shared_mat) {
          // one shared 16x16 matrix serves both diagonal blocks of the chunk
#pragma unroll
          for (int blk = 0; blk < 2; ++blk) {
            const int kk = km + 16 * blk;
            const int sr = kk;
            const int sc = 8 * j + 2 * ((nb + 16 * blk) >> 3);
            *reinterpret_cast<uint32_t*>(&smat[sr * kMatStride + sc]) = w[j];
            const int kz = km + 16 * (1 - blk);
            const int srz = kz;
            *reinterpret_cast<uint32_t*>(&smat[srz * kMatStride + sc]) = 0u;
          }
        } else {
          *reinterpret_cast<uint32_t*>(&smat[srow * kMatStride + scol]) = w[j];
          if (NV) {
            const int kz = km + 16 * (1 - half);
            const int srz = kz;
            *reinterpret_cast<uint32_t*>(&smat[srz * kMatStride + scol]) = 0u;
          }
        }
      }
    }
  }
  __syncthreads();

  // ---- this lane's matrix fragments: bfrag[j][ks][h] ---------------------------------------
  uint32_t bfrag[KC][4][2][2];
  {
    // W: this warp's output chunk is chunk (warp % W) of its block; input chunk kc supplies rows 32 kc .. 32 kc + 31
    const int cbase = W ? (warp % KC) * kChunk : (shared_mat ? 0 : warp * kChunk);
#pragma unroll
    for (int kc = 0; kc < KC; ++kc) {
#pragma unroll
      for (int ks = 0; ks < 2; ++ks) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t r[4];
          const int srow = 32 * kc + 16 * ks + 8 * h + (lane & 7);
          const int scol = cbase + 8 * (lane >> 3);
          ldmatrix_x4_trans(r, smem_base + kRingBytes + (srow * kMatStride + scol) * 2);
#pragma unroll
          for (int j = 0; j < 4; ++j) bfrag[kc][j][ks][h] = r[j];
        }
      }
    }
  }

  const float gs = NV ? *p.global_scale : 0.0f;
  const float gs6 = gs / 6.0f;
  // prologue: this lane's column factors, bf16 pairs for channels 16ks + 8h + 2q + {0,1} of the chunk
  uint32_t gam[2][2] = {{0, 0}, {0, 0}};
  if (PRO && active) {
#pragma unroll
    for (int ks = 0; ks < 2; ++ks)
#pragma unroll
      for (int h = 0; h < 2; ++h)
        gam[ks][h] = *reinterpret_cast<const uint32_t*>(p.col_scale + col0 + 16 * ks + 8 * h + 2 * q4);
  }
  float* tp = DEBUG ? p.transformed + (int64_t)(row_begin + g) * p.cols + col0 + 8 * q4 : nullptr;
  const int64_t q_stride = p.ldq;
  // store phase: thread t writes 16 bytes of codes of row t/8, segment t%8 (= chunk) of the slab
  const int st_row = threadIdx.x >> 3, st_seg = threadIdx.x & 7;
  const bool st_ok = slab_col0 + st_seg * kChunk < p.cols;
  uint8_t* q_dst = p.q + (int64_t)(row_begin + st_row) * q_stride + (slab_col0 >> 1) + st_seg * 16;
  const int sf_slab0 = (int)(slab_col0 / TD);           // first scale group of the slab (inside this call's columns)
  const int sf_total = (int)(p.cols / TD);
  const int64_t sf_g0 = p.sf_group0;                    // where this call's groups start inside a row of sf

  // loop-invariant ldmatrix offsets inside a stage: [mt][ks]
  uint32_t a_off[2][2];
  {
    const int arow = (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {
      const int r = arow + 16 * mt;
      const int sw = (r >> 1) & 3;
#pragma unroll
      for (int ks = 0; ks < 2; ++ks)
        a_off[mt][ks] = warp * (kStageBytes / kWarps) + r * 64 + ((((lane >> 4) + 2 * ks) ^ sw) << 4);
    }
  }
  uint32_t use_stage_off = 0;
  const int64_t q_tile_stride = (int64_t)kTileRows * q_stride;
  // staging offsets of this lane's 4 rows of a tile
  const int out_q_lane = g * kOutRow + warp * 16 + q4 * 4;
  const int out_sf_lane = g * kSfRow + (NV ? warp * 2 + (q4 >> 1) : warp);
  const bool sf_writer = NV ? (q4 & 1) == 0 : q4 == 0;

  for (int t = 0; t < n_tiles; ++t) {
    issue_tile(t + kStages - 1);
    if (TMA) {
      // tile t sits in stage t % kStages; its barrier completes phase (t / kStages) & 1.  A wait that runs out
      // raises the CTA's abort word (every later wait then returns at once) and the kernel reports it.
      if (active) sm100::mbar_wait(bar0 + (t % kStages) * kWarps * 8, (uint32_t)(t / kStages) & 1u, abort_flag);
    } else {
      cp_async_wait<kStages - 1>();
    }
    const int r0 = row_begin + t * kTileRows;
    uint8_t* out_q = sout + (t & 1) * (kOutBytes + kSfBytes);
    uint8_t* out_sf = out_q + kOutBytes;

    if (W) __syncthreads();  // the tile's chunks were copied by eight different warps
    if (active) {
      if (!W) __syncwarp();  // the tile was copied by all lanes of this warp
      // A fragments: rows (lane%8) + 8*((lane/8)%2) of a 16-row tile, 16-byte piece (lane/16) + 2ks
      const uint32_t tile = smem_base + use_stage_off;
      use_stage_off = use_stage_off + kStageBytes == kRingBytes ? 0u : use_stage_off + kStageBytes;
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {  // two 16-row MMA tiles: rows g+16mt and g+8+16mt
        uint32_t a0[4], a1[4];
        // W: start with the first chunk of this warp's block (the ring regions of the warps are kStageBytes / kWarps apart)
        const uint32_t tile0 = W ? tile - (warp % KC) * (kStageBytes / kWarps) : tile;
        ldmatrix_x4(a0, tile0 + a_off[mt][0]);
        ldmatrix_x4(a1, tile0 + a_off[mt][1]);
        if (PRO) {
          // registers 0/2 hold row g + 16mt, registers 1/3 row g + 8 + 16mt; 0/1 channels 2q.., 2/3 channels 8 + 2q..
          const float rs0 = p.row_scale[min(r0 + g + 16 * mt, last_row)];
          const float rs1 = p.row_scale[min(r0 + g + 8 + 16 * mt, last_row)];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float rs = (i & 1) ? rs1 : rs0;
            float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a0[i]));
            __nv_bfloat162 r = __floats2bfloat162_rn(f.x * rs, f.y * rs);
            r = __hmul2(r, *reinterpret_cast<const __nv_bfloat162*>(&gam[0][i >> 1]));
            a0[i] = *reinterpret_cast<const uint32_t*>(&r);
            f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a1[i]));
            r = __floats2bfloat162_rn(f.x * rs, f.y * rs);
            r = __hmul2(r, *reinterpret_cast<const __nv_bfloat162*>(&gam[1][i >> 1]));
            a1[i] = *reinterpret_cast<const uint32_t*>(&r);
          }
        }
        float acc[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          mma_bf16_16816_zero(acc[j], a0[0], a0[1], a0[2], a0[3], bfrag[0][j][0][0], bfrag[0][j][0][1]);
          mma_bf16_16816(acc[j], a1[0], a1[1], a1[2], a1[3], bfrag[0][j][1][0], bfrag[0][j][1][1]);
        }
#pragma unroll
        for (int kc = 1; kc < KC; ++kc) {  // the other chunks of the block (wide matrices only)
          ldmatrix_x4(a0, tile0 + kc * (kStageBytes / kWarps) + a_off[mt][0]);
          ldmatrix_x4(a1, tile0 + kc * (kStageBytes / kWarps) + a_off[mt][1]);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            mma_bf16_16816(acc[j], a0[0], a0[1], a0[2], a0[3], bfrag[kc][j][0][0], bfrag[kc][j][0][1]);
            mma_bf16_16816(acc[j], a1[0], a1[1], a1[2], a1[3], bfrag[kc][j][1][0], bfrag[kc][j][1][1]);
          }
        }
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int trow = g + 8 * (half + 2 * mt);  // row inside the tile
          float v[8];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            v[2 * j] = acc[j][2 * half];
            v[2 * j + 1] = acc[j][2 * half + 1];
          }
          if (RB) {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = bf16_round(v[i]);
          }
          if (DEBUG && r0 + trow < row_end) {
            float* t4 = tp + (int64_t)(t * kTileRows + trow - g) * p.cols;
            *reinterpret_cast<float4*>(t4) = make_float4(v[0], v[1], v[2], v[3]);
            *reinterpret_cast<float4*>(t4 + 4) = make_float4(v[4], v[5], v[6], v[7]);
          }
          uint32_t packed, sbyte;
          if (QUEST) {
            uint32_t keep;
            quantize_row_quest(v, packed, sbyte, keep);
            if (p.clip_mask != nullptr && r0 + trow < row_end)
              p.clip_mask[(int64_t)(r0 + trow) * (p.cols >> 3) + ((col0 + 8 * q4) >> 3)] = (uint8_t)keep;
          } else {
            quantize_row<NV>(v, gs, gs6, packed, sbyte);
          }
          *reinterpret_cast<uint32_t*>(out_q + out_q_lane + (trow - g) * kOutRow) = packed;
          if (sf_writer) out_sf[out_sf_lane + (trow - g) * kSfRow] = (uint8_t)sbyte;
        }
      }
    }
    __syncthreads();  // the tile's codes and scales are staged (buffers alternate, one barrier per tile)

    // ---- coalesced stores: each row of the slab is 128 contiguous bytes of codes ------------
    if (st_ok && r0 + st_row < row_end) {
      const uint4 v = *reinterpret_cast<const uint4*>(out_q + st_row * kOutRow + st_seg * 16);
      *reinterpret_cast<uint4*>(q_dst) = v;
    }
    q_dst += q_tile_stride;
    if (warp == 0) {
      const int row = r0 + lane;
      if (row < row_end) {
        constexpr int NG = kWarps * GPC;          // scale groups per slab row: 8 (MX) or 16 (NV)
        const uint32_t* sv = reinterpret_cast<const uint32_t*>(out_sf + lane * kSfRow);
#pragma unroll
        for (int c = 0; c < NG / 4; ++c) {        // 4 consecutive groups = one 32-bit word
          const int grp = sf_slab0 + 4 * c;
          if (grp >= sf_total) break;
          const uint32_t word = sv[c];
          uint8_t* dst;
          if (BL) {
            dst = p.sf + ((int64_t)(row >> 7) * (p.sf_cols >> 2) + ((sf_g0 + grp) >> 2)) * 512 + (row & 31) * 16 +
                  ((row >> 5) & 3) * 4;
          } else {
            dst = p.sf + (int64_t)row * p.sf_cols + sf_g0 + grp;
          }
          if (grp + 4 <= sf_total) {
            *reinterpret_cast<uint32_t*>(dst) = word;
          } else {
            for (int b = 0; grp + b < sf_total; ++b) dst[b] = (uint8_t)(word >> (8 * b));
          }
        }
      }
    }
  }
  if (TMA && threadIdx.x == 0 && *abort_flag) atomicExch(&g_quant_timeout, 1);
}

// Grid: x = slabs, y = row splits.  Every CTA takes an equal share (+-1) of the 32-row tiles.
// The number of row splits is the largest that keeps all CTAs co-resident in `waves` waves of
// (SMs x CTAs per SM), so the last wave is not a mostly empty tail.
template <bool NV, bool DEBUG, bool RB, bool BL, bool PRO = false, bool QUEST = false, int W = 0, bool TMA = false>
static int launch_quant_t(QuantParams p, cudaStream_t stream) {
  const int64_t slabs = (p.cols + kSlab - 1) / kSlab;
  const int64_t tiles = (p.rows + kTileRows - 1) / kTileRows;
  // Waves of resident CTAs: narrow matrices (few slabs) do best in a single wave, wide ones in three
  // (measured at 16384 rows: 4096 channels 4470/4240/3970 GB/s for 1/2/3 waves, 14336 channels
  // 4930/5170/5200).  WUSH_B200_QUANT_WAVES overrides the choice.
  static const int waves_env = env_int("WUSH_B200_QUANT_WAVES", 0);
  const int waves = waves_env > 0 ? waves_env : (slabs <= 16 ? 1 : (slabs <= 32 ? 2 : 3));
  const int64_t resident = (int64_t)sm_count() * (W ? 1 : WUSH_Q_MINBLOCKS);
  int64_t splits = (resident * waves) / slabs;
  if (splits < 1) splits = 1;
  if (splits > tiles) splits = tiles;
  if (splits > 65535) splits = 65535;
  p.row_splits = (int)splits;
  dim3 grid((unsigned)slabs, (unsigned)splits);
  auto kern = fused_quantize_kernel<NV, DEBUG, RB, BL, PRO, QUEST, W, TMA>;
  constexpr int smem = kQuantSmem + (W ? (32 * W - 32) * kMatStride * 2 : 0) + (TMA ? kStages * kWarps * 8 + 16 : 0);
  static PerDevice attr_set;     // per instantiation and device
  int rc = opt_in_smem(attr_set, kern, smem);
  if (rc != 0) return rc;
  CUtensorMap xmap = {};
  if (TMA) {
    // x as [rows][cols] bf16 with row stride ldx; box = one warp's 32 x 32 tile; 64-byte swizzle = the ring's layout
    rc = make_tensor_map_2d(&xmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.x, (uint64_t)p.rows, (uint64_t)p.cols,
                            (uint64_t)p.ldx * 2, kChunk, kTileRows, CU_TENSOR_MAP_SWIZZLE_64B);
    if (rc != 0) return rc;
  }
  kern<<<grid, kWarps * 32, smem, stream>>>(xmap, p);
  return (int)cudaGetLastError();
}

template <bool NV, bool DEBUG>
static int launch_quant(const QuantParams& p, cudaStream_t stream) {
  if (const int rc100 = require_sm100()) return rc100;
  const bool rb = p.round_bf16 != 0, bl = p.sf_layout == WUSH_SF_BLOCKED;
  static const int use_tma = env_int("WUSH_B200_QUANT_TMA", 1);   // 0: the cp.async ring everywhere
  if (p.row_scale != nullptr) {
    // the prologue exists for the production path only (no bf16 rounding of the transformed values, no debug output)
    if (DEBUG || rb) return WUSH_ERR_BAD_FLAG;
    if (use_tma && p.ldx % 8 == 0)
      return bl ? launch_quant_t<NV, false, false, true, true, false, 0, true>(p, stream)
                : launch_quant_t<NV, false, false, false, true, false, 0, true>(p, stream);
    return bl ? launch_quant_t<NV, false, false, true, true>(p, stream) : launch_quant_t<NV, false, false, false, true>(p, stream);
  }
  if (rb) return bl ? launch_quant_t<NV, DEBUG, true, true>(p, stream) : launch_quant_t<NV, DEBUG, true, false>(p, stream);
  if (!DEBUG && use_tma && p.ldx % 8 == 0)
    return bl ? launch_quant_t<NV, false, false, true, false, false, 0, true>(p, stream)
              : launch_quant_t<NV, false, false, false, false, false, 0, true>(p, stream);
  return bl ? launch_quant_t<NV, DEBUG, false, true>(p, stream) : launch_quant_t<NV, DEBUG, false, false>(p, stream);
}

static int check_quant_args(bool nv, const void* x, const void* mat, int64_t mat_cols, const float* gs,
                            const uint8_t* q, const uint8_t* sf, int64_t sf_cols, int sf_layout,
                            int64_t rows, int64_t cols, int flags) {
  const int g = nv ? 16 : 32;
  if (!x || !mat || !q || !sf || (nv && !gs)) return WUSH_ERR_NULL_POINTER;
  if (rows < 0 || cols <= 0 || cols % 32 != 0) return WUSH_ERR_BAD_SHAPE;
  if (flags & ~(WUSH_QUANT_ROUND_BF16 | WUSH_QUANT_WIDE_MATRIX)) return WUSH_ERR_BAD_FLAG;
  if (flags & WUSH_QUANT_WIDE_MATRIX) {
    // one square matrix of mat_cols channels, wider than (or, for NVFP4, twice) the quantization group
    if (flags & WUSH_QUANT_ROUND_BF16) return WUSH_ERR_BAD_FLAG;
    if (mat_cols != 64 && mat_cols != 128 && !(nv && mat_cols == 32)) return WUSH_ERR_BAD_SHAPE;
    if (cols % mat_cols != 0) return WUSH_ERR_BAD_SHAPE;
    if ((uintptr_t)mat & 15) return WUSH_ERR_BAD_ALIGNMENT;
  } else if (mat_cols != cols && mat_cols != g) {
    return WUSH_ERR_BAD_SHAPE;
  }
  if (sf_cols % 4 != 0 || sf_cols < cols / g) return WUSH_ERR_BAD_SHAPE;
  if (sf_layout != WUSH_SF_ROW_MAJOR && sf_layout != WUSH_SF_BLOCKED) return WUSH_ERR_BAD_FLAG;
  if (((uintptr_t)x & 15) || ((uintptr_t)q & 15) || ((uintptr_t)sf & 3)) return WUSH_ERR_BAD_ALIGNMENT;
  if (mat_cols == cols && ((uintptr_t)mat & 15)) return WUSH_ERR_BAD_ALIGNMENT;
  return WUSH_OK;
}

// Wide shared matrices (WUSH_QUANT_WIDE_MATRIX): production instantiations only.
template <bool NV, bool QUEST>
static int launch_quant_wide(const QuantParams& p, cudaStream_t stream) {
  if (const int rc100 = require_sm100()) return rc100;
  const bool bl = p.sf_layout == WUSH_SF_BLOCKED;
  switch (p.mat_cols) {
    case 32:
      if (!NV) return WUSH_ERR_BAD_SHAPE;
      return bl ? launch_quant_t<NV, false, false, true, false, QUEST, NV ? 1 : 2>(p, stream)
                : launch_quant_t<NV, false, false, false, false, QUEST, NV ? 1 : 2>(p, stream);
    case 64:
      return bl ? launch_quant_t<NV, false, false, true, false, QUEST, 2>(p, stream)
                : launch_quant_t<NV, false, false, false, false, QUEST, 2>(p, stream);
    case 128:
      return bl ? launch_quant_t<NV, false, false, true, false, QUEST, 4>(p, stream)
                : launch_quant_t<NV, false, false, false, false, QUEST, 4>(p, stream);
    default:
      return WUSH_ERR_BAD_SHAPE;
  }
}

int quantize_timeout_fetch_and_clear() {
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_quant_timeout, sizeof(int));
  if (e != cudaSuccess) return (int)e;
  if (v == 0) return 0;
  const int zero = 0;
  e = cudaMemcpyToSymbol(g_quant_timeout, &zero, sizeof(int));
  return e != cudaSuccess ? (int)e : WUSH_ERR_DEVICE_TIMEOUT;
}

}  // namespace wush

using namespace wush;

extern "C" int wush_fused_quantize_mx(const void* x, const void* mat, int64_t mat_cols, uint8_t* q, uint8_t* sf,
                                      int64_t sf_cols, int sf_layout, int64_t rows, int64_t cols, int flags,
                                      void* stream) {
  int rc = check_quant_args(false, x, mat, mat_cols, nullptr, q, sf, sf_cols, sf_layout, rows, cols, flags);
  if (rc != WUSH_OK) return rc;
  if (rows == 0) return WUSH_OK;
  QuantParams p{(const __nv_bfloat16*)x, (const __nv_bfloat16*)mat, mat_cols, nullptr, q, sf, nullptr,
                sf_cols, sf_layout, cols, cols / 2, 0, rows, cols, 0, (flags & WUSH_QUANT_ROUND_BF16) ? 1 : 0, nullptr, nullptr};
  if (flags & WUSH_QUANT_WIDE_MATRIX) return launch_quant_wide<false, false>(p, (cudaStream_t)stream);
  return launch_quant<false, false>(p, (cudaStream_t)stream);
}

extern "C" int wush_fused_quantize_mx_quest(const void* x, const void* mat, int64_t mat_cols, uint8_t* q, uint8_t* sf,
                                            int64_t sf_cols, int sf_layout, uint8_t* clip_mask, int64_t rows,
                                            int64_t cols, int flags, void* stream) {
  int rc = check_quant_args(false, x, mat, mat_cols, nullptr, q, sf, sf_cols, sf_layout, rows, cols, flags);
  if (rc != WUSH_OK) return rc;
  if (rows == 0) return WUSH_OK;
  if (const int rc100 = require_sm100()) return rc100;
  QuantParams p{(const __nv_bfloat16*)x, (const __nv_bfloat16*)mat, mat_cols, nullptr, q, sf, nullptr,
                sf_cols, sf_layout, cols, cols / 2, 0, rows, cols, 0, (flags & WUSH_QUANT_ROUND_BF16) ? 1 : 0, nullptr, nullptr,
                clip_mask};
  if (flags & WUSH_QUANT_WIDE_MATRIX) return launch_quant_wide<false, true>(p, (cudaStream_t)stream);
  const bool bl = sf_layout == WUSH_SF_BLOCKED;
  if (p.round_bf16)
    return bl ? launch_quant_t<false, false, true, true, false, true>(p, (cudaStream_t)stream)
              : launch_quant_t<false, false, true, false, false, true>(p, (cudaStream_t)stream);
  return bl ? launch_quant_t<false, false, false, true, false, true>(p, (cudaStream_t)stream)
            : launch_quant_t<false, false, false, false, false, true>(p, (cudaStream_t)stream);
}

extern "C" int wush_fused_quantize_nv(const void* x, const void* mat, int64_t mat_cols, const float* global_scale,
                                      uint8_t* q, uint8_t* sf, int64_t sf_cols, int sf_layout, int64_t rows,
                                      int64_t cols, int flags, void* stream) {
  int rc = check_quant_args(true, x, mat, mat_cols, global_scale, q, sf, sf_cols, sf_layout, rows, cols, flags);
  if (rc != WUSH_OK) return rc;
  if (rows == 0) return WUSH_OK;
  QuantParams p{(const __nv_bfloat16*)x, (const __nv_bfloat16*)mat, mat_cols, global_scale, q, sf, nullptr,
                sf_cols, sf_layout, cols, cols / 2, 0, rows, cols, 0, (flags & WUSH_QUANT_ROUND_BF16) ? 1 : 0, nullptr, nullptr};
  if (flags & WUSH_QUANT_WIDE_MATRIX) return launch_quant_wide<true, false>(p, (cudaStream_t)stream);
  return launch_quant<true, false>(p, (cudaStream_t)stream);
}

extern "C" int wush_fused_quantize_debug(int fmt, const void* x, const void* mat, int64_t mat_cols,
                                         const float* global_scale, uint8_t* q, uint8_t* sf, int64_t sf_cols,
                                         int sf_layout, float* transformed, int64_t rows, int64_t cols, int flags,
                                         void* stream) {
  if (fmt != 0 && fmt != 1) return WUSH_ERR_BAD_FLAG;
  if (!transformed) return WUSH_ERR_NULL_POINTER;
  int rc = check_quant_args(fmt == 1, x, mat, mat_cols, global_scale, q, sf, sf_cols, sf_layout, rows, cols, flags);
  if (rc != WUSH_OK) return rc;
  if ((uintptr_t)transformed & 15) return WUSH_ERR_BAD_ALIGNMENT;
  if (flags & WUSH_QUANT_WIDE_MATRIX) return WUSH_ERR_BAD_FLAG;
  if (rows == 0) return WUSH_OK;
  QuantParams p{(const __nv_bfloat16*)x, (const __nv_bfloat16*)mat, mat_cols, global_scale, q, sf, transformed,
                sf_cols, sf_layout, cols, cols / 2, 0, rows, cols, 0, (flags & WUSH_QUANT_ROUND_BF16) ? 1 : 0, nullptr, nullptr};
  return fmt == 1 ? launch_quant<true, true>(p, (cudaStream_t)stream)
                  : launch_quant<false, true>(p, (cudaStream_t)stream);
}

extern "C" int wush_fused_quantize_strided(int format, const void* x, int64_t ldx, const void* mat, int64_t mat_cols,
                                           const float* global_scale, uint8_t* q, int64_t ldq, uint8_t* sf,
                                           int64_t sf_cols, int sf_layout, int64_t sf_group0, const float* row_scale,
                                           const void* col_scale, int64_t rows, int64_t cols, int flags, void* stream) {
  if (format != WUSH_FORMAT_MXFP4 && format != WUSH_FORMAT_NVFP4) return WUSH_ERR_BAD_FLAG;
  const bool nv = format == WUSH_FORMAT_NVFP4;
  const int g = nv ? 16 : 32;
  if (!x || !mat || !q || !sf || (nv && !global_scale)) return WUSH_ERR_NULL_POINTER;
  if (rows < 0 || cols <= 0 || cols % 32 != 0) return WUSH_ERR_BAD_SHAPE;
  if (mat_cols != cols && mat_cols != g) return WUSH_ERR_BAD_SHAPE;
  if (ldx < cols || ldx % 8 != 0 || ldq < cols / 2 || ldq % 16 != 0) return WUSH_ERR_BAD_SHAPE;
  if (sf_group0 < 0 || sf_group0 % 4 != 0 || sf_cols % 4 != 0 || sf_cols < sf_group0 + cols / g) return WUSH_ERR_BAD_SHAPE;
  if (sf_layout != WUSH_SF_ROW_MAJOR && sf_layout != WUSH_SF_BLOCKED) return WUSH_ERR_BAD_FLAG;
  if (flags & ~WUSH_QUANT_ROUND_BF16) return WUSH_ERR_BAD_FLAG;
  if (((uintptr_t)x & 15) || ((uintptr_t)q & 15) || ((uintptr_t)sf & 3)) return WUSH_ERR_BAD_ALIGNMENT;
  if (mat_cols == cols && ((uintptr_t)mat & 15)) return WUSH_ERR_BAD_ALIGNMENT;
  if ((row_scale == nullptr) != (col_scale == nullptr)) return WUSH_ERR_NULL_POINTER;
  if (((uintptr_t)row_scale & 3) || ((uintptr_t)col_scale & 3)) return WUSH_ERR_BAD_ALIGNMENT;
  if (rows == 0) return WUSH_OK;
  QuantParams p{(const __nv_bfloat16*)x, (const __nv_bfloat16*)mat, mat_cols, global_scale, q, sf, nullptr,
                sf_cols, sf_layout, ldx, ldq, sf_group0, rows, cols, 0, (flags & WUSH_QUANT_ROUND_BF16) ? 1 : 0,
                row_scale, (const __nv_bfloat16*)col_scale};
  return nv ? launch_quant<true, false>(p, (cudaStream_t)stream) : launch_quant<false, false>(p, (cudaStream_t)stream);
}
