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
// warp-level bf16 MMAs with operand fragments held in registers.  Two index permutations
// make every global access a full 16-byte vector:
//   * contraction index: lane q (= lane % 4) of a fragment row loads channels 8q..8q+7 of
//     the chunk with one 16-byte load and feeds them to the MMA's k slots
//     {2q, 2q+1, 2q+8, 2q+9} of two consecutive k-steps; the matrix fragments use the same
//     permutation, so the product is unchanged;
//   * output index: column 2q+i of n-tile j is assigned to output channel 8q+2j+i, so lane
//     q ends up owning output channels 8q..8q+7 of the chunk -- 4 packed bytes, and the 4
//     lanes of a row own the chunk's 16 contiguous bytes.
//
// Work split: a CTA owns a slab of 8 chunks (256 channels, 512 B per row) and a range of
// rows; warp w owns chunk w and keeps that chunk's matrix fragments in 16 registers for the
// CTA's lifetime.  Rows are walked 32 at a time with the next tile's loads issued before the
// current tile's math (register double buffering).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/wush_b200.h"
#include "common.cuh"

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
  int64_t rows, cols;
  int64_t rows_per_cta;
  int round_bf16;
};

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 8 floats -> 8 E2M1 codes in one 32-bit word, v[0] in the lowest nibble.  Round to nearest
// even, saturating; NaN becomes +6 (code 7).
__device__ __forceinline__ uint32_t pack_e2m1x8(const float (&v)[8]) {
  uint32_t out;
  asm volatile(
      "{\n"
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
  asm volatile("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;\n" : "=h"(h) : "f"(0.0f), "f"(v));
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
__device__ __forceinline__ void quantize_row(float (&v)[8], float gs, int q4, uint32_t& packed,
                                             uint32_t& scale_byte) {
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  if (!NV) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  float mul;
  if (!NV) {
    // E8M0 byte of RN(0.75 * amax): the fp32 exponent field for normal amax (0.75*m with m in
    // [1,2) rounds to 1 both ways), byte 1 for a subnormal strictly above 2^-127, else 0.
    const uint32_t bits = __float_as_uint(amax);
    uint32_t e = bits >> 23;
    if (e == 0) e = (amax * 0.75f > 5.877471754111438e-39f) ? 1u : 0u;
    scale_byte = e;
    // multiplier 3 * 2^(127-e) = 1.5 * 2^(128-e); exact for e in 1..254
    mul = __uint_as_float(((255u - e) << 23) | 0x400000u);
    if (e == 0 || e == 255u) {
      // e == 0: 3 * 2^127 overflows fp32, apply it in two exact steps; e == 255: inf/NaN input
      const float pre = (e == 0) ? 1.8446744073709552e19f : 0.0f;  // 2^64
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] *= pre;
      mul = (e == 0) ? 2.7670116110564327e19f : __uint_as_float(0x7fc00000u);  // 3 * 2^63
    }
  } else {
    scale_byte = e4m3_byte(amax * gs / 6.0f);
    // true-division semantics of the oracle: x * gs / s; a zero scale gives inf / NaN codes
    mul = gs / e4m3_value(scale_byte);
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] *= mul;
  packed = pack_e2m1x8(v);
  if (!NV && amax == 0.0f) packed = 0x88888888u;  // the reference encodes an all-zero group as -0
}

template <bool NV, bool DEBUG>
__global__ void __launch_bounds__(kWarps * 32, 2) fused_quantize_kernel(const QuantParams p) {
  constexpr int TD = NV ? 16 : 32;  // transform size == quantization group
  // matrix rows for this slab: [TD][kSlab] bf16, padded against bank conflicts
  __shared__ __align__(16) __nv_bfloat16 smat[TD][kSlab + 8];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, q4 = lane & 3;
  const int64_t slab_col0 = (int64_t)blockIdx.x * kSlab;
  const int64_t col0 = slab_col0 + warp * kChunk;
  const bool shared_mat = p.mat_cols == TD;

  // ---- stage the slab's matrices -------------------------------------------------------
  if (shared_mat) {
    for (int i = threadIdx.x; i < TD * TD; i += blockDim.x) smat[i / TD][i % TD] = p.mat[i];
  } else {
    constexpr int kVecPerRow = kSlab / 8;
    for (int i = threadIdx.x; i < TD * kVecPerRow; i += blockDim.x) {
      const int r = i / kVecPerRow, c = (i % kVecPerRow) * 8;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (slab_col0 + c < p.cols)
        v = *reinterpret_cast<const uint4*>(p.mat + (int64_t)r * p.mat_cols + slab_col0 + c);
      *reinterpret_cast<uint4*>(&smat[r][c]) = v;
    }
  }
  __syncthreads();
  if (col0 >= p.cols) return;

  // ---- this lane's matrix fragments ----------------------------------------------------
  // n-tile j, k-step ks: b0 = M[8q+4ks+{0,1}][n], b1 = M[8q+4ks+{2,3}][n], n = 8(g/2)+2j+(g%2)
  uint32_t bfrag[4][2][2];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int n = 8 * (g >> 1) + 2 * j + (g & 1);
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int k = 8 * q4 + 4 * ks + 2 * h;
        __nv_bfloat16 lo, hi;
        if (NV) {
          // block-diagonal: chunk channel k pairs with outputs of the same 16-group only
          const bool same = (k >> 4) == (n >> 4);
          const int cb = shared_mat ? (n & 15) : warp * kChunk + n;
          lo = same ? smat[k & 15][cb] : __float2bfloat16(0.0f);
          hi = same ? smat[(k + 1) & 15][cb] : __float2bfloat16(0.0f);
        } else {
          const int cb = shared_mat ? n : warp * kChunk + n;
          lo = smat[k][cb];
          hi = smat[k + 1][cb];
        }
        bfrag[j][ks][h] = (uint32_t)__bfloat16_as_ushort(lo) | ((uint32_t)__bfloat16_as_ushort(hi) << 16);
      }
    }
  }

  const float gs = NV ? *p.global_scale : 0.0f;
  const int64_t row_begin = (int64_t)blockIdx.y * p.rows_per_cta;
  const int64_t row_end = min(row_begin + p.rows_per_cta, p.rows);
  if (row_begin >= row_end) return;
  const int64_t last_row = p.rows - 1;
  const __nv_bfloat16* xcol = p.x + col0 + 8 * q4;

  auto load_tile = [&](int64_t r0, uint4 (&a)[4]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int64_t r = min(r0 + g + 8 * i, last_row);  // clamp: rows past the end are discarded
      a[i] = ld_nc_v4(xcol + r * p.cols);
    }
  };

  uint4 cur[4], nxt[4];
  load_tile(row_begin, cur);
  for (int64_t r0 = row_begin; r0 < row_end; r0 += kTileRows) {
    const int64_t rn = r0 + kTileRows;
    if (rn < row_end) load_tile(rn, nxt);

#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {  // two 16-row MMA tiles: rows g+16mt and g+8+16mt
      const uint4 lo = cur[2 * mt], hi = cur[2 * mt + 1];
      float acc[4][4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;
        mma_bf16_16816(acc[j], lo.x, hi.x, lo.y, hi.y, bfrag[j][0][0], bfrag[j][0][1]);
        mma_bf16_16816(acc[j], lo.z, hi.z, lo.w, hi.w, bfrag[j][1][0], bfrag[j][1][1]);
      }
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int64_t row = r0 + g + 8 * half + 16 * mt;
        float v[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          v[2 * j] = acc[j][2 * half];
          v[2 * j + 1] = acc[j][2 * half + 1];
        }
        if (p.round_bf16) {
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = bf16_round(v[i]);
        }
        if (DEBUG && row < row_end) {
          float* t = p.transformed + row * p.cols + col0 + 8 * q4;
          *reinterpret_cast<float4*>(t) = make_float4(v[0], v[1], v[2], v[3]);
          *reinterpret_cast<float4*>(t + 4) = make_float4(v[4], v[5], v[6], v[7]);
        }
        uint32_t packed, sbyte;
        quantize_row<NV>(v, gs, q4, packed, sbyte);
        if (row < row_end) {
          *reinterpret_cast<uint32_t*>(p.q + row * (p.cols >> 1) + (col0 >> 1) + 4 * q4) = packed;
          if (NV) {
            if ((q4 & 1) == 0) p.sf[sf_offset(p.sf_layout, p.sf_cols, row, (col0 >> 4) + (q4 >> 1))] = (uint8_t)sbyte;
          } else {
            if (q4 == 0) p.sf[sf_offset(p.sf_layout, p.sf_cols, row, col0 >> 5)] = (uint8_t)sbyte;
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) cur[i] = nxt[i];
  }
}

template <bool NV, bool DEBUG>
static int launch_quant(QuantParams p, cudaStream_t stream) {
  const int64_t slabs = (p.cols + kSlab - 1) / kSlab;
  // enough CTAs for about four co-resident waves of 2 CTAs/SM, rows in multiples of the tile
  static const int ctas_per_sm = env_int("WUSH_B200_QUANT_CTAS_PER_SM", 8);
  const int sms = sm_count();
  int64_t want_y = ((int64_t)ctas_per_sm * sms + slabs - 1) / slabs;
  int64_t rpc = (p.rows + want_y - 1) / want_y;
  rpc = ((rpc + kTileRows - 1) / kTileRows) * kTileRows;
  if (rpc < kTileRows) rpc = kTileRows;
  p.rows_per_cta = rpc;
  const int64_t gy = (p.rows + rpc - 1) / rpc;
  if (gy > 65535) {
    p.rows_per_cta = ((p.rows + 65534) / 65535 + kTileRows - 1) / kTileRows * kTileRows;
  }
  dim3 grid((unsigned)slabs, (unsigned)((p.rows + p.rows_per_cta - 1) / p.rows_per_cta));
  fused_quantize_kernel<NV, DEBUG><<<grid, kWarps * 32, 0, stream>>>(p);
  return (int)cudaGetLastError();
}

static int check_quant_args(bool nv, const void* x, const void* mat, int64_t mat_cols, const float* gs,
                            const uint8_t* q, const uint8_t* sf, int64_t sf_cols, int sf_layout,
                            int64_t rows, int64_t cols, int flags) {
  const int g = nv ? 16 : 32;
  if (!x || !mat || !q || !sf || (nv && !gs)) return WUSH_ERR_NULL_POINTER;
  if (rows < 0 || cols <= 0 || cols % 32 != 0) return WUSH_ERR_BAD_SHAPE;
  if (mat_cols != cols && mat_cols != g) return WUSH_ERR_BAD_SHAPE;
  if (sf_cols % 4 != 0 || sf_cols < cols / g) return WUSH_ERR_BAD_SHAPE;
  if (sf_layout != WUSH_SF_ROW_MAJOR && sf_layout != WUSH_SF_BLOCKED) return WUSH_ERR_BAD_FLAG;
  if (flags & ~WUSH_QUANT_ROUND_BF16) return WUSH_ERR_BAD_FLAG;
  if (((uintptr_t)x & 15) || ((uintptr_t)q & 3)) return WUSH_ERR_BAD_ALIGNMENT;
  if (mat_cols == cols && ((uintptr_t)mat & 15)) return WUSH_ERR_BAD_ALIGNMENT;
  return WUSH_OK;
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
                sf_cols, sf_layout, rows, cols, 0, (flags & WUSH_QUANT_ROUND_BF16) ? 1 : 0};
  return launch_quant<false, false>(p, (cudaStream_t)stream);
}

extern "C" int wush_fused_quantize_nv(const void* x, const void* mat, int64_t mat_cols, const float* global_scale,
                                      uint8_t* q, uint8_t* sf, int64_t sf_cols, int sf_layout, int64_t rows,
                                      int64_t cols, int flags, void* stream) {
  int rc = check_quant_args(true, x, mat, mat_cols, global_scale, q, sf, sf_cols, sf_layout, rows, cols, flags);
  if (rc != WUSH_OK) return rc;
  if (rows == 0) return WUSH_OK;
  QuantParams p{(const __nv_bfloat16*)x, (const __nv_bfloat16*)mat, mat_cols, global_scale, q, sf, nullptr,
                sf_cols, sf_layout, rows, cols, 0, (flags & WUSH_QUANT_ROUND_BF16) ? 1 : 0};
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
  if (rows == 0) return WUSH_OK;
  QuantParams p{(const __nv_bfloat16*)x, (const __nv_bfloat16*)mat, mat_cols, global_scale, q, sf, transformed,
                sf_cols, sf_layout, rows, cols, 0, (flags & WUSH_QUANT_ROUND_BF16) ? 1 : 0};
  return fmt == 1 ? launch_quant<true, true>(p, (cudaStream_t)stream)
                  : launch_quant<false, true>(p, (cudaStream_t)stream);
}
