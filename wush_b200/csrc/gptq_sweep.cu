// Inner step of the GPTQ / Babai column sweep for one group-sized block of weight columns (sm_100a).
//
// After the host has rotated the block (QR of basis . transform^T, y_new = Q^T y), every weight row is
// independent: solve the triangular system for its transformed coefficients, choose the group scale,
// round to E2M1, and -- unless plain round-to-nearest is asked for -- walk the coordinates from last
// to first, rounding one coordinate with the scale frozen and pushing its error onto the targets of
// the coordinates still to come (Babai's nearest plane).  One thread owns one weight row and keeps
// the whole group in float64 registers, so a block of any number of rows is one launch instead of
// the reference's 10 + 3 G tensor passes.  All arithmetic is float64 in the reference's operation
// order; the scale casts and the E2M1 tie rule are those of its torch quantizer.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "../../include/wush_b200.h"

namespace wush {
namespace sweep {

constexpr int THREADS = 128;

// ---- scale casts (torch's float64 -> float32 -> float8 conversions) -------------------------------
// E8M0: power-of-two rounding of a non-negative float32, half rounds up; byte 0 stands for 2^-127, and a
// float32 subnormal maps to byte 1 only above 2^-127.  Returns the byte; *deq its value.
__device__ __forceinline__ uint32_t cast_e8m0(double s, double* deq) {
  const uint32_t b = __float_as_uint(__double2float_rn(s));
  const uint32_t exp = (b >> 23) & 0xFF;
  uint32_t out = exp + ((b >> 22) & 1);
  if (exp == 0) out = (b & 0x7FFFFF) > 0x400000 ? 1 : 0;
  if (exp == 0xFF || out > 0xFF) out = 0xFF;
  *deq = out == 0xFF ? __longlong_as_double(0x7FF8000000000000LL) : ldexp(1.0, (int)out - 127);
  return out;
}

// E4M3 (fn): round to nearest even onto 3 mantissa bits, subnormal step 2^-9, no saturation: what rounds
// above 448 (and inf/NaN) becomes NaN (0x7F).  The scale is never negative.
__device__ __forceinline__ uint32_t cast_e4m3(double s, double* deq) {
  const double a = (double)__double2float_rn(s);
  if (!(a <= 3.5e38)) {
    *deq = __longlong_as_double(0x7FF8000000000000LL);
    return 0x7F;
  }
  int e = a > 0.0 ? ilogb(a) : 0;
  if (e < -6) e = -6;
  const double step = ldexp(1.0, e - 3);
  const double q = rint(a / step) * step;       // round half to even
  if (q > 448.0) {
    *deq = __longlong_as_double(0x7FF8000000000000LL);
    return 0x7F;
  }
  *deq = q;
  if (q < 0.015625) return (uint32_t)(q * 512.0);            // subnormal: mantissa = q / 2^-9
  const int e2 = ilogb(q);
  return ((uint32_t)(e2 + 7) << 3) | (uint32_t)((q / ldexp(1.0, e2) - 1.0) * 8.0);
}

// ---- E2M1 round-to-nearest, ties to the even code; exact zero and (-0.25, 0] encode as -0 (code 8),
// NaN as code 7: the behaviour of the reference's bucketize on its signed grid ------------------------
__device__ __forceinline__ uint32_t rtn_e2m1(double v, double* val) {
  if (v != v) {
    *val = 6.0;
    return 7;
  }
  const double a = fabs(v);
  uint32_t idx;
  double m;
  if (a <= 0.25) { idx = 0; m = 0.0; }
  else if (a < 0.75) { idx = 1; m = 0.5; }
  else if (a <= 1.25) { idx = 2; m = 1.0; }
  else if (a < 1.75) { idx = 3; m = 1.5; }
  else if (a <= 2.5) { idx = 4; m = 2.0; }
  else if (a < 3.5) { idx = 5; m = 3.0; }
  else if (a <= 5.0) { idx = 6; m = 4.0; }
  else { idx = 7; m = 6.0; }
  const bool neg = v < 0.0 || (idx == 0 && v <= 0.0);
  *val = neg ? -m : m;
  return idx | (neg ? 8u : 0u);
}

struct Params {
  const double* rn;     // [nblocks][G][G] upper triangular
  const double* ynew;   // [nblocks][G][rows]
  const double* tmat;   // [nblocks][G][G]
  uint8_t* codes;       // [rows][cols/2]
  uint8_t* scales;      // [rows][cols/G]
  void* fake;           // [rows][cols] bf16 or fp32, may be null
  double* coef;         // [nblocks][G][rows], may be null
  int64_t rows, cols;
  int col_block0;
  int rtn_only;
  int fake_f32;
};

template <bool NV>
__global__ void __launch_bounds__(THREADS) sweep_block_kernel(const Params p) {
  constexpr int G = NV ? 16 : 32;
  constexpr double GS = NV ? 10.0 : 3.0, SS = NV ? 6.0 : 4.0;
  __shared__ double s_rn[G * G];
  __shared__ double s_t[G * G];
  const int blk = blockIdx.y;
  for (int i = threadIdx.x; i < G * G; i += THREADS) {
    s_rn[i] = p.rn[(int64_t)blk * G * G + i];
    s_t[i] = p.tmat[(int64_t)blk * G * G + i];
  }
  __syncthreads();
  const int64_t r = (int64_t)blockIdx.x * THREADS + threadIdx.x;
  if (r >= p.rows) return;

  double y[G], xt[G];
  const double* yb = p.ynew + (int64_t)blk * G * p.rows + r;
#pragma unroll
  for (int i = 0; i < G; ++i) y[i] = yb[(int64_t)i * p.rows];

  // back substitution: rn . xt = y
#pragma unroll
  for (int i = G - 1; i >= 0; --i) {
    double acc = y[i];
#pragma unroll
    for (int j = i + 1; j < G; ++j) acc -= s_rn[i * G + j] * xt[j];
    xt[i] = acc / s_rn[i * G + i];
  }

  // group scale from the solved coefficients
  double amax = 0.0;
#pragma unroll
  for (int i = 0; i < G; ++i) amax = fmax(amax, fabs(xt[i]));
  double sdeq;
  const uint32_t sbyte = NV ? cast_e4m3(amax * GS / SS, &sdeq) : cast_e8m0(amax * GS / SS, &sdeq);

  uint32_t code[G];
  if (p.rtn_only) {
#pragma unroll
    for (int i = 0; i < G; ++i) {
      double val;
      code[i] = rtn_e2m1(xt[i] * GS / sdeq, &val);
      xt[i] = val * sdeq / GS;
    }
  } else {
    // nearest plane, last coordinate first; every later re-quantization of an already rounded
    // coordinate reproduces its code, except that a rounded +0 comes back as -0 (code 8)
#pragma unroll
    for (int i = G - 1; i >= 0; --i) {
      const double xi = y[i] / s_rn[i * G + i];
      double val;
      code[i] = rtn_e2m1(xi * GS / sdeq, &val);
      if (i > 0 && code[i] == 0) { code[i] = 8; val = -0.0; }
      const double f = val * sdeq / GS;
      xt[i] = f;
#pragma unroll
      for (int k = 0; k < i; ++k) y[k] -= s_rn[k * G + i] * f;
    }
  }

  // outputs: packed codes, scale byte, dequantized transformed weights, coefficients
  const int cb = p.col_block0 + blk;
  uint32_t packed[G / 8];
#pragma unroll
  for (int w = 0; w < G / 8; ++w) {
    uint32_t v = 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) v |= code[8 * w + e] << (4 * e);   // element 2i in the low nibble of byte i
    packed[w] = v;
  }
  uint8_t* cdst = p.codes + r * (p.cols / 2) + (int64_t)cb * (G / 2);
  if (NV) *reinterpret_cast<uint2*>(cdst) = make_uint2(packed[0], packed[1]);
  else *reinterpret_cast<uint4*>(cdst) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
  p.scales[r * (p.cols / G) + cb] = (uint8_t)sbyte;
  if (p.fake) {
    // torch's float64 -> bf16 conversion goes through float32
    if (p.fake_f32) {
      float* f = reinterpret_cast<float*>(p.fake) + r * p.cols + (int64_t)cb * G;
#pragma unroll
      for (int i = 0; i < G; ++i) f[i] = __double2float_rn(xt[i]);
    } else {
      __nv_bfloat16* f = reinterpret_cast<__nv_bfloat16*>(p.fake) + r * p.cols + (int64_t)cb * G;
#pragma unroll
      for (int i = 0; i < G; i += 2)
        *reinterpret_cast<__nv_bfloat162*>(f + i) =
            __floats2bfloat162_rn(__double2float_rn(xt[i]), __double2float_rn(xt[i + 1]));
    }
  }
  if (p.coef) {
    double* c = p.coef + (int64_t)blk * G * p.rows + r;
#pragma unroll 4
    for (int k = 0; k < G; ++k) {
      double acc = 0.0;
#pragma unroll
      for (int i = 0; i < G; ++i) acc += s_t[i * G + k] * xt[i];
      c[(int64_t)k * p.rows] = acc;
    }
  }
}

}  // namespace sweep
}  // namespace wush

extern "C" WUSH_API int wush_gptq_block_step(const double* rn, const double* ynew, const double* tmat, int nblocks,
                                    int col_block0, int64_t rows, int64_t cols, int format, int flags, uint8_t* codes,
                                    uint8_t* scales, void* fake, double* coef, void* stream) {
  using namespace wush::sweep;
  if (!rn || !ynew || !tmat || !codes || !scales) return WUSH_ERR_NULL_POINTER;
  if (format != WUSH_FORMAT_MXFP4 && format != WUSH_FORMAT_NVFP4) return WUSH_ERR_BAD_FLAG;
  if (flags & ~(WUSH_SWEEP_RTN_ONLY | WUSH_SWEEP_FAKE_F32)) return WUSH_ERR_BAD_FLAG;
  const int g = format == WUSH_FORMAT_NVFP4 ? 16 : 32;
  if (rows < 0 || cols <= 0 || cols % g || nblocks < 0 || col_block0 < 0 || (int64_t)(col_block0 + nblocks) * g > cols)
    return WUSH_ERR_BAD_SHAPE;
  if (nblocks > 65535) return WUSH_ERR_TOO_LARGE;
  if ((reinterpret_cast<uintptr_t>(codes) | reinterpret_cast<uintptr_t>(fake)) & 15) return WUSH_ERR_BAD_ALIGNMENT;
  if (rows == 0 || nblocks == 0) return WUSH_OK;
  Params p{rn, ynew, tmat, codes, scales, fake, coef, rows, cols, col_block0, (flags & WUSH_SWEEP_RTN_ONLY) != 0,
           (flags & WUSH_SWEEP_FAKE_F32) != 0};
  const dim3 grid((unsigned)((rows + THREADS - 1) / THREADS), (unsigned)nblocks);
  if (format == WUSH_FORMAT_NVFP4) sweep_block_kernel<true><<<grid, THREADS, 0, (cudaStream_t)stream>>>(p);
  else sweep_block_kernel<false><<<grid, THREADS, 0, (cudaStream_t)stream>>>(p);
  return (int)cudaGetLastError();
}
