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
#include "common.cuh"

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
  const double* ynew;   // [nblocks][G][rows]: rotated targets, or the raw targets when qt is given
  const double* qt;     // [nblocks][G][G] Q^T of the block's QR, or null when ynew is already rotated
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
    s_t[i] = p.qt ? p.qt[(int64_t)blk * G * G + i] : 0.0;
  }
  __syncthreads();
  const int64_t r = (int64_t)blockIdx.x * THREADS + threadIdx.x;
  const bool active = r < p.rows;

  double y[G], xt[G];
  if (active) {
    const double* yb = p.ynew + (int64_t)blk * G * p.rows + r;
    if (p.qt) {
      // rotate the raw targets: y = Q^T y_raw, one raw coordinate at a time (rolled: a full 32 x 32 unroll
      // makes the compiler hoist a thousand shared-memory loads into registers and spill)
#pragma unroll
      for (int i = 0; i < G; ++i) y[i] = 0.0;
#pragma unroll 4
      for (int k = 0; k < G; ++k) {
        const double xk = yb[(int64_t)k * p.rows];
#pragma unroll
        for (int i = 0; i < G; ++i) y[i] += s_t[i * G + k] * xk;
      }
    } else {
#pragma unroll
      for (int i = 0; i < G; ++i) y[i] = yb[(int64_t)i * p.rows];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * G; i += THREADS) s_t[i] = p.tmat[(int64_t)blk * G * G + i];
  __syncthreads();
  if (!active) return;

  // back substitution: rn . xt = y
#pragma unroll
  for (int i = G - 1; i >= 0; --i) {
    asm volatile("" ::: "memory");   // keep each row's shared-memory loads with its row (no hoisting, no spills)
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
      asm volatile("" ::: "memory");
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

// ---------------------------------------------------------------------------------------------------
// Block preparation: everything the sweep needs per block that is G x G dense algebra, in one CTA of
// G x G threads (thread i + G j owns element (row i, column j); a column is one G-lane shuffle segment) -- the WUSH transform from the Gram matrix of
// the block's targets (cyclic Jacobi eigen-decomposition with a round-robin ordering: G/2 disjoint rotations
// per round), its rounding to the model dtype, M = basis . T^T, and the Householder QR of M.  Replaces a
// chain of ~20 small cuSOLVER / cuBLAS launches (two of them with a host synchronisation) per block.
// ---------------------------------------------------------------------------------------------------
// 1/sqrt(z) and 1/z to float64 accuracy from the float32 hardware approximation and two Newton steps: the
// float64 division and square root are long instruction sequences, and the rotation parameters below sit on
// the critical path of every Jacobi round.  z must lie inside the float32 range.
__device__ __forceinline__ double fast_rsqrt(double z) {
  double x = (double)rsqrtf((float)z);
  x = x * (1.5 - 0.5 * z * x * x);
  return x * (1.5 - 0.5 * z * x * x);
}
__device__ __forceinline__ double fast_rcp(double z) {
  double x = (double)__frcp_rn((float)z);
  x = x * (2.0 - z * x);
  return x * (2.0 - z * x);
}

struct PrepParams {
  const double* gram;    // [nblocks][G][G] y y^T of the block's targets (unused unless the transform is 'wush'/'wus')
  const double* basis;   // first block's G x G upper-triangular diagonal block of the Cholesky factor
  int64_t ldb;           // its row stride
  int64_t basis_step;    // elements between consecutive blocks' diagonal blocks (G * ldb + G inside one factor)
  double* tmat;          // [nblocks][G][G] out: block transform (in: when transform == GIVEN)
  double* rn;            // [nblocks][G][G] out: R of the QR of basis . T^T
  double* qt;            // [nblocks][G][G] out: Q^T
  int transform;         // WUSH_TRANSFORM_*
  int round_f32;         // round T to fp32 instead of bf16 (the model dtype)
  double inv_sqrt_rows;  // R^-1/2
  int* status;           // set to 1 when a transform is not finite
};

template <int G>
__global__ void __launch_bounds__(G* G) sweep_prep_kernel(const PrepParams p) {
  constexpr int LD = G + 1;
  __shared__ double sA[G * LD], sV[G * LD], sB[G * LD], sT[G * LD];
  __shared__ double s_c[G / 2], s_s[G / 2], s_lam[G], s_sq[G], s_col[G];
  __shared__ int s_p[G / 2], s_q[G / 2], s_ord[G], s_any[32];
  const int tid = threadIdx.x, i = tid % G, j = tid / G;
  const int blk = blockIdx.x;
  const double* basis = p.basis + (int64_t)blk * p.basis_step;
  sB[i * LD + j] = j >= i ? basis[(int64_t)i * p.ldb + j] : 0.0;
  const double had_scale = G == 32 ? 0.17677669529663687 : 0.25;      // G^-1/2
  auto had = [&](int r, int c) { return (__popc(r & c) & 1) ? -had_scale : had_scale; };   // Sylvester

  if (p.transform == WUSH_TRANSFORM_GIVEN) {
    sT[i * LD + j] = p.tmat[(int64_t)blk * G * G + i * G + j];
  } else if (p.transform == WUSH_TRANSFORM_IDENTITY) {
    sT[i * LD + j] = i == j ? 1.0 : 0.0;
  } else if (p.transform == WUSH_TRANSFORM_HADAMARD) {
    sT[i * LD + j] = had(i, j);
  } else {
    // ---- eigen-decomposition of the Gram matrix: A = V diag(lam) V^T ---------------------------------
    sA[i * LD + j] = p.gram[(int64_t)blk * G * G + i * G + j];
    sV[i * LD + j] = i == j ? 1.0 : 0.0;
    __syncthreads();
    // The rotations are done by the first JT threads alone, synchronised by a named barrier: a round is three
    // short dependent phases, and a barrier over all G*G threads costs more than the work between two of them.
    constexpr int JT = G * G / 4 < 64 ? 64 : G * G / 4;
    if (tid < JT) {
      auto jbar = [] { asm volatile("bar.sync 1, %0;\n" ::"n"(JT) : "memory"); };
      for (int sweep = 0; sweep < 30; ++sweep) {
        // converged when every off-diagonal element is below 1e-13 of the largest diagonal element: the
        // transform built from the vectors is rounded to bf16 / fp32 afterwards, and Jacobi converges
        // quadratically from there anyway (the simultaneous rotations of a round work on slightly stale values,
        // so this ordering needs a few more sweeps than the sequential cyclic one: about 11 for a Gram matrix
        // of condition 1e8)
        double dmax = 0.0;
        for (int k = 0; k < G; ++k) dmax = fmax(dmax, fabs(sA[k * LD + k]));
        bool big = false;
        for (int e = tid; e < G * G; e += JT) {
          const int r = e % G, cidx = e / G;
          big |= r != cidx && fabs(sA[r * LD + cidx]) > 1e-13 * dmax;
        }
        if (tid % 32 == 0) s_any[tid / 32] = 0;
        jbar();
        if (big) s_any[tid / 32] = 1;
        jbar();
        int any = 0;
        for (int w = 0; w < JT / 32; ++w) any |= s_any[w];
        if (!any) break;
        for (int round = 0; round < G - 1; ++round) {
          if (tid < G / 2) {
            // round-robin pairing: seat 0 is fixed, the other G-1 players rotate
            auto seat = [&](int m) { return m == 0 ? 0 : 1 + (m - 1 + round) % (G - 1); };
            int a = seat(tid), b = seat(G - 1 - tid);
            const int pp = min(a, b), qq = max(a, b);
            const double apq = sA[pp * LD + qq], app = sA[pp * LD + pp], aqq = sA[qq * LD + qq];
            double c = 1.0, s = 0.0;
            if (apq * apq > 1e-36 * fabs(app * aqq) && apq != 0.0) {
              // t = tan(theta) = sgn(tau) / (|tau| + sqrt(1 + tau^2)), tau = (aqq - app) / (2 apq), written
              // without the quotient tau: t = sgn * |b| / (|d| + sqrt(d^2 + b^2))
              const double d = aqq - app, b2 = 2.0 * apq, z = d * d + b2 * b2;
              double t;
              if (z > 1e-30 && z < 1e30) {
                t = fabs(b2) * fast_rcp(fabs(d) + z * fast_rsqrt(z));
              } else {
                t = fabs(b2) / (fabs(d) + sqrt(z));
              }
              if ((d < 0.0) != (b2 < 0.0)) t = -t;
              c = fast_rsqrt(1.0 + t * t);
              s = t * c;
            }
            s_p[tid] = pp; s_q[tid] = qq; s_c[tid] = c; s_s[tid] = s;
          }
          jbar();
          for (int e = tid; e < G * G / 2; e += JT) {   // columns: [Ap Aq] <- [c Ap - s Aq, s Ap + c Aq], same for V
            const int r = e % G, k = e / G, pp = s_p[k], qq = s_q[k];
            const double c = s_c[k], s = s_s[k];
            const double ap = sA[r * LD + pp], aq = sA[r * LD + qq];
            sA[r * LD + pp] = c * ap - s * aq;
            sA[r * LD + qq] = s * ap + c * aq;
            const double vp = sV[r * LD + pp], vq = sV[r * LD + qq];
            sV[r * LD + pp] = c * vp - s * vq;
            sV[r * LD + qq] = s * vp + c * vq;
          }
          jbar();
          for (int e = tid; e < G * G / 2; e += JT) {   // rows of A
            const int cc = e % G, k = e / G, pp = s_p[k], qq = s_q[k];
            const double c = s_c[k], s = s_s[k];
            const double ap = sA[pp * LD + cc], aq = sA[qq * LD + cc];
            sA[pp * LD + cc] = c * ap - s * aq;
            sA[qq * LD + cc] = s * ap + c * aq;
          }
          jbar();
        }
      }
    }
    __syncthreads();
    // ---- order by descending eigenvalue, fix the signs, singular values -------------------------------
    if (tid < G) s_lam[tid] = sA[tid * LD + tid];
    __syncthreads();
    if (tid < G) {
      int rank = 0;
      for (int k = 0; k < G; ++k) rank += (s_lam[k] > s_lam[tid]) || (s_lam[k] == s_lam[tid] && k < tid);
      s_ord[rank] = tid;
    }
    __syncthreads();
    if (tid < G) {
      const int col = s_ord[tid];
      double best = -1.0, lead = 1.0;
      for (int r = 0; r < G; ++r) {
        const double v = sV[r * LD + col];
        if (fabs(v) > best) { best = fabs(v); lead = v; }
      }
      s_col[tid] = lead < 0.0 ? -1.0 : 1.0;                                  // largest component positive
      s_sq[tid] = sqrt(fmax(s_lam[col], 0.0)) * p.inv_sqrt_rows;             // singular value * R^-1/2
    }
    __syncthreads();
    if (tid == 0) {
      double mean = 0.0;
      for (int k = 0; k < G; ++k) mean += s_sq[k];
      mean /= G;
      for (int k = 0; k < G; ++k) s_sq[k] = sqrt(s_sq[k] + 0.01 * mean) * s_col[k];   // damped, square root, sign
    }
    __syncthreads();
    // rhs = (Had . diag(s^1/2)) V^T  ->  sA (the Gram matrix is no longer needed)
    {
      double acc = 0.0;
      const bool wus = p.transform == WUSH_TRANSFORM_WUS;
      for (int k = 0; k < G; ++k) acc += (wus ? (i == k ? 1.0 : 0.0) : had(i, k)) * s_sq[k] * sV[j * LD + s_ord[k]];
      __syncthreads();
      sA[i * LD + j] = acc;
    }
    __syncthreads();
    // T . basis^T = rhs: one back substitution per row of T
    if (tid < G) {
      for (int c = G - 1; c >= 0; --c) {
        double acc = sA[tid * LD + c];
        for (int k = c + 1; k < G; ++k) acc -= sB[c * LD + k] * sT[tid * LD + k];
        sT[tid * LD + c] = acc / sB[c * LD + c];
      }
    }
    __syncthreads();
  }
  if (p.transform != WUSH_TRANSFORM_GIVEN) {
    // the reference rounds the transform to the model dtype and continues in float64 with the rounded values
    const float f = __double2float_rn(sT[i * LD + j]);
    const double t = p.round_f32 ? (double)f : (double)__bfloat162float(__float2bfloat16_rn(f));
    if (!(fabs(t) <= 1.7e308) && p.status) atomicExch(p.status, 1);
    sT[i * LD + j] = t;
    p.tmat[(int64_t)blk * G * G + i * G + j] = t;
  }
  __syncthreads();

  // ---- M = basis . T^T, then Householder QR: M -> R in place, Q^T accumulated from the identity ----------
  {
    double acc = 0.0;
    for (int k = i; k < G; ++k) acc += sB[i * LD + k] * sT[j * LD + k];
    sA[i * LD + j] = acc;             // M
    sV[i * LD + j] = i == j ? 1.0 : 0.0;   // Q^T
  }
  __syncthreads();
  for (int c = 0; c < G - 1; ++c) {
    // every warp derives the reflector of column c (lane i holds M[i][c])
    const double mic = sA[i * LD + c];
    double x2 = i > c ? mic * mic : 0.0;
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) x2 += __shfl_xor_sync(0xffffffffu, x2, o, G);
    const double alpha = __shfl_sync(0xffffffffu, mic, c, G);
    __syncthreads();                  // column c has been read by everyone before its owner rewrites it
    if (x2 > 0.0) {
      const double z = alpha * alpha + x2;
      const bool fast = z > 1e-30 && z < 1e30;
      const double nrm = fast ? z * fast_rsqrt(z) : sqrt(z);
      const double beta = alpha >= 0.0 ? -nrm : nrm;
      const double tau = fast ? (beta - alpha) * fast_rcp(beta) : (beta - alpha) / beta;
      const double inv = fast ? fast_rcp(alpha - beta) : 1.0 / (alpha - beta);
      const double v = i == c ? 1.0 : (i > c ? mic * inv : 0.0);
      // apply H = I - tau v v^T to column j of M and of Q^T
      double dm = v * sA[i * LD + j], dq = v * sV[i * LD + j];
#pragma unroll
      for (int o = G / 2; o > 0; o >>= 1) {
        dm += __shfl_xor_sync(0xffffffffu, dm, o, G);
        dq += __shfl_xor_sync(0xffffffffu, dq, o, G);
      }
      if (j == c) sA[i * LD + j] = i == c ? beta : (i > c ? 0.0 : sA[i * LD + j]);
      else if (j > c) sA[i * LD + j] -= tau * dm * v;
      sV[i * LD + j] -= tau * dq * v;
    }
    __syncthreads();
  }
  p.rn[(int64_t)blk * G * G + i * G + j] = j >= i ? sA[i * LD + j] : 0.0;
  p.qt[(int64_t)blk * G * G + i * G + j] = sV[i * LD + j];
}

}  // namespace sweep
}  // namespace wush

extern "C" WUSH_API int wush_gptq_block_step(const double* rn, const double* ynew, const double* qt, const double* tmat, int nblocks,
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
  if (const int rc100 = wush::require_sm100()) return rc100;
  if (rows == 0 || nblocks == 0) return WUSH_OK;
  Params p{rn, ynew, qt, tmat, codes, scales, fake, coef, rows, cols, col_block0, (flags & WUSH_SWEEP_RTN_ONLY) != 0,
           (flags & WUSH_SWEEP_FAKE_F32) != 0};
  const dim3 grid((unsigned)((rows + THREADS - 1) / THREADS), (unsigned)nblocks);
  if (format == WUSH_FORMAT_NVFP4) sweep_block_kernel<true><<<grid, THREADS, 0, (cudaStream_t)stream>>>(p);
  else sweep_block_kernel<false><<<grid, THREADS, 0, (cudaStream_t)stream>>>(p);
  return (int)cudaGetLastError();
}

extern "C" WUSH_API int wush_gptq_block_prepare(const double* gram, const double* basis, int64_t ldb, int64_t basis_step,
                                                int nblocks, int format, int transform, int flags, int64_t rows,
                                                double* tmat, double* rn, double* qt, int* status, void* stream) {
  using namespace wush::sweep;
  if (!basis || !tmat || !rn || !qt) return WUSH_ERR_NULL_POINTER;
  if (format != WUSH_FORMAT_MXFP4 && format != WUSH_FORMAT_NVFP4) return WUSH_ERR_BAD_FLAG;
  if (transform < WUSH_TRANSFORM_IDENTITY || transform > WUSH_TRANSFORM_GIVEN) return WUSH_ERR_BAD_FLAG;
  if ((transform == WUSH_TRANSFORM_WUSH || transform == WUSH_TRANSFORM_WUS) && !gram) return WUSH_ERR_NULL_POINTER;
  if (flags & ~WUSH_SWEEP_FAKE_F32) return WUSH_ERR_BAD_FLAG;
  const int g = format == WUSH_FORMAT_NVFP4 ? 16 : 32;
  if (nblocks < 0 || ldb < g || rows <= 0) return WUSH_ERR_BAD_SHAPE;
  if (const int rc100 = wush::require_sm100()) return rc100;
  if (nblocks == 0) return WUSH_OK;
  PrepParams p{gram, basis, ldb, basis_step, tmat, rn, qt, transform, (flags & WUSH_SWEEP_FAKE_F32) != 0,
               1.0 / sqrt((double)rows), status};
  if (g == 32) sweep_prep_kernel<32><<<nblocks, 32 * 32, 0, (cudaStream_t)stream>>>(p);
  else sweep_prep_kernel<16><<<nblocks, 16 * 16, 0, (cudaStream_t)stream>>>(p);
  return (int)cudaGetLastError();
}
