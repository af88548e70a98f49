// Block-scaled FP4 matrix-vector product for decode: y[m, n] = alpha * sum_k a[m, k] * b[n, k] for 1..4 activation
// rows.  With so few rows the product is a single pass over the weight bytes, so this kernel streams them with plain
// coalesced 16-byte loads and does the arithmetic on the CUDA cores instead of staging 128-row tiles for the tensor
// cores: no tensor maps, no TMEM, no cluster hand-over, and every SM has work (2 weight rows per warp; 1, 2 or 4 warps share them along k).
//
// Arithmetic.  E2M1 codes are converted to fp16 pairs in hardware (cvt.rn.f16x2.e2m1x2); a product of two E2M1
// values is a multiple of 0.25 below 36, so a chain of 8 fp16 fused multiply-adds is exact (below 512 in steps of
// 0.25).  Group sums are then added and scaled in fp32: MXFP4 by the two power-of-two scales, NVFP4 by the two E4M3
// scales.  Only the order of the fp32 additions differs from the tensor-core kernel.
//
// Layouts are those of the GEMM entry points: codes [rows, k/2] with element 2i in the low nibble, scales in the
// blocked 128 x 4 layout (to_blocked, inference_lib/src/fp_quant/module/qutlass_ops.py:145-166).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "common.cuh"
#include "fp4_gemv.cuh"

namespace wush {
namespace gemv {

constexpr int WARPS = 4;        // warps per CTA
constexpr int RW = 2;           // weight rows per warp: every warp walks the whole k range of its rows
constexpr int BATCH = 4;        // 16-byte units per lane and row whose loads are issued together

struct Params {
  const uint8_t* a;
  const uint8_t* b;
  const uint8_t* sfa;
  const uint8_t* sfb;
  const float* alpha;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  __nv_bfloat16* y;
  int64_t ldr, ldy;
  int n, k;
  int sf_cols;                 // scale bytes per row (k / group), a multiple of 4
  int ksplit;                  // 1, 2 or 4 warps of a CTA share a pair of rows, each taking a part of the k range
};

__device__ __forceinline__ int64_t sf_off(int row, int g, int sf_cols) {
  return ((int64_t)(row >> 7) * (sf_cols >> 2) + (g >> 2)) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4 + (g & 3);
}

// 8 E2M1 codes (one 32-bit word, element 0 in the lowest nibble) -> 4 fp16 pairs in element order
__device__ __forceinline__ void e2m1x8_to_f16x2(uint32_t w, uint32_t& h0, uint32_t& h1, uint32_t& h2, uint32_t& h3) {
  asm("{\n"
      ".reg .b8 b0, b1, b2, b3;\n"
      "mov.b32 {b0, b1, b2, b3}, %4;\n"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n"
      "cvt.rn.f16x2.e2m1x2 %1, b1;\n"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n"
      "cvt.rn.f16x2.e2m1x2 %3, b3;\n"
      "}\n"
      : "=r"(h0), "=r"(h1), "=r"(h2), "=r"(h3)
      : "r"(w));
}

__device__ __forceinline__ uint32_t hfma2(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.f16x2 %0, %1, %2, %3;\n" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

__device__ __forceinline__ uint32_t hmul2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.f16x2 %0, %1, %2;\n" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

__device__ __forceinline__ float half2_sum(uint32_t s) {
  const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&s));
  return f.x + f.y;
}

__device__ __forceinline__ float e8m0_value(uint32_t e) {
  // 2^(e - 127); e = 0 is the subnormal 2^-127, e = 255 is NaN
  return __uint_as_float(e == 0 ? 0x00400000u : (e == 255 ? 0x7fc00000u : e << 23));
}

__device__ __forceinline__ float2 e4m3x2_value(uint32_t two_bytes) {
  uint32_t h;
  asm("{\n.reg .b16 t;\ncvt.u16.u32 t, %1;\ncvt.rn.f16x2.e4m3x2 %0, t;\n}\n" : "=r"(h) : "r"(two_bytes));
  return __half22float2(*reinterpret_cast<const __half2*>(&h));
}

// Shared memory: the activations as fp16, converted once per CTA.  Unit u (32 values) of row m is four 16-byte
// quarters stored at a_sm[(m * 4 + q) * units + u], so that the lanes of a warp (consecutive units) read
// consecutive 16-byte words; then the activation scales as fp32, [m][units] (MXFP4) or [m][2 * units] (NVFP4).
template <bool NV, int M>
__global__ void __launch_bounds__(WARPS * 32) fp4_gemv_kernel(const Params p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  constexpr int V = M * RW;                               // sums per lane
  constexpr int VP = V <= 2 ? 2 : (V <= 4 ? 4 : 8);       // padded to a power of two for the lane reduction
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int units = p.k >> 5;                  // 16-byte units (32 codes) per row
  const int64_t ldb = p.k >> 1;                // bytes per row of codes
  uint4* a_sm = reinterpret_cast<uint4*>(smem_raw);
  float* a_sf = reinterpret_cast<float*>(smem_raw + (size_t)M * 4 * units * 16);
  const int iters = (units + 31) >> 5;          // passes of 32 units
  const int S = p.ksplit;
  const int pair = warp / S, split = warp - pair * S;
  const int row0 = (blockIdx.x * (WARPS / S) + pair) * RW;
  const int per = (iters + S - 1) / S;
  const int it_begin = split * per, it_end = min(iters, it_begin + per);

  // Programmatic dependent launch: this kernel may start while the previous kernel of the stream is still running.
  // Until the wait below returns it must not read what that kernel may write, so it only asks the L2 to fetch its
  // rows of the weights (a prefetch is a hint to the cache that stays coherent, not a read) and lets its own
  // successor start; the loads that follow then mostly hit the L2.
  {
    const int lines = (int)((ldb + 127) >> 7);
#pragma unroll
    for (int r = 0; r < RW; ++r) {
      const uint8_t* rowp = p.b + (int64_t)min(row0 + r, p.n - 1) * ldb;
      for (int l = it_begin * 4 + lane; l < min(it_end * 4, lines); l += 32)
        asm volatile("prefetch.global.L2 [%0];\n" ::"l"(rowp + (int64_t)l * 128));
    }
  }
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  asm volatile("griddepcontrol.wait;\n" ::: "memory");

  // the first batch of weight loads goes out before the activations are staged
  uint4 bw[BATCH][RW];
  uint32_t sb[BATCH][RW];
  // row-dependent parts of the addresses, once per warp: the codes of the row and its place inside the 128 x 4 scale atoms
  const uint8_t* brow[RW];
  const uint8_t* sfrow[RW];
#pragma unroll
  for (int r = 0; r < RW; ++r) {
    const int row = min(row0 + r, p.n - 1);
    brow[r] = p.b + (int64_t)row * ldb;
    sfrow[r] = p.sfb + sf_off(row, 0, p.sf_cols);
  }
  auto issue = [&](int it0) {
#pragma unroll
    for (int j = 0; j < BATCH; ++j) {
      const int u = min((it0 + j) * 32 + lane, units - 1);
      // scale group(s) of unit u: atom (g >> 2) is 512 bytes further, byte (g & 3) inside the row's word
      const int sfo = NV ? (u >> 1) * 512 + (u & 1) * 2 : (u >> 2) * 512 + (u & 3);
#pragma unroll
      for (int r = 0; r < RW; ++r) {
        bw[j][r] = __ldg(reinterpret_cast<const uint4*>(brow[r] + (int64_t)u * 16));
        sb[j][r] = NV ? (uint32_t)__ldg(reinterpret_cast<const uint16_t*>(sfrow[r] + sfo)) : (uint32_t)__ldg(sfrow[r] + sfo);
      }
    }
  };
  issue(it_begin);

  for (int idx = threadIdx.x; idx < M * units; idx += WARPS * 32) {
    const int m = idx / units, u = idx - m * units;
    const uint4 aw = *reinterpret_cast<const uint4*>(p.a + (int64_t)m * ldb + (int64_t)u * 16);
    const uint32_t w[4] = {aw.x, aw.y, aw.z, aw.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint4 h;
      e2m1x8_to_f16x2(w[q], h.x, h.y, h.z, h.w);
      a_sm[(m * 4 + q) * units + u] = h;
    }
    if (NV) {
      const float2 s = e4m3x2_value(*reinterpret_cast<const uint16_t*>(p.sfa + sf_off(m, 2 * u, p.sf_cols)));
      a_sf[(m * units + u) * 2] = s.x;
      a_sf[(m * units + u) * 2 + 1] = s.y;
    } else {
      a_sf[m * units + u] = e8m0_value(p.sfa[sf_off(m, u, p.sf_cols)]);
    }
  }
  __syncthreads();

  float acc[VP];
#pragma unroll
  for (int i = 0; i < VP; ++i) acc[i] = 0.0f;

  for (int it0 = it_begin; it0 < it_end; it0 += BATCH) {
#pragma unroll
    for (int j = 0; j < BATCH; ++j) {
      const int u = (it0 + j) * 32 + lane;
      if (it0 + j < it_end && u < units) {     // lanes and batch slots past the end loaded a repeated unit: skipped
        uint32_t bh[RW][16];
#pragma unroll
        for (int r = 0; r < RW; ++r) {
          const uint32_t w[4] = {bw[j][r].x, bw[j][r].y, bw[j][r].z, bw[j][r].w};
#pragma unroll
          for (int q = 0; q < 4; ++q) e2m1x8_to_f16x2(w[q], bh[r][4 * q], bh[r][4 * q + 1], bh[r][4 * q + 2], bh[r][4 * q + 3]);
        }
#pragma unroll
        for (int m = 0; m < M; ++m) {
          uint32_t s0[RW], s1[RW];             // fp16 pair sums of the two halves of the unit (8 products per half)
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const uint4 ah = a_sm[(m * 4 + q) * units + u];
            const uint32_t av[4] = {ah.x, ah.y, ah.z, ah.w};
#pragma unroll
            for (int r = 0; r < RW; ++r) {
              uint32_t& s = q < 2 ? s0[r] : s1[r];
              s = (q & 1) ? hfma2(av[0], bh[r][4 * q], s) : hmul2(av[0], bh[r][4 * q]);
#pragma unroll
              for (int i = 1; i < 4; ++i) s = hfma2(av[i], bh[r][4 * q + i], s);
            }
          }
#pragma unroll
          for (int r = 0; r < RW; ++r) {
            if (NV) {
              const float2 fb = e4m3x2_value(sb[j][r]);
              const float2 fa = *reinterpret_cast<const float2*>(&a_sf[(m * units + u) * 2]);
              acc[m * RW + r] = fmaf(half2_sum(s1[r]) * fb.y, fa.y, fmaf(half2_sum(s0[r]) * fb.x, fa.x, acc[m * RW + r]));
            } else {
              const float s = half2_sum(s0[r]) + half2_sum(s1[r]);
              acc[m * RW + r] = fmaf(s * e8m0_value(sb[j][r]), a_sf[m * units + u], acc[m * RW + r]);
            }
          }
        }
      }
    }
    if (it0 + BATCH < it_end) issue(it0 + BATCH);
  }

  // lane reduction: each step folds half of the sums onto the other half of the lanes, then plain butterflies;
  // afterwards the 32 / VP lanes of group i hold the total of sum i
  int bit = 16;
#pragma unroll
  for (int width = VP / 2; width >= 1; width >>= 1, bit >>= 1) {
    const bool hi = (lane & bit) != 0;
#pragma unroll
    for (int i = 0; i < width; ++i) {
      const float keep = hi ? acc[i + width] : acc[i];
      const float send = hi ? acc[i] : acc[i + width];
      acc[i] = keep + __shfl_xor_sync(0xffffffffu, send, bit);
    }
  }
  float total = acc[0];
  for (; bit >= 1; bit >>= 1) total += __shfl_xor_sync(0xffffffffu, total, bit);
  constexpr int LANES_PER_SUM = 32 / VP;
  const int idx = lane / LANES_PER_SUM;
  const bool writer = lane % LANES_PER_SUM == 0 && idx < V;
  if (S > 1) {                                 // the warps that share the rows add their parts in split order
    __shared__ float part[WARPS][8];
    if (writer) part[warp][idx] = total;
    __syncthreads();
    if (split != 0) return;
    if (writer)
      for (int i = 1; i < S; ++i) total += part[warp + i][idx];
  }
  if (writer) {
    const int m = idx / RW, col = row0 + idx % RW;
    if (col < p.n) {
      // the GEMM's epilogue: product rounded to bf16, then bias and residual added as bf16 tensors would be
      __nv_bfloat16 v = __float2bfloat16_rn(total * *p.alpha);
      if (p.bias != nullptr) v = __float2bfloat16_rn(__bfloat162float(v) + __bfloat162float(p.bias[col]));
      if (p.residual != nullptr)
        v = __float2bfloat16_rn(__bfloat162float(v) + __bfloat162float(p.residual[(int64_t)m * p.ldr + col]));
      p.y[(int64_t)m * p.ldy + col] = v;
    }
  }
}

template <bool NV, int M>
static int launch_m(Params p, cudaStream_t stream) {
  const int units = p.k >> 5;
  // Warps per pair of rows: one, unless the k range needs more than BATCH passes of 32 units; then the passes are
  // split over 2 or 4 warps so that all of a warp's loads are in flight at once.  (Splitting further to get more
  // warps for small matrices measured no better: every CTA converts the whole activation row.)
  const int iters = (units + 31) >> 5;
  int split = 1;
  while (split < WARPS && (iters + split - 1) / split > BATCH) split *= 2;
  p.ksplit = split;
  const size_t smem = (size_t)M * units * (64 + (NV ? 8 : 4));
  auto kern = fp4_gemv_kernel<NV, M>;
  static PerDevice attr_set;
  if (smem > 48 * 1024) {
    const int rc = opt_in_smem(attr_set, kern, (int)smem);
    if (rc != 0) return rc;
  }
  const int rows_per_cta = RW * WARPS / split;
  const unsigned grid = (unsigned)((p.n + rows_per_cta - 1) / rows_per_cta);
  // launched so that it may overlap the tail of the kernel before it (see the top of the kernel)
  static const int pdl = env_int("WUSH_B200_GEMV_PDL", 1);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(WARPS * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return (int)cudaLaunchKernelEx(&cfg, kern, p);
}

int max_rows() {
  static const int v = env_int("WUSH_B200_GEMV_MAX_M", 4);
  return v < 0 ? 0 : (v > 4 ? 4 : v);
}

int max_k() {
  static const int v = env_int("WUSH_B200_GEMV_MAX_K", 8192);
  return v;
}

int launch(bool nv, const uint8_t* a, const uint8_t* b, const uint8_t* sfa, const uint8_t* sfb, const float* alpha,
           const void* bias, const void* residual, int64_t ldr, void* y, int64_t ldy, int m, int n, int k,
           cudaStream_t stream) {
  Params p{a, b, sfa, sfb, alpha, (const __nv_bfloat16*)bias, (const __nv_bfloat16*)residual, (__nv_bfloat16*)y,
           ldr, ldy, n, k, k / (nv ? 16 : 32), 1};
  switch (m) {
    case 1: return nv ? launch_m<true, 1>(p, stream) : launch_m<false, 1>(p, stream);
    case 2: return nv ? launch_m<true, 2>(p, stream) : launch_m<false, 2>(p, stream);
    case 3: return nv ? launch_m<true, 3>(p, stream) : launch_m<false, 3>(p, stream);
    case 4: return nv ? launch_m<true, 4>(p, stream) : launch_m<false, 4>(p, stream);
    default: return WUSH_ERR_BAD_SHAPE;
  }
}

}  // namespace gemv
}  // namespace wush
