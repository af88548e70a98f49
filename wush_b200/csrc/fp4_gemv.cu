// MXFP4 GEMM for decode-sized M (M <= 16) on sm_100a: Y[M,N] (bf16) = alpha * (A . sfa) (B . sfb)^T.
//
// With at most 16 activation rows the GEMM is one pass over the weights -- (N*K/2 + N*K/32) bytes against
// 2*M*N*K flops -- so it is bound by HBM, and the tcgen05 path (128-row tiles, split-K partial tiles in
// global memory and a second kernel to reduce them) spends most of its time on fixed costs.  This kernel
// streams the weights once:
//   * the activations (codes as they are, scales as fp32) are staged in shared memory once per CTA;
//   * a CTA of 16 warps works on 16/KS weight tiles of 8 rows at a time, KS warps sharing a tile along K; a warp
//     loads its weight codes straight into registers with 16-byte loads, eight 128-element chunks (4 KB per
//     warp) in flight and the next batch requested before the current one is consumed, transposes the words
//     inside every quad of lanes so that a lane holds 8 codes of each of the chunk's four scale groups, and
//     converts them with cvt.rn.f16x2.e2m1x2;
//   * products run on the warp-level tensor-core MMA m16n8k16 (f16 x f16 -> fp32; E2M1 values are exact in
//     f16).  The k-order inside an MMA is permuted so that all 16 k-values belong to ONE scale group: the two
//     MMAs of a group accumulate into a scratch fragment, which is folded into the running sum with the
//     product of the two group scales in fp32 -- no scale ever passes through f16;
//   * the KS partial sums of a tile are added through shared memory and written as bf16.
// Nothing is written to global memory but the result, and there is no second launch.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/wush_b200.h"
#include "common.cuh"

namespace wush {
namespace gemv {

constexpr int WARPS = 16, THREADS = WARPS * 32;
constexpr int CHUNK = 128;            // K elements per step: 64 bytes of codes per row, 4 scale groups = 1 scale atom
constexpr int BATCH = 8;              // chunks a warp keeps in flight: 8 x 16 bytes per lane

struct Params {
  const uint8_t* a;     // [m, k/2]
  const uint8_t* sfa;   // blocked scales of A (one 128-row block)
  const uint8_t* b;     // [n, k/2]
  const uint8_t* sfb;   // blocked scales of B
  const float* alpha;
  __nv_bfloat16* y;     // [m, n]
  int m, n, k;
  int chunks;           // k / 128 == scale atoms per row block
  int n_tiles;          // n / 8
  int code_stride;      // bytes per staged activation row (k/2 + 16: rows land in different banks)
  int sx_stride;        // floats per staged scale row (k/32 + 1)
};

// 8 packed E2M1 codes -> four f16x2 (element 2i of a byte pair is the low nibble).  One byte per conversion,
// extracted with integer shifts: unpacking a 32-bit register into four .b8 registers in one PTX block came back
// with byte 2 replaced by byte 0 on this toolchain.
__device__ __forceinline__ uint32_t cvt_e2m1x2(uint32_t byte) {
  uint32_t h;
  const unsigned short t = (unsigned short)byte;
  asm("{\n.reg .b8 lo, hi;\nmov.b16 {lo, hi}, %1;\ncvt.rn.f16x2.e2m1x2 %0, lo;\n}\n" : "=r"(h) : "h"(t));
  return h;
}
__device__ __forceinline__ void cvt_e2m1x8(uint32_t w, uint32_t (&h)[4]) {
  h[0] = cvt_e2m1x2(w & 0xFF);
  h[1] = cvt_e2m1x2((w >> 8) & 0xFF);
  h[2] = cvt_e2m1x2((w >> 16) & 0xFF);
  h[3] = cvt_e2m1x2(w >> 24);
}

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float e8m0_to_float(uint32_t byte) { return __uint_as_float(byte << 23); }   // 2^(byte-127)

// 4 x 4 transposition of 32-bit words among the four lanes of a quad: lane q gives word j to lane j and ends up
// with word q of lanes 0..3 (in lane order).
__device__ __forceinline__ void quad_transpose(uint4& v, int q) {
  uint32_t w[4] = {v.x, v.y, v.z, v.w};
  // stage 1: exchange with lane q ^ 1 the words whose bit 0 differs from ours
  {
    const bool odd = q & 1;
    const uint32_t s0 = odd ? w[0] : w[1], s1 = odd ? w[2] : w[3];
    const uint32_t r0 = __shfl_xor_sync(0xffffffffu, s0, 1), r1 = __shfl_xor_sync(0xffffffffu, s1, 1);
    if (odd) { w[0] = r0; w[2] = r1; } else { w[1] = r0; w[3] = r1; }
  }
  // stage 2: exchange with lane q ^ 2 the words whose bit 1 differs from ours
  {
    const bool up = q & 2;
    const uint32_t s0 = up ? w[0] : w[2], s1 = up ? w[1] : w[3];
    const uint32_t r0 = __shfl_xor_sync(0xffffffffu, s0, 2), r1 = __shfl_xor_sync(0xffffffffu, s1, 2);
    if (up) { w[0] = r0; w[1] = r1; } else { w[2] = r0; w[3] = r1; }
  }
  v = make_uint4(w[0], w[1], w[2], w[3]);
}

// One work item of a warp: weight tile `tile` (8 rows), chunks [cb, ce) with ce - cb <= BATCH.  Lane (row lane/4,
// quarter q) loads the 16 bytes = one scale group q of every chunk (a quad reads the row's 64 contiguous bytes),
// and the scale words of chunks q and q + 4 of the batch for its row.
struct Batch {
  uint4 w[BATCH];
  uint32_t s[2];
};

__device__ __forceinline__ void issue_batch(const Params& p, Batch& l, int tile, int cb, int ce, int lane) {
  const int q = lane & 3, row = tile * 8 + (lane >> 2);
  const uint8_t* src = p.b + (int64_t)row * (p.k / 2) + q * 16;
#pragma unroll
  for (int j = 0; j < BATCH; ++j)
    if (cb + j < ce) l.w[j] = __ldg(reinterpret_cast<const uint4*>(src + (int64_t)(cb + j) * (CHUNK / 2)));
  const int64_t sbase = (int64_t)(row >> 7) * p.chunks * 512 + (row & 31) * 16 + ((row & 127) >> 5) * 4;
#pragma unroll
  for (int e = 0; e < 2; ++e)
    if (cb + q + 4 * e < ce) l.s[e] = __ldg(reinterpret_cast<const uint32_t*>(p.sfb + sbase + (int64_t)(cb + q + 4 * e) * 512));
}

template <int KS>      // warps sharing one weight tile (k-slices); WARPS / KS tiles are in progress per CTA
__global__ void __launch_bounds__(THREADS, 1) fp4_gemv_mx_kernel(const Params p) {
  constexpr int TILES = WARPS / KS;
  extern __shared__ __align__(16) uint8_t smem[];
  uint8_t* xs = smem;                                                        // [16][code_stride] activation codes
  float* sx = reinterpret_cast<float*>(smem + 16 * p.code_stride);           // [16][sx_stride] activation scales
  float* part = sx + 16 * p.sx_stride;                                       // [WARPS][32][4] partial sums
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q = lane & 3, r = lane >> 2;
  const int ks = warp % KS, slot = warp / KS;
  const int c0 = (int)((int64_t)ks * p.chunks / KS), c1 = (int)((int64_t)(ks + 1) * p.chunks / KS);
  const int n_batches = (c1 - c0 + BATCH - 1) / BATCH;       // per tile, for this warp
  const int stride_tiles = gridDim.x * TILES;
  const int tile0 = blockIdx.x * TILES + slot;
  const int rounds = (p.n_tiles + stride_tiles - 1) / stride_tiles;   // the same for every warp of the grid

  // the first weights are already on their way while the activations are staged
  Batch cur, nxt;
  if (tile0 < p.n_tiles && n_batches > 0) issue_batch(p, cur, tile0, c0, min(c0 + BATCH, c1), lane);

  const int row_bytes = p.k / 2;
  for (int i = threadIdx.x; i < 16 * (row_bytes / 16); i += THREADS) {
    const int row = i / (row_bytes / 16), col = i % (row_bytes / 16);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < p.m) v = __ldg(reinterpret_cast<const uint4*>(p.a + (int64_t)row * row_bytes) + col);
    *reinterpret_cast<uint4*>(xs + row * p.code_stride + col * 16) = v;
  }
  const int groups = p.k / 32;
  for (int i = threadIdx.x; i < 16 * groups; i += THREADS) {
    const int row = i / groups, g = i % groups;
    sx[row * p.sx_stride + g] = row < p.m ? e8m0_to_float(p.sfa[(int64_t)(g >> 2) * 512 + row * 16 + (g & 3)]) : 0.0f;
  }
  __syncthreads();
  const float alpha = *p.alpha;

  for (int round = 0; round < rounds; ++round) {
    const int tile = tile0 + round * stride_tiles;
    const bool live = tile < p.n_tiles;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (live) {
      for (int bi = 0; bi < n_batches; ++bi) {
        const int cb = c0 + bi * BATCH, ce = min(cb + BATCH, c1);
        // the next batch (of this tile, or the first of this warp's next tile) while this one is consumed
        if (bi + 1 < n_batches) issue_batch(p, nxt, tile, ce, min(ce + BATCH, c1), lane);
        else if (tile + stride_tiles < p.n_tiles) issue_batch(p, nxt, tile + stride_tiles, c0, min(c0 + BATCH, c1), lane);
#pragma unroll
        for (int j = 0; j < BATCH; ++j) {
          if (cb + j < ce) {
            const int c = cb + j;
            uint4 wv = cur.w[j];
            quad_transpose(wv, q);          // now: codes 8q..8q+7 of groups 0..3 of the chunk
            const uint32_t wg[4] = {wv.x, wv.y, wv.z, wv.w};
            // scale words of the chunk for the weight rows of this lane's output columns 2q and 2q+1
            const uint32_t sword = cur.s[j >> 2];
            const uint32_t sw0 = __shfl_sync(0xffffffffu, sword, (2 * q) * 4 + (j & 3));
            const uint32_t sw1 = __shfl_sync(0xffffffffu, sword, (2 * q + 1) * 4 + (j & 3));
            const uint8_t* xr = xs + r * p.code_stride + c * (CHUNK / 2) + q * 4;
            const float* sr = sx + r * p.sx_stride + c * 4;
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint32_t a_lo[4], a_hi[4], b[4];      // rows r and r + 8: codes 8q..8q+7 of the group as four f16x2
              cvt_e2m1x8(*reinterpret_cast<const uint32_t*>(xr + g * 16), a_lo);
              cvt_e2m1x8(*reinterpret_cast<const uint32_t*>(xr + 8 * p.code_stride + g * 16), a_hi);
              cvt_e2m1x8(wg[g], b);
              float tmp[4] = {0.0f, 0.0f, 0.0f, 0.0f};
              mma_f16(tmp, a_lo[0], a_hi[0], a_lo[1], a_hi[1], b[0], b[1]);   // codes 8q .. 8q+3 of every quarter
              mma_f16(tmp, a_lo[2], a_hi[2], a_lo[3], a_hi[3], b[2], b[3]);   // codes 8q+4 .. 8q+7
              const float s_lo = sr[g], s_hi = sr[8 * p.sx_stride + g];
              const float w0 = e8m0_to_float((sw0 >> (8 * g)) & 0xFF), w1 = e8m0_to_float((sw1 >> (8 * g)) & 0xFF);
              acc[0] += tmp[0] * (s_lo * w0);
              acc[1] += tmp[1] * (s_lo * w1);
              acc[2] += tmp[2] * (s_hi * w0);
              acc[3] += tmp[3] * (s_hi * w1);
            }
          }
        }
        cur = nxt;
      }
    }
    // add the KS k-slices of every tile in progress and store
    *reinterpret_cast<float4*>(part + (warp * 32 + lane) * 4) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    __syncthreads();
    for (int e = threadIdx.x; e < TILES * 128; e += THREADS) {
      const int sl = e >> 7, rem = e & 127;
      float sum = 0.0f;
#pragma unroll
      for (int w = 0; w < KS; ++w) sum += part[(sl * KS + w) * 128 + rem];
      const int i = rem & 3, ln = rem >> 2;
      const int tl = blockIdx.x * TILES + sl + round * stride_tiles;
      const int row = (ln >> 2) + ((i & 2) ? 8 : 0), col = tl * 8 + 2 * (ln & 3) + (i & 1);
      if (tl < p.n_tiles && row < p.m) p.y[(int64_t)row * p.n + col] = __float2bfloat16_rn(sum * alpha);
    }
    __syncthreads();
  }
}

// Launch when the shape qualifies; returns kNotApplicable when the caller should use the tcgen05 path instead.
constexpr int kNotApplicable = -1000;
int launch_mx(const uint8_t* a, const uint8_t* b, const uint8_t* sfa, const uint8_t* sfb, const float* alpha, void* y,
              int64_t m, int64_t n, int64_t k, cudaStream_t stream) {
  static const int enabled = env_int("WUSH_B200_GEMV", 0);   // off until verified on hardware
  if (!enabled || m > 16 || m < 1 || k % CHUNK != 0 || n % 8 != 0) return kNotApplicable;
  Params p{a, sfa, b, sfb, alpha, (__nv_bfloat16*)y, (int)m, (int)n, (int)k, (int)(k / CHUNK), (int)(n / 8),
           (int)(k / 2 + 16), (int)(k / 32 + 1)};
  const int sms = sm_count();
  const size_t smem = (size_t)16 * p.code_stride + (size_t)16 * p.sx_stride * 4 + (size_t)WARPS * 512;
  if (smem > 200 * 1024) return kNotApplicable;
  // k-slices per tile: 4 (4 tiles per CTA and round) unless 8 or 16 balance the rounds of the grid better
  int ks = 4;
  double best = 0.0;
  for (int cand : {4, 8, 16}) {
    const int64_t per_round = (int64_t)sms * (WARPS / cand);
    const int64_t rounds = (p.n_tiles + per_round - 1) / per_round;
    const double eff = (double)p.n_tiles / (double)(rounds * per_round);
    if (eff > best + 0.05 && p.chunks >= cand) { best = eff; ks = cand; }
  }
  const int tiles_per_cta = WARPS / ks;
  const int64_t ctas = (p.n_tiles + tiles_per_cta - 1) / tiles_per_cta;
  const int grid = (int)(ctas < sms ? ctas : sms);
  static bool attr_set[3] = {false, false, false};
  auto launch = [&](auto kern, int slot) -> int {
    if (!attr_set[slot]) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      if (e != cudaSuccess) return (int)e;
      attr_set[slot] = true;
    }
    kern<<<grid, THREADS, smem, stream>>>(p);
    return (int)cudaGetLastError();
  };
  if (ks == 16) return launch(fp4_gemv_mx_kernel<16>, 0);
  if (ks == 8) return launch(fp4_gemv_mx_kernel<8>, 1);
  return launch(fp4_gemv_mx_kernel<4>, 2);
}

}  // namespace gemv
}  // namespace wush
