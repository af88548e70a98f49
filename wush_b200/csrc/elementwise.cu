// The element-wise neighbours of the quantized linear layers in a decoder block, as single HBM passes:
//   row_sumsq   sum of squares of every row of a bf16 matrix in fp32 (the reduction of RMSNorm; with a column-sharded
//               residual stream the per-GPU partial sums are added across GPUs before the scaling is applied, which
//               the fused quantize kernel does on the fly: see its row_scale / col_scale arguments)
//   swiglu      act = bf16(silu(gate)) * up, the input of down_proj
// Both are memory-bound: 16-byte loads, one warp (row_sumsq) or one thread per 8 elements (swiglu).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/wush_b200.h"
#include "common.cuh"

namespace wush {

__global__ void __launch_bounds__(256) row_sumsq_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, float* __restrict__ out,
                                                        int64_t rows, int64_t cols) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < rows; r += warps) {
    const __nv_bfloat16* row = x + r * ldx;
    float acc = 0.0f;
    for (int64_t c = lane * 8; c < cols; c += 256) {      // cols % 8 == 0
      const uint4 v = ld_nc_v4(row + c);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
        acc = fmaf(f.x, f.x, acc);
        acc = fmaf(f.y, f.y, acc);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) out[r] = acc;
  }
}

__device__ __forceinline__ float silu_f(float v) {
  // v * sigmoid(v) with the hardware exponential and reciprocal (about 2 ulp in fp32, below the bf16 rounding that follows)
  return v * __frcp_rn(1.0f + __expf(-v));
}

__global__ void __launch_bounds__(256) swiglu_kernel(const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ up,
                                                     int64_t ld_in, __nv_bfloat16* __restrict__ out, int64_t ld_out,
                                                     int64_t rows, int64_t cols8) {
  const int64_t total = rows * cols8;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / cols8, c = (i - r * cols8) * 8;
    const uint4 g = ld_nc_v4(gate + r * ld_in + c), u = ld_nc_v4(up + r * ld_in + c);
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
    uint32_t ow[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 gf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gw[k]));
      const __nv_bfloat162 s = __floats2bfloat162_rn(silu_f(gf.x), silu_f(gf.y));      // silu rounds to bf16 ...
      const __nv_bfloat162 p = __hmul2(s, *reinterpret_cast<const __nv_bfloat162*>(&uw[k]));   // ... then the product does
      ow[k] = *reinterpret_cast<const uint32_t*>(&p);
    }
    *reinterpret_cast<uint4*>(out + r * ld_out + c) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
  }
}

}  // namespace wush

extern "C" int wush_row_sumsq(const void* x, int64_t ldx, float* out, int64_t rows, int64_t cols, void* stream) {
  if (!x || !out) return WUSH_ERR_NULL_POINTER;
  if (rows < 0 || cols <= 0 || cols % 8 != 0 || ldx < cols || ldx % 8 != 0) return WUSH_ERR_BAD_SHAPE;
  if ((uintptr_t)x & 15) return WUSH_ERR_BAD_ALIGNMENT;
  if (rows == 0) return WUSH_OK;
  if (const int rc = wush::require_sm100()) return rc;
  int64_t blocks = (rows + 7) / 8;
  const int64_t cap = (int64_t)wush::sm_count() * 8;
  if (blocks > cap) blocks = cap;
  wush::row_sumsq_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, ldx, out, rows, cols);
  return (int)cudaGetLastError();
}

extern "C" int wush_swiglu(const void* gate, const void* up, int64_t ld_in, void* out, int64_t ld_out, int64_t rows,
                           int64_t cols, void* stream) {
  if (!gate || !up || !out) return WUSH_ERR_NULL_POINTER;
  if (rows < 0 || cols <= 0 || cols % 8 != 0 || ld_in < cols || ld_in % 8 != 0 || ld_out < cols || ld_out % 8 != 0)
    return WUSH_ERR_BAD_SHAPE;
  if (((uintptr_t)gate & 15) || ((uintptr_t)up & 15) || ((uintptr_t)out & 15)) return WUSH_ERR_BAD_ALIGNMENT;
  if (rows == 0) return WUSH_OK;
  if (const int rc = wush::require_sm100()) return rc;
  const int64_t total = rows * (cols / 8);
  int64_t blocks = (total + 255) / 256;
  const int64_t cap = (int64_t)wush::sm_count() * 16;
  if (blocks > cap) blocks = cap;
  wush::swiglu_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)gate, (const __nv_bfloat16*)up, ld_in, (__nv_bfloat16*)out, ld_out, rows, cols / 8);
  return (int)cudaGetLastError();
}
