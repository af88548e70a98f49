// Scale-factor re-layout: row-major padded bytes -> 128x4 blocked tiles.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/wush_b200.h"
#include "common.cuh"

namespace wush {

// One thread per 4 output bytes (one row of one 128x4 tile = 4 consecutive groups).
__global__ void sf_to_blocked_kernel(const uint8_t* __restrict__ in, uint32_t* __restrict__ out, int64_t rows,
                                     int64_t cols, int64_t col_blocks, int64_t total_words) {
  for (int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; w < total_words;
       w += (int64_t)gridDim.x * blockDim.x) {
    // w indexes the blocked output: tile = w / 128, inside: (r % 32) * 4 + (r / 32 % 4)
    const int64_t tile = w >> 7;
    const int in_tile = (int)(w & 127);
    const int64_t rb = tile / col_blocks, cb = tile % col_blocks;
    const int64_t r = rb * 128 + (in_tile >> 2) + 32 * (in_tile & 3);
    uint32_t v = 0;
    if (r < rows) {
      const uint8_t* src = in + r * cols + cb * 4;
#pragma unroll
      for (int c = 0; c < 4; ++c)
        if (cb * 4 + c < cols) v |= (uint32_t)src[c] << (8 * c);
    }
    out[w] = v;
  }
}

}  // namespace wush

extern "C" int wush_sf_to_blocked(const uint8_t* in, uint8_t* out, int64_t rows, int64_t cols, void* stream) {
  if (!in || !out) return WUSH_ERR_NULL_POINTER;
  if (rows < 0 || cols < 0) return WUSH_ERR_BAD_SHAPE;
  if ((uintptr_t)out & 3) return WUSH_ERR_BAD_ALIGNMENT;
  const int64_t row_blocks = (rows + 127) / 128, col_blocks = (cols + 3) / 4;
  const int64_t words = row_blocks * col_blocks * 128;
  if (words == 0) return WUSH_OK;
  if (const int rc100 = wush::require_sm100()) return rc100;
  const int threads = 256;
  int64_t blocks = (words + threads - 1) / threads;
  const int64_t cap = (int64_t)wush::sm_count() * 16;
  if (blocks > cap) blocks = cap;
  wush::sf_to_blocked_kernel<<<(unsigned)blocks, threads, 0, (cudaStream_t)stream>>>(
      in, reinterpret_cast<uint32_t*>(out), rows, cols, col_blocks, words);
  return (int)cudaGetLastError();
}

extern "C" int wush_b200_arch(void) { return 100; }
