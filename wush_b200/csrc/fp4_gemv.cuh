// Decode path of the block-scaled FP4 product (1..4 activation rows): see fp4_gemv.cu.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

namespace wush {
namespace gemv {

// largest number of activation rows the matrix-vector kernel takes (0 switches it off; WUSH_B200_GEMV_MAX_M)
int max_rows();
// largest k it takes: beyond it the tensor-core path measured faster (WUSH_B200_GEMV_MAX_K)
int max_k();

// Arguments as for the GEMM entry points, already validated by the caller.  Returns 0 or a cudaError_t.
int launch(bool nv, const uint8_t* a, const uint8_t* b, const uint8_t* sfa, const uint8_t* sfb, const float* alpha,
           const void* bias, const void* residual, int64_t ldr, void* y, int64_t ldy, int m, int n, int k,
           cudaStream_t stream);

}  // namespace gemv
}  // namespace wush
