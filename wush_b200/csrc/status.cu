// Device-side error reporting.  Every kernel that waits on an mbarrier does so with a poll limit; a wait that
// runs out raises a flag, the CTA unwinds (frees its tensor memory) and the kernel sets the caller's status
// word.  wush_status_check turns that word into the WUSH_ERR_DEVICE_TIMEOUT return code;
// wush_selftest_bounded_wait exercises the mechanism with a barrier nothing ever arrives on.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/wush_b200.h"
#include "common.cuh"
#include "sm100.cuh"

namespace wush {
__global__ void bounded_wait_selftest_kernel(int* status, uint32_t max_polls) {
  __shared__ uint64_t bar;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    sm100::mbar_init(sm100::smem_u32(&bar), 1);
    abort_flag = 0;
    sm100::mbar_init_fence();
  }
  __syncthreads();
  // phase 0 of the barrier never completes: nothing arrives on it
  if (threadIdx.x == 32) sm100::mbar_wait_limited(sm100::smem_u32(&bar), 0, &abort_flag, max_polls);
  __syncthreads();
  // the other threads see the flag and leave, as the roles of the GEMM kernels do
  if (threadIdx.x == 0 && abort_flag && status) atomicExch(status, 1);
}

}  // namespace wush

extern "C" int wush_status_check(int* status_dev, void* stream) {
  if (!status_dev) return WUSH_ERR_NULL_POINTER;
  int host = 0;
  cudaError_t e = cudaMemcpyAsync(&host, status_dev, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
  if (e != cudaSuccess) return (int)e;
  // the quantize kernels have no status argument: their bulk-copy waits report through a word inside the library
  const int quant = wush::quantize_timeout_fetch_and_clear();
  if (quant > 0) return quant;                       // a cudaError_t
  if (host == 0 && quant == 0) return WUSH_OK;
  if (host != 0) {
    e = cudaMemsetAsync(status_dev, 0, sizeof(int), (cudaStream_t)stream);
    if (e != cudaSuccess) return (int)e;
  }
  return WUSH_ERR_DEVICE_TIMEOUT;
}

extern "C" int wush_selftest_bounded_wait(int* status_dev, int max_polls, void* stream) {
  if (!status_dev) return WUSH_ERR_NULL_POINTER;
  if (max_polls <= 0 || max_polls > (1 << 16)) return WUSH_ERR_BAD_FLAG;
  const int rc = wush::require_sm100();
  if (rc != 0) return rc;
  wush::bounded_wait_selftest_kernel<<<1, 64, 0, (cudaStream_t)stream>>>(status_dev, (uint32_t)max_polls);
  return (int)cudaGetLastError();
}
