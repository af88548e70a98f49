// Small device/host helpers shared by the kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

namespace wush {

// 16-byte read-only load that does not allocate in L1 (streamed once).
template <typename T>
__device__ __forceinline__ uint4 ld_nc_v4(const T* ptr) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(ptr));
  return v;
}

// Integer tuning knob read once from the environment (for sweeps); `fallback` otherwise.
inline int env_int(const char* name, int fallback) {
  const char* s = getenv(name);
  if (!s || !*s) return fallback;
  return atoi(s);
}

inline int sm_count() {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms;
}

}  // namespace wush
