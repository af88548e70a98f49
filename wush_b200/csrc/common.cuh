// Small device/host helpers shared by the kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include <atomic>

#include "../../include/wush_b200.h"

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

// ---- per-device bookkeeping ----------------------------------------------------------------------
// A kernel's opt-in to more than 48 KB of dynamic shared memory, the number of clusters that fit and the
// address of a __device__ array all belong to ONE device.  A process may drive several GPUs (layers
// placed on cuda:0 and cuda:1), so everything of that kind is cached per device index, never in a plain
// function-static variable.
constexpr int kMaxDevices = 64;

// Index of the current device in [0, kMaxDevices), or -1.
inline int device_slot() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
  return dev;
}

// One int of state per device; zero-initialised when it has static storage (0 = "not set yet").
struct PerDevice {
  std::atomic<int> v[kMaxDevices];
  int get(int dev) const { return v[dev].load(std::memory_order_acquire); }
  void set(int dev, int x) { v[dev].store(x, std::memory_order_release); }
};

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per device and kernel; `flags` is a static
// PerDevice owned by the call site (one per kernel instantiation).  Racing first calls both set the
// attribute, which is idempotent.  Returns 0 or a cudaError_t.
template <class Kernel>
inline int opt_in_smem(PerDevice& flags, Kernel kernel, int bytes) {
  const int dev = device_slot();
  if (dev >= 0 && flags.get(dev)) return 0;
  const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) return (int)e;
  if (dev >= 0) flags.set(dev, 1);
  return 0;
}

// 0 when the current device is compute capability 10.x, WUSH_ERR_NOT_SM100 otherwise (the library holds
// sm_100a code only: a launch elsewhere would fail with "no kernel image"), or a positive cudaError_t.
inline int require_sm100() {
  static PerDevice seen;   // 1 = sm_100, 2 = something else
  const int dev = device_slot();
  if (dev < 0) {
    int d = 0;
    const cudaError_t e = cudaGetDevice(&d);
    return e != cudaSuccess ? (int)e : WUSH_ERR_NOT_SM100;
  }
  int s = seen.get(dev);
  if (!s) {
    int major = 0;
    const cudaError_t e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) return (int)e;
    s = major == 10 ? 1 : 2;
    seen.set(dev, s);
  }
  return s == 1 ? WUSH_OK : WUSH_ERR_NOT_SM100;
}

// The quantize kernels' device-side timeout word (fused_quantize.cu), after the caller synchronized: 0 = clear,
// WUSH_ERR_DEVICE_TIMEOUT = it was set (and has been cleared), > 0 = a cudaError_t.
int quantize_timeout_fetch_and_clear();

}  // namespace wush
