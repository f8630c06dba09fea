// Per-kernel launch preparation done once per (kernel, device) instead of on
// every launch: the opt-in to more than 48 KB of dynamic shared memory
// (an attribute of the kernel in the current device's context) and the
// compiled register count.
#pragma once
#include <cuda_runtime.h>

#include <map>
#include <mutex>
#include <utility>

namespace wave {

struct KernelInfo {
  int num_regs = 0;
};

// Sets cudaFuncAttributeMaxDynamicSharedMemorySize to `smem_bytes` for
// `kernel` on the current device the first time it is asked to, and returns
// the kernel's attributes from then on without touching the runtime.
template <typename Kernel> cudaError_t prepare_kernel(Kernel kernel, int smem_bytes, KernelInfo *info) {
  static std::mutex mu;
  static std::map<std::pair<const void *, int>, KernelInfo> seen;
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess)
    return err;
  const std::pair<const void *, int> key(reinterpret_cast<const void *>(kernel), dev);
  std::lock_guard<std::mutex> lock(mu);
  auto it = seen.find(key);
  if (it == seen.end()) {
    cudaFuncAttributes attr;
    if ((err = cudaFuncGetAttributes(&attr, kernel)) != cudaSuccess)
      return err;
    if ((err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes)) != cudaSuccess)
      return err;
    KernelInfo k;
    k.num_regs = attr.numRegs;
    it = seen.emplace(key, k).first;
  }
  if (info)
    *info = it->second;
  return cudaSuccess;
}

} // namespace wave
