// Per-device launch configuration shared by the launchers: SM count and the dynamic shared-memory
// opt-in of a kernel, both cached by device index (a process may drive several GPUs: data-parallel
// replicas or pipeline stages in one process).
#pragma once
#include <cuda_runtime.h>

#include <map>
#include <mutex>
#include <utility>

namespace oxb {

constexpr int kMaxDevices = 64;

inline int current_device() {
  int dev = 0;
  cudaGetDevice(&dev);
  return dev < 0 || dev >= kMaxDevices ? 0 : dev;
}

// Number of SMs of the current device.
inline int sm_count() {
  static int cached[kMaxDevices] = {};
  const int dev = current_device();
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 1;
    cached[dev] = n;
  }
  return cached[dev];
}

// Raises the dynamic shared-memory limit of `kernel` on the current device when `bytes` exceeds
// what was configured there so far (keyed by kernel address and device).
template <typename K>
inline void ensure_dynamic_smem(K kernel, size_t bytes) {
  static std::map<std::pair<const void*, int>, size_t> configured;
  static std::mutex mu;
  if (bytes <= 48 * 1024) return;
  const std::pair<const void*, int> key(reinterpret_cast<const void*>(kernel), current_device());
  std::lock_guard<std::mutex> g(mu);
  size_t& have = configured[key];
  if (bytes > have) {
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
    have = bytes;
  }
}

}  // namespace oxb
