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

// Programmatic dependent launch of the kernels that support it (they call pdl_wait() before their
// first dependent access): process-wide switch, off until the embedding program turns it on.
inline bool& pdl_enabled() {
  static bool on = false;
  return on;
}

// One launch through cudaLaunchKernelEx. `pdl`: the kernel may become resident before the previous
// kernel of the stream has finished (only honoured when pdl_enabled()). `cooperative`: all CTAs
// resident at once; such a launch never takes the programmatic attribute.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                 cudaStream_t stream, bool pdl, bool cooperative, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  if (cooperative) {
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  } else if (pdl && pdl_enabled()) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

}  // namespace oxb
