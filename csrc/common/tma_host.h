// Host-side helpers: building CUtensorMap objects through the driver entry
// point obtained at run time (the extension does not link libcuda), and a
// small cache so that steady-state launches do not re-encode descriptors.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <stdexcept>
#include <string>
#include <unordered_map>

namespace oxb {

typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                    const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                    const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline PFN_encodeTiled get_encode_tiled() {
  static PFN_encodeTiled fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || p == nullptr) {
      throw std::runtime_error("oxb: cuTensorMapEncodeTiled is not available from this driver");
    }
    fn = reinterpret_cast<PFN_encodeTiled>(p);
  });
  return fn;
}

struct TmaKey {
  const void* ptr;
  uint64_t d0, d1, d2;
  uint64_t s1, s2;
  uint32_t b0, b1, b2;
  uint32_t dtype_swizzle;
  uint64_t d3 = 1, s3 = 0;
  uint32_t b3 = 1;
  bool operator==(const TmaKey& o) const {
    return ptr == o.ptr && d0 == o.d0 && d1 == o.d1 && d2 == o.d2 && s1 == o.s1 && s2 == o.s2 &&
           b0 == o.b0 && b1 == o.b1 && b2 == o.b2 && dtype_swizzle == o.dtype_swizzle && d3 == o.d3 &&
           s3 == o.s3 && b3 == o.b3;
  }
};
struct TmaKeyHash {
  size_t operator()(const TmaKey& k) const {
    uint64_t h = 1469598103934665603ull;
    auto mix = [&h](uint64_t v) {
      h ^= v;
      h *= 1099511628211ull;
    };
    mix(reinterpret_cast<uint64_t>(k.ptr));
    mix(k.d0); mix(k.d1); mix(k.d2); mix(k.s1); mix(k.s2);
    mix(k.b0); mix(k.b1); mix(k.b2); mix(k.dtype_swizzle); mix(k.d3); mix(k.s3); mix(k.b3);
    return static_cast<size_t>(h);
  }
};

// 2-D to 4-D tiled map over a tensor whose innermost dimension is contiguous.
// dims / box are innermost-first; strides are in bytes for dimensions 1, 2 and 3.
inline CUtensorMap make_tma_map(const void* ptr, CUtensorMapDataType dtype, int elem_bytes, int rank,
                                uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_bytes,
                                uint64_t stride2_bytes, uint32_t b0, uint32_t b1, uint32_t b2,
                                CUtensorMapSwizzle swizzle, uint64_t d3 = 1, uint64_t stride3_bytes = 0,
                                uint32_t b3 = 1) {
  static std::unordered_map<TmaKey, CUtensorMap, TmaKeyHash> cache;
  static std::mutex mu;
  TmaKey key{ptr, d0, d1, d2, stride1_bytes, stride2_bytes, b0, b1, b2,
             (static_cast<uint32_t>(dtype) << 8) | static_cast<uint32_t>(swizzle) |
                 (static_cast<uint32_t>(rank) << 24)};
  key.d3 = d3;
  key.s3 = stride3_bytes;
  key.b3 = b3;
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
  }
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0 || (stride1_bytes & 15) != 0 ||
      (rank >= 3 && (stride2_bytes & 15) != 0) || (rank == 4 && (stride3_bytes & 15) != 0) ||
      ((uint64_t)b0 * elem_bytes) % 16 != 0) {
    throw std::runtime_error(
        "oxb: TMA needs a 16-byte aligned base, strides and inner box extent (got ptr=" +
        std::to_string(reinterpret_cast<uintptr_t>(ptr)) + " stride1=" +
        std::to_string(stride1_bytes) + ")");
  }
  CUtensorMap map;
  cuuint64_t gdim[4] = {d0, d1, d2, d3};
  cuuint64_t gstr[3] = {stride1_bytes, stride2_bytes, stride3_bytes};
  cuuint32_t box[4] = {b0, b1, b2, b3};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = get_encode_tiled()(&map, dtype, static_cast<cuuint32_t>(rank), const_cast<void*>(ptr),
                                  gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    throw std::runtime_error("oxb: cuTensorMapEncodeTiled failed with code " + std::to_string(r));
  }
  {
    std::lock_guard<std::mutex> g(mu);
    if (cache.size() > 65536) cache.clear();
    cache.emplace(key, map);
  }
  return map;
}

}  // namespace oxb
