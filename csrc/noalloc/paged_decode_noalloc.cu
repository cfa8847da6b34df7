// Allocation-free entry point of the paged split-KV decode attention: the split partials live
// in a file-scope __device__ array of this library instead of caller-provided buffers.
// See oxb_noalloc.h for who needs this and for the limits.
#include "oxb_noalloc.h"

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <initializer_list>

#include <mutex>

#include "../kernels/attn.cuh"

namespace {

constexpr size_t kScratchFloats = OXB_NOALLOC_SCRATCH_BYTES / sizeof(float);

// Device-resident scratch. In host code this name is only a handle for the runtime, never an
// address a kernel may be given; the address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) float g_scratch[kScratchFloats];

constexpr int kMaxDevices = 64;
float* g_scratch_ptr[kMaxDevices] = {nullptr};
std::mutex g_mu;

__global__ void set_int_kernel(int* dst, int value) { *dst = value; }

int fail(int code, char* err, int err_len, const char* msg) {
  if (err != nullptr && err_len > 0) snprintf(err, static_cast<size_t>(err_len), "%s", msg);
  return code;
}

}  // namespace

extern "C" __attribute__((visibility("default"))) int oxb_paged_decode_noalloc(
    const void* q, long long q_stride, const void* k_cache, const void* v_cache,
    const int* block_tables, const int* seq_lens, void* out, long long out_stride, int batch, int hq,
    int hkv, int head_dim, int num_blocks, int max_blocks, int pages_per_split, int max_splits,
    int window, float scale, void* stream, int* status, char* err, int err_len) {
  if (q == nullptr || k_cache == nullptr || v_cache == nullptr || block_tables == nullptr ||
      seq_lens == nullptr || out == nullptr)
    return fail(OXB_NOALLOC_BAD_ARGUMENT, err, err_len, "oxb_paged_decode_noalloc: null pointer argument");
  if (batch <= 0 || hq <= 0 || hkv <= 0 || hq % hkv != 0 || hq / hkv > 16 ||
      (head_dim != 64 && head_dim != 128) || num_blocks <= 0 || max_blocks <= 0 || pages_per_split < 1 ||
      max_splits < 1 || window < 0)
    return fail(OXB_NOALLOC_BAD_ARGUMENT, err, err_len,
                "oxb_paged_decode_noalloc: need batch, heads, num_blocks, max_blocks > 0, hq % hkv == 0, "
                "group <= 16, head_dim 64 or 128, pages_per_split >= 1, max_splits >= 1, window >= 0");
  if (hkv > 65535 || max_splits > 65535)
    return fail(OXB_NOALLOC_BAD_ARGUMENT, err, err_len,
                "oxb_paged_decode_noalloc: hkv and max_splits are grid dimensions (<= 65535)");
  // the kernels read q, K and V and write out with 16-byte accesses
  const uintptr_t align_bits = reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_cache) |
                               reinterpret_cast<uintptr_t>(v_cache) | reinterpret_cast<uintptr_t>(out);
  if ((align_bits & 15) != 0 || (reinterpret_cast<uintptr_t>(block_tables) & 3) != 0 ||
      (reinterpret_cast<uintptr_t>(seq_lens) & 3) != 0 ||
      (status != nullptr && (reinterpret_cast<uintptr_t>(status) & 3) != 0))
    return fail(OXB_NOALLOC_BAD_ARGUMENT, err, err_len,
                "oxb_paged_decode_noalloc: q, k_cache, v_cache and out must be 16-byte aligned "
                "(block_tables, seq_lens, status 4-byte aligned)");
  const long long row = static_cast<long long>(hq) * head_dim;
  if (q_stride < row || out_stride < row || (q_stride & 7) != 0 || (out_stride & 7) != 0)
    return fail(OXB_NOALLOC_BAD_ARGUMENT, err, err_len,
                "oxb_paged_decode_noalloc: q_stride and out_stride must be multiples of 8 elements and "
                "at least hq * head_dim");
  // batch * hq * max_splits * (head_dim + 2) + 64 floats, every factor checked against the scratch
  // size before it is multiplied in, so the product cannot wrap
  size_t rows_total = 1;
  for (const size_t f : {static_cast<size_t>(batch), static_cast<size_t>(hq), static_cast<size_t>(max_splits)}) {
    if (f > kScratchFloats || rows_total > kScratchFloats / f) {
      rows_total = kScratchFloats;  // certainly too large
      break;
    }
    rows_total *= f;
  }
  const size_t per_row = static_cast<size_t>(head_dim) + 2;
  if (rows_total > (kScratchFloats - 64) / per_row) {
    char msg[256];
    snprintf(msg, sizeof(msg),
             "oxb_paged_decode_noalloc: batch*hq*max_splits*(head_dim+2)+64 floats exceeds the "
             "built-in scratch of %zu floats (%u MiB); lower batch or max_splits",
             kScratchFloats, OXB_NOALLOC_SCRATCH_BYTES >> 20);
    return fail(OXB_NOALLOC_TOO_LARGE, err, err_len, msg);
  }
  const size_t n_o = rows_total * static_cast<size_t>(head_dim);

  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return fail(OXB_NOALLOC_CUDA_ERROR, err, err_len, "oxb_paged_decode_noalloc: cudaGetDevice failed");
  float* base = nullptr;
  {
    // first call on this device: resolve the device address of the scratch array (no allocation)
    std::lock_guard<std::mutex> lock(g_mu);
    if (g_scratch_ptr[dev] == nullptr) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_scratch);
      if (e != cudaSuccess || p == nullptr) {
        char msg[200];
        snprintf(msg, sizeof(msg), "oxb_paged_decode_noalloc: cudaGetSymbolAddress failed: %s",
                 cudaGetErrorString(e));
        return fail(OXB_NOALLOC_CUDA_ERROR, err, err_len, msg);
      }
      g_scratch_ptr[dev] = static_cast<float*>(p);
    }
    base = g_scratch_ptr[dev];
  }

  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // layout: [0, 64) header (pages_per_split), then the partial outputs, then (max, sum) pairs
  int* pps = reinterpret_cast<int*>(base);
  set_int_kernel<<<1, 1, 0, s>>>(pps, pages_per_split);
  e = cudaPeekAtLastError();
  if (e != cudaSuccess) {
    char msg[200];
    snprintf(msg, sizeof(msg), "oxb_paged_decode_noalloc: launch failed: %s", cudaGetErrorString(e));
    cudaGetLastError();
    return fail(OXB_NOALLOC_CUDA_ERROR, err, err_len, msg);
  }

  oxb::DecodeAttnParams p{};
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.q_stride = q_stride;
  p.k_cache = static_cast<const __nv_bfloat16*>(k_cache);
  p.v_cache = static_cast<const __nv_bfloat16*>(v_cache);
  p.block_tables = block_tables;
  p.seq_lens = seq_lens;
  p.pages_per_split = pps;
  p.part_o = base + 64;
  p.part_ml = base + 64 + n_o;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.out_stride = out_stride;
  p.max_blocks = max_blocks;
  p.Hq = hq;
  p.Hkv = hkv;
  p.max_splits = max_splits;
  p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.num_blocks = num_blocks;  // block ids are always bounded on this path
  p.status = status;
  e = oxb::launch_paged_decode(p, batch, head_dim, s);  // the merge is skipped if the first launch failed
  cudaGetLastError();
  if (e != cudaSuccess) {
    char msg[200];
    snprintf(msg, sizeof(msg), "oxb_paged_decode_noalloc: launch failed: %s", cudaGetErrorString(e));
    return fail(OXB_NOALLOC_CUDA_ERROR, err, err_len, msg);
  }
  return OXB_NOALLOC_OK;
}
