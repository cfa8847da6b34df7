// bf16 GEMV for small batches on one GPU: y[m, n] = sum_k W[n, k] x[m, k], M <= 8.
//
// One warp owns two weight rows and walks K with 16-byte loads (8 lanes cover one 128-byte run of a
// row, the loop is unrolled so that a warp keeps 2 x 2 KB of weights in flight); the activation
// rows are re-read from L1/L2. Weights may be row-major or in the tile-major layout of the tcgen05
// GEMM. With `swiglu` the two rows of a warp are a gate row and its up row (weights interleaved in
// units of 32 rows), so SiLU(gate) * up is formed in the warp and written as one output column.
// Covers the reference's B=1 decode GEMVs for unquantised weights (oxide-backend-cuda
// launch_wrappers.cu:202-247 dispatches cuBLAS for them).
#include "gemv_bf16.cuh"

#include "../common/device_info.h"
#include "../common/sm100.cuh"

namespace oxb {

namespace {

constexpr int kWarpsPerCta = 8;

__device__ __forceinline__ float gemv_act(float x, int act) {
  if (act == 0) return x / (1.f + __expf(-x));
  return 0.5f * x * (1.f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
}

template <int MB>
__global__ void __launch_bounds__(kWarpsPerCta * 32) gemv_bf16_kernel(const GemvParams p) {
  pdl_wait();  // the activation rows come from the kernel before this one
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pair = blockIdx.x * kWarpsPerCta + warp;  // index of this warp's row pair
  const int n_pairs = p.N >> 1;
  if (pair >= n_pairs) return;
  int rows[2];
  if (p.swiglu) {
    rows[0] = (pair >> 5) * 64 + (pair & 31);  // gate row; its up row is 32 further
    rows[1] = rows[0] + 32;
  } else {
    rows[0] = 2 * pair;
    rows[1] = 2 * pair + 1;
  }
  const int kt_count = p.K >> 6;
  const __nv_bfloat16* wbase[2];
#pragma unroll
  for (int t = 0; t < 2; ++t)
    wbase[t] = p.tiled ? p.w + (static_cast<long long>(rows[t] >> 7) * kt_count) * 8192 + (rows[t] & 127) * 64
                       : p.w + static_cast<long long>(rows[t]) * p.K;
  float acc[2][MB];
#pragma unroll
  for (int t = 0; t < 2; ++t)
#pragma unroll
    for (int m = 0; m < MB; ++m) acc[t][m] = 0.f;

  const int chunks = p.K >> 3;  // 16-byte chunks per row
#pragma unroll 4
  for (int c = lane; c < chunks; c += 32) {
    const int k = c << 3;
    // tile-major: k-tile (k / 64) lives 128 * 64 elements after the previous one
    const long long off = p.tiled ? static_cast<long long>(k >> 6) * 8192 + (k & 63) : k;
    uint4 w[2];
#pragma unroll
    for (int t = 0; t < 2; ++t) w[t] = __ldg(reinterpret_cast<const uint4*>(wbase[t] + off));
#pragma unroll
    for (int m = 0; m < MB; ++m) {
      const int mm = m < p.M ? m : p.M - 1;
      const uint4 xv = __ldg(reinterpret_cast<const uint4*>(p.x + static_cast<long long>(mm) * p.ldx + k));
      const __nv_bfloat162* xh = reinterpret_cast<const __nv_bfloat162*>(&xv);
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        const __nv_bfloat162* wh = reinterpret_cast<const __nv_bfloat162*>(&w[t]);
        float s = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 a = __bfloat1622float2(wh[e]), b = __bfloat1622float2(xh[e]);
          s += a.x * b.x + a.y * b.y;
        }
        acc[t][m] += s;
      }
    }
  }
  pdl_launch_dependents();  // the weight stream is done: the next kernel may become resident
#pragma unroll
  for (int m = 0; m < MB; ++m) {
    float v0 = warp_sum(acc[0][m]), v1 = warp_sum(acc[1][m]);
    if (lane != 0 || m >= p.M) continue;
    if (p.bias != nullptr) {
      v0 += __bfloat162float(p.bias[rows[0]]);
      v1 += __bfloat162float(p.bias[rows[1]]);
    }
    if (p.swiglu) {
      const float y = gemv_act(v0, p.act) * v1;
      const long long o = static_cast<long long>(m) * p.ldo + pair;
      if (p.out_f32 != nullptr) p.out_f32[o] = y;
      else p.out_bf16[o] = __float2bfloat16(y);
    } else {
      const long long o = static_cast<long long>(m) * p.ldo + rows[0];
      if (p.out_f32 != nullptr) {
        p.out_f32[o] = v0;
        p.out_f32[o + 1] = v1;
      } else {
        p.out_bf16[o] = __float2bfloat16(v0);
        p.out_bf16[o + 1] = __float2bfloat16(v1);
      }
    }
  }
}

}  // namespace

void launch_gemv_bf16(const GemvParams& p, cudaStream_t stream) {
  if (p.M <= 0 || p.N <= 0) return;
  const int n_pairs = p.N >> 1;
  const int grid = (n_pairs + kWarpsPerCta - 1) / kWarpsPerCta;
  if (p.M == 1) launch_kernel(gemv_bf16_kernel<1>, dim3(grid), dim3(kWarpsPerCta * 32), 0, stream, /*pdl=*/true, false, p);
  else if (p.M == 2) launch_kernel(gemv_bf16_kernel<2>, dim3(grid), dim3(kWarpsPerCta * 32), 0, stream, /*pdl=*/true, false, p);
  else if (p.M <= 4) launch_kernel(gemv_bf16_kernel<4>, dim3(grid), dim3(kWarpsPerCta * 32), 0, stream, /*pdl=*/true, false, p);
  else launch_kernel(gemv_bf16_kernel<8>, dim3(grid), dim3(kWarpsPerCta * 32), 0, stream, /*pdl=*/true, false, p);
}

}  // namespace oxb
