// Activation quantiser of the block-scaled fp4 (NVFP4) GEMM, sm_100a.
//
// One CTA per row: row amax -> second-level scale g = amax / (448 * 6) (fp32, kept per row and
// multiplied back in the GEMM epilogue); every 16 values get a ue4m3 scale s = block amax / (6 g),
// rounded up to the next representable value so that no quantised value saturates; the values
// become e2m1 (round to nearest even, saturating), two per byte with the even element in the low
// nibble. Scales are written in the 512-byte atom layout that tcgen05.cp moves to tensor memory:
// [row tile of 128][K / 64][(row % 32) * 16 + (row / 32 % 4) * 4 + (k / 16 % 4)].
//
// Format parity: BlockNvFp4_16 (oxide-quant/src/nvfp4.rs:27-129: e4m3 micro-scale = absmax / 6,
// E2M1 table {0, .5, 1, 1.5, 2, 3, 4, 6}, optional global scale); the reference computes with these
// blocks on the CPU only.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/sm100.cuh"
#include "gemm_bf16.cuh"
#include "gemm_fp8_block.cuh"

namespace oxb {

namespace {

__device__ __forceinline__ uint32_t e2m1_code(float v) {
  // nearest of {0, .5, 1, 1.5, 2, 3, 4, 6}, ties to the even code, saturating
  const float a = fabsf(v);
  uint32_t c;
  if (a <= 0.25f) c = 0;
  else if (a < 0.75f) c = 1;
  else if (a <= 1.25f) c = 2;
  else if (a < 1.75f) c = 3;
  else if (a <= 2.5f) c = 4;
  else if (a < 3.5f) c = 5;
  else if (a <= 5.0f) c = 6;
  else c = 7;
  return c | (v < 0.f ? 8u : 0u);
}

__global__ void __launch_bounds__(128) quant_act_nvfp4_kernel(const __nv_bfloat16* x, long long x_ld, uint8_t* q,
                                                              uint8_t* sf, float* gscale, int rows_per_group,
                                                              int K, const uint32_t* group_counts,
                                                              const QuantActWait w, uint32_t spin_limit) {
  __shared__ float s_red[4];
  const int group = blockIdx.y;
  const int row = blockIdx.x;
  if (w.flags != nullptr) {
    // The rows were written by peers (MoE dispatch) and the per-group counts are final only once
    // every source has signalled: wait, bounded; the last CTA through the gate re-arms the flags.
    __shared__ int s_ok;
    if (threadIdx.x == 0) {
      int ok = 1;
      const uint32_t limit = spin_budget(spin_limit);
      for (int s = 0; s < w.n_src && ok; ++s) {
        uint32_t it = 0, v;
        do {
          asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(w.flags + s) : "memory");
          if (v >= w.expected) break;
        } while (++it <= limit);
        if (v < w.expected) {
          set_status_peer_timeout(w.status);
          ok = 0;
        }
      }
      const uint32_t old = atomicAdd(w.ticket, 1u);
      if (old == gridDim.x * gridDim.y - 1) {
        for (int s = 0; s < w.n_src; ++s) const_cast<uint32_t*>(w.flags)[s] = 0;
        __threadfence();
        *w.ticket = 0;
      }
      s_ok = ok;
    }
    __syncthreads();
    if (!s_ok) return;
  }
  if (group_counts != nullptr && row >= static_cast<int>(__ldcg(group_counts + group))) return;
  const long long grow = static_cast<long long>(group) * rows_per_group + row;
  const __nv_bfloat16* xr = x + grow * x_ld;
  const int n_blk = K / 16;
  // pass 1: row amax
  float amax = 0.f;
  for (int b = threadIdx.x; b < n_blk; b += blockDim.x) {
    const uint4 v0 = __ldcg(reinterpret_cast<const uint4*>(xr + b * 16));   // L2: peers may have written it
    const uint4 v1 = __ldcg(reinterpret_cast<const uint4*>(xr + b * 16 + 8));
    const __nv_bfloat16* e0 = reinterpret_cast<const __nv_bfloat16*>(&v0);
    const __nv_bfloat16* e1 = reinterpret_cast<const __nv_bfloat16*>(&v1);
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fmaxf(fabsf(__bfloat162float(e0[j])), fabsf(__bfloat162float(e1[j]))));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = fmaxf(fmaxf(s_red[0], s_red[1]), fmaxf(s_red[2], s_red[3]));
  const float g = amax > 0.f ? amax / (448.f * 6.f) : 1.f;
  if (threadIdx.x == 0) gscale[grow] = g;
  // pass 2: blocks of 16
  const long long tile = grow >> 7;
  const int r128 = static_cast<int>(grow & 127);
  uint8_t* sf_row = sf + tile * static_cast<long long>(K / 64) * 512 + (r128 & 31) * 16 + (r128 >> 5) * 4;
  uint8_t* qr = q + grow * (K / 2);
  for (int b = threadIdx.x; b < n_blk; b += blockDim.x) {
    const uint4 v0 = __ldcg(reinterpret_cast<const uint4*>(xr + b * 16));
    const uint4 v1 = __ldcg(reinterpret_cast<const uint4*>(xr + b * 16 + 8));
    float v[16];
    const __nv_bfloat16* e0 = reinterpret_cast<const __nv_bfloat16*>(&v0);
    const __nv_bfloat16* e1 = reinterpret_cast<const __nv_bfloat16*>(&v1);
    float bmax = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      v[j] = __bfloat162float(e0[j]);
      v[8 + j] = __bfloat162float(e1[j]);
      bmax = fmaxf(bmax, fmaxf(fabsf(v[j]), fabsf(v[8 + j])));
    }
    // ue4m3 scale, rounded up (a scale rounded down would push the block maximum above 6)
    const float want = bmax / (6.f * g);
    uint8_t sb = static_cast<uint8_t>(__nv_cvt_float_to_fp8(want, __NV_SATFINITE, __NV_E4M3));
    float sd = __half2float(__half(__nv_cvt_fp8_to_halfraw(sb, __NV_E4M3)));
    if (sd < want && sb < 0x7E) {
      ++sb;
      sd = __half2float(__half(__nv_cvt_fp8_to_halfraw(sb, __NV_E4M3)));
    }
    const float inv = sd > 0.f ? 1.f / (sd * g) : 0.f;
    uint32_t w0 = 0, w1 = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      w0 |= e2m1_code(v[j] * inv) << (4 * j);
      w1 |= e2m1_code(v[8 + j] * inv) << (4 * j);
    }
    *reinterpret_cast<uint2*>(qr + b * 8) = make_uint2(w0, w1);
    sf_row[(b >> 2) * 512 + (b & 3)] = sb;
  }
}

}  // namespace

void launch_quant_act_nvfp4(const __nv_bfloat16* x, long long x_ld, uint8_t* q, uint8_t* sf, float* gscale,
                            int groups, int rows_per_group, int K, const uint32_t* group_counts,
                            const QuantActWait& wait, uint32_t spin_limit, cudaStream_t stream) {
  if (groups <= 0 || rows_per_group <= 0) return;
  quant_act_nvfp4_kernel<<<dim3(rows_per_group, groups), 128, 0, stream>>>(x, x_ld, q, sf, gscale, rows_per_group, K,
                                                                         group_counts, wait, spin_limit);
}

}  // namespace oxb
