// Small-batch bf16 GEMV (M <= 8 rows): the weight-streaming counterpart of the tcgen05 GEMM for
// single-GPU latency-mode decoding, where a 128-row MMA tile would be almost empty.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace oxb {

struct GemvParams {
  const __nv_bfloat16* w;   // [N, K] row-major, or tile-major [N/128][K/64][128][64] when tiled != 0
  const __nv_bfloat16* x;   // [M, K], row stride ldx
  long long ldx;
  const __nv_bfloat16* bias;  // [N] or null
  float* out_f32;             // one of the two outputs, row stride ldo
  __nv_bfloat16* out_bf16;
  long long ldo;
  int M, N, K;
  int tiled;
  int swiglu;  // 1: rows are gate|up interleaved in units of 32; output [M, N/2] = act(gate) * up
  int act;     // 0 = SiLU, 1 = tanh-GELU
};

void launch_gemv_bf16(const GemvParams& p, cudaStream_t stream);

}  // namespace oxb
