#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace oxb {

struct MmvqParams {
  const uint8_t* w;        // [N rows] of packed blocks, row_bytes apart
  long long row_bytes;
  const __nv_bfloat16* x;  // [M, K], row stride ldx
  long long ldx;
  const __nv_bfloat16* bias;  // [N] nullable
  float* out_f32;             // one of the two outputs, row stride ldo
  __nv_bfloat16* out_bf16;
  long long ldo;
  int M, N, K;
  int add;  // 1: out += result (fused residual)
  // Optional int8 view of x (Q8_1-style, from launch_quant_q8_1): when set, Q4_K and Q8_0 weights take
  // the integer dot-product path (dp4a) instead of expanding weights to fp32.
  const int8_t* xq;   // [M, K], row stride K
  const float* xd;    // [M, K / 32] block scales
  const float* xs;    // [M, K / 32] block sums (scale * sum of the int8 values)
};

// x [M, K] bf16 -> int8 blocks of 32 with an fp32 scale (amax / 127) and the block sum.
void launch_quant_q8_1(const __nv_bfloat16* x, long long ldx, int8_t* xq, float* xd, float* xs, int M,
                       int K, cudaStream_t stream);

// Return false when the type has no device decoder.
bool launch_mmvq(int qtype, const MmvqParams& p, cudaStream_t stream);
bool launch_dequant_rows(int qtype, const uint8_t* w, long long row_bytes, const int* row_ids,
                         int n_rows, int K, __nv_bfloat16* out, long long ldo, float scale,
                         int n_src_rows, cudaStream_t stream);
long long quant_row_bytes(int qtype, long long K);

}  // namespace oxb
