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
  // Mixed-type stack (launch_mmvq_mixed): output rows [row_begin of segment i, row_end) come from
  // segment i, whose rows are seg_row_bytes apart and packed as seg_type. n_seg == 0: `w` alone.
  int n_seg;
  const uint8_t* seg_w[4];
  long long seg_row_bytes[4];
  int seg_type[4];
  int seg_row_end[4];
};

// x [M, K] bf16 -> int8 blocks of 32 with an fp32 scale (amax / 127) and the block sum.
void launch_quant_q8_1(const __nv_bfloat16* x, long long ldx, int8_t* xq, float* xd, float* xs, int M,
                       int K, cudaStream_t stream);

// Return false when the type has no device decoder.
bool launch_mmvq(int qtype, const MmvqParams& p, cudaStream_t stream);
// One launch over up to four stacked weight matrices of different block types that share K (the
// Q | K | V or gate | up projections of a mixed-precision GGUF file). Needs the int8 activations
// (xq / xd / xs). Returns false when a segment's type has no integer path or an operand is misaligned.
bool launch_mmvq_mixed(const MmvqParams& p, cudaStream_t stream);
bool mmvq_has_int8_path(int qtype);
bool launch_dequant_rows(int qtype, const uint8_t* w, long long row_bytes, const int* row_ids,
                         int n_rows, int K, __nv_bfloat16* out, long long ldo, float scale,
                         int n_src_rows, cudaStream_t stream);
long long quant_row_bytes(int qtype, long long K);

}  // namespace oxb
