// Block-scaled fp8 (e4m3) GEMM: 1 x 128 activation scales, 128 x 128 weight scales, fp32
// accumulation with per-K-block promotion, bf16 output.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace oxb {

struct Fp8GemmParams {
  int M, N, K;
  const float* sa_t;  // [ceil(K/128), sa_ld] activation scales, transposed (row index contiguous)
  int sa_ld;
  const float* sw;    // [ceil(N/128), ceil(K/128)] weight scales
  __nv_bfloat16* C;   // [M, N]
  long long ldc;
  const __nv_bfloat16* bias;  // [N] or null
  int* status;
  // Row-parallel use under tensor parallelism (GEMM -> reduce-scatter in one kernel): when n_owners > 0
  // row r belongs to rank r / rows_per_owner and the bf16 partial row is stored into that rank's
  // receive slab [source rank][rows_per_owner][slab_ld] (local or peer memory); the last CTA (ticket)
  // then signals every owner once. Same protocol as the bf16 GEMM's slab epilogue.
  __nv_bfloat16* slab[8];
  uint32_t* arrive[8];
  uint32_t* done_ticket;
  int n_owners, rows_per_owner, my_rank;
  long long slab_ld;
};

// Bounded wait of the activation quantiser on the all-gather flags of its input rows.
struct QuantActWait {
  const uint32_t* flags;  // [n_src] or null: no wait
  uint32_t expected;
  int n_src, rows_per_src;
  uint32_t* ticket;       // re-arms the flags when the last CTA has passed
  int* status;
};

void launch_gemm_fp8_block(const CUtensorMap& tmA, const CUtensorMap& tmB, const Fp8GemmParams& p,
                           cudaStream_t stream);

// x [M, K] bf16 -> q [M, K] e4m3 and sa_t [ceil(K/128), sa_ld] (scale = amax / 448 per 1 x 128 block).
void launch_quant_act_fp8(const __nv_bfloat16* x, long long x_ld, uint8_t* q, long long q_ld,
                          float* sa_t, int sa_ld, int M, int K, const QuantActWait& wait,
                          cudaStream_t stream);

}  // namespace oxb
