// Quantized-weight kernels for every GGUF block type (sm_100a):
//   mmvq        : y[m, n] = sum_k W_q[n, k] x[m, k] for small batches (m <= 8 per pass). One warp
//                 per weight row; each lane expands 32-weight groups in registers and multiplies
//                 them with every activation row, so the packed weights are read from HBM once.
//                 Optional bias and fused residual add.
//   dequant_rows: expands selected rows (or all rows) of a quantized matrix to bf16; feeds the
//                 tcgen05 GEMM for larger batches and the embedding gather.
// Reference counterparts: gemv_q4_0/q5_0/q4_1/q5_1/iq4_nl/tq2_0 (quant_gemv_standard.cu:3-369),
// gemv_q2_k/q3_k/q5_k (quant_gemv_kquants.cu:1189-1376), mmvq_* (quant_gemv_standard.cu:423-859),
// dequantize_*_to_f16 (cublas_ops.cu:18-217), dequantize_token_embd_* (megakernel_ops.cu:2-116).
#include "quant_ops.cuh"

#include "../common/sm100.cuh"
#include "quant_blocks.cuh"

namespace oxb {

namespace {

constexpr int kRowsPerCta = 8;  // one warp per weight row

template <int T, int MB>
__global__ void __launch_bounds__(kRowsPerCta * 32) mmvq_kernel(const MmvqParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * kRowsPerCta + warp;
  if (n >= p.N) return;
  const int m0 = blockIdx.y * MB;
  const uint8_t* wrow = p.w + static_cast<long long>(n) * p.row_bytes;
  const int groups = p.K >> 5;

  float acc[MB];
#pragma unroll
  for (int m = 0; m < MB; ++m) acc[m] = 0.f;

  for (int grp = lane; grp < groups; grp += 32) {
    float w[32];
    dequant32<T>(wrow, grp, w);
#pragma unroll
    for (int m = 0; m < MB; ++m) {
      if (m0 + m < p.M) {
        const uint4* xp =
            reinterpret_cast<const uint4*>(p.x + static_cast<long long>(m0 + m) * p.ldx + grp * 32);
        float s = 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint4 v = __ldg(xp + c);
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(h[j]);
            s += w[c * 8 + 2 * j] * f.x + w[c * 8 + 2 * j + 1] * f.y;
          }
        }
        acc[m] += s;
      }
    }
  }
#pragma unroll
  for (int m = 0; m < MB; ++m) {
    const float v = warp_sum(acc[m]);
    if (lane == 0 && m0 + m < p.M) {
      float r = v;
      if (p.bias != nullptr) r += __bfloat162float(p.bias[n]);
      const long long o = static_cast<long long>(m0 + m) * p.ldo + n;
      if (p.out_f32 != nullptr) {
        p.out_f32[o] = p.add ? p.out_f32[o] + r : r;
      } else {
        if (p.add) r += __bfloat162float(p.out_bf16[o]);
        p.out_bf16[o] = __float2bfloat16(r);
      }
    }
  }
}

template <int T>
__global__ void __launch_bounds__(256) dequant_rows_kernel(const uint8_t* w, long long row_bytes,
                                                           const int* row_ids, int K,
                                                           __nv_bfloat16* out, long long ldo,
                                                           float scale, int n_src_rows) {
  const int r = blockIdx.x;
  int src = row_ids != nullptr ? row_ids[r] : r;
  if (src < 0 || src >= n_src_rows) src = 0;
  const uint8_t* wrow = w + static_cast<long long>(src) * row_bytes;
  __nv_bfloat16* o = out + static_cast<long long>(r) * ldo;
  for (int grp = blockIdx.y * blockDim.x + threadIdx.x; grp < (K >> 5);
       grp += gridDim.y * blockDim.x) {
    float v[32];
    dequant32<T>(wrow, grp, v);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint4 q;
      q.x = pack_bf16x2(v[c * 8 + 0] * scale, v[c * 8 + 1] * scale);
      q.y = pack_bf16x2(v[c * 8 + 2] * scale, v[c * 8 + 3] * scale);
      q.z = pack_bf16x2(v[c * 8 + 4] * scale, v[c * 8 + 5] * scale);
      q.w = pack_bf16x2(v[c * 8 + 6] * scale, v[c * 8 + 7] * scale);
      *reinterpret_cast<uint4*>(o + grp * 32 + c * 8) = q;
    }
  }
}

template <int T>
void mmvq_dispatch(const MmvqParams& p, cudaStream_t s) {
  const int gx = (p.N + kRowsPerCta - 1) / kRowsPerCta;
  if (p.M == 1) {
    mmvq_kernel<T, 1><<<dim3(gx, 1), kRowsPerCta * 32, 0, s>>>(p);
  } else if (p.M == 2) {
    mmvq_kernel<T, 2><<<dim3(gx, 1), kRowsPerCta * 32, 0, s>>>(p);
  } else if (p.M <= 4) {
    mmvq_kernel<T, 4><<<dim3(gx, 1), kRowsPerCta * 32, 0, s>>>(p);
  } else {
    mmvq_kernel<T, 8><<<dim3(gx, (p.M + 7) / 8), kRowsPerCta * 32, 0, s>>>(p);
  }
}

template <int T>
void dequant_dispatch(const uint8_t* w, long long row_bytes, const int* row_ids, int n_rows, int K,
                      __nv_bfloat16* out, long long ldo, float scale, int n_src_rows,
                      cudaStream_t s) {
  int gy = ((K >> 5) + 255) / 256;
  if (gy < 1) gy = 1;
  dequant_rows_kernel<T><<<dim3(n_rows, gy), 256, 0, s>>>(w, row_bytes, row_ids, K, out, ldo, scale,
                                                          n_src_rows);
}

}  // namespace

#define OXB_QDISPATCH(type, CALL)                                   \
  switch (type) {                                                   \
    case kQ_Q4_0: CALL(kQ_Q4_0); break;                             \
    case kQ_Q4_1: CALL(kQ_Q4_1); break;                             \
    case kQ_Q5_0: CALL(kQ_Q5_0); break;                             \
    case kQ_Q5_1: CALL(kQ_Q5_1); break;                             \
    case kQ_Q8_0: CALL(kQ_Q8_0); break;                             \
    case kQ_Q2_K: CALL(kQ_Q2_K); break;                             \
    case kQ_Q3_K: CALL(kQ_Q3_K); break;                             \
    case kQ_Q4_K: CALL(kQ_Q4_K); break;                             \
    case kQ_Q5_K: CALL(kQ_Q5_K); break;                             \
    case kQ_Q6_K: CALL(kQ_Q6_K); break;                             \
    case kQ_IQ4_NL: CALL(kQ_IQ4_NL); break;                         \
    case kQ_TQ2_0: CALL(kQ_TQ2_0); break;                           \
    case kQ_NVFP4: CALL(kQ_NVFP4); break;                           \
    default: return false;                                          \
  }

bool launch_mmvq(int qtype, const MmvqParams& p, cudaStream_t stream) {
  if (p.M <= 0 || p.N <= 0) return true;
#define CALL(T) mmvq_dispatch<T>(p, stream)
  OXB_QDISPATCH(qtype, CALL)
#undef CALL
  return true;
}

bool launch_dequant_rows(int qtype, const uint8_t* w, long long row_bytes, const int* row_ids,
                         int n_rows, int K, __nv_bfloat16* out, long long ldo, float scale,
                         int n_src_rows, cudaStream_t stream) {
  if (n_rows <= 0) return true;
#define CALL(T) dequant_dispatch<T>(w, row_bytes, row_ids, n_rows, K, out, ldo, scale, n_src_rows, stream)
  OXB_QDISPATCH(qtype, CALL)
#undef CALL
  return true;
}

long long quant_row_bytes(int qtype, long long K) {
  switch (qtype) {
    case kQ_F32: return K * 4;
    case kQ_F16: case kQ_BF16: return K * 2;
    case kQ_Q4_0: case kQ_IQ4_NL: return K / 32 * 18;
    case kQ_Q4_1: return K / 32 * 20;
    case kQ_Q5_0: return K / 32 * 22;
    case kQ_Q5_1: return K / 32 * 24;
    case kQ_Q8_0: return K / 32 * 34;
    case kQ_Q2_K: return K / 256 * 84;
    case kQ_Q3_K: return K / 256 * 110;
    case kQ_Q4_K: return K / 256 * 144;
    case kQ_Q5_K: return K / 256 * 176;
    case kQ_Q6_K: return K / 256 * 210;
    case kQ_TQ2_0: return K / 256 * 66;
    case kQ_NVFP4: return K / 16 * 16;
    default: return -1;
  }
}

}  // namespace oxb
