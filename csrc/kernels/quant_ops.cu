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

#include "../common/device_info.h"
#include "../common/sm100.cuh"
#include "quant_blocks.cuh"
#include "quant_expand.cuh"

namespace oxb {

namespace {

constexpr int kRowsPerCta = 8;  // one warp per weight row

template <int T, int MB>
__global__ void __launch_bounds__(kRowsPerCta * 32) mmvq_kernel(const MmvqParams p) {
  pdl_wait();  // the activation rows come from the kernel before this one
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
  pdl_launch_dependents();  // the weight stream is done: the next kernel may become resident
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

// ---- vectorised fast paths for the two block types of a usual Q4_K checkpoint -------------------
// The generic kernel above expands a block byte by byte (it exists for every GGUF type); these two
// read a block with 16-byte / 2-byte vector loads and never materialise the weights: a block's
// contribution is  d * sc * sum(q * x) - dmin * mn * sum(x).

__device__ __forceinline__ void mmvq_store(const MmvqParams& p, int n, int m, float v) {
  float r = v;
  if (p.bias != nullptr) r += __bfloat162float(p.bias[n]);
  const long long o = static_cast<long long>(m) * p.ldo + n;
  if (p.out_f32 != nullptr) {
    p.out_f32[o] = p.add ? p.out_f32[o] + r : r;
  } else {
    if (p.add) r += __bfloat162float(p.out_bf16[o]);
    p.out_bf16[o] = __float2bfloat16(r);
  }
}

__device__ __forceinline__ float nib_to_float(uint32_t bytes, uint32_t sel) {
  // byte `sel & 3` of `bytes` (a value 0..15) placed in the mantissa of 2^23, minus 2^23: exact, and
  // two full-rate instructions instead of a quarter-rate integer-to-float conversion
  return __uint_as_float(__byte_perm(bytes, 0x4B000000u, sel)) - 8388608.f;
}

// One warp per weight row, one Q4_K super-block (256 weights, 128 bytes of nibbles) per iteration.
// Lane l owns 32-bit word l of those bytes: 4 low-nibble weights of sub-block 2j and 4 high-nibble
// weights of sub-block 2j+1 (j = l / 8). The weight load is one coalesced 128-byte access per warp
// and the activation loads are 8-byte accesses that are contiguous across lanes (a lane-strided
// mapping costs one L1 wavefront per lane and made this kernel L1-bound at 1.5 T weights/s).
template <int MB>
__global__ void __launch_bounds__(kRowsPerCta * 32) mmvq_q4k_kernel(const MmvqParams p) {
  pdl_wait();  // the activation rows come from the kernel before this one
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * kRowsPerCta + warp;
  if (n >= p.N) return;
  const int m0 = blockIdx.y * MB;
  const uint8_t* wrow = p.w + static_cast<long long>(n) * p.row_bytes;
  const int n_sb = p.K >> 8;
  const int j = lane >> 3, cw = lane & 7;
  float acc[MB];
#pragma unroll
  for (int m = 0; m < MB; ++m) acc[m] = 0.f;

#pragma unroll 4
  for (int sb = 0; sb < n_sb; ++sb) {
    const uint8_t* b = wrow + static_cast<long long>(sb) * 144;
    const uint32_t qw = __ldg(reinterpret_cast<const uint32_t*>(b + 16) + lane);
    const uint32_t dm = __ldg(reinterpret_cast<const uint32_t*>(b));
    const uint32_t s0 = __ldg(reinterpret_cast<const uint32_t*>(b + 4));
    const uint32_t s1 = __ldg(reinterpret_cast<const uint32_t*>(b + 8));
    const uint32_t s2 = __ldg(reinterpret_cast<const uint32_t*>(b + 12));
    const float d = __half2float(__ushort_as_half(static_cast<uint16_t>(dm & 0xFFFFu)));
    const float dmin = __half2float(__ushort_as_half(static_cast<uint16_t>(dm >> 16)));
    int sc[2], mn[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int sub = 2 * j + h;
      if (sub < 4) {
        sc[h] = byte_of3(s0, s1, s2, sub) & 63;
        mn[h] = byte_of3(s0, s1, s2, sub + 4) & 63;
      } else {
        sc[h] = (byte_of3(s0, s1, s2, sub + 4) & 0xF) | ((byte_of3(s0, s1, s2, sub - 4) >> 6) << 4);
        mn[h] = (byte_of3(s0, s1, s2, sub + 4) >> 4) | ((byte_of3(s0, s1, s2, sub) >> 6) << 4);
      }
    }
    const uint32_t lo = qw & 0x0F0F0F0Fu, hi = (qw >> 4) & 0x0F0F0F0Fu;
    const float l0 = nib_to_float(lo, 0x7650), l1 = nib_to_float(lo, 0x7651), l2 = nib_to_float(lo, 0x7652),
                l3 = nib_to_float(lo, 0x7653);
    const float h0 = nib_to_float(hi, 0x7650), h1 = nib_to_float(hi, 0x7651), h2 = nib_to_float(hi, 0x7652),
                h3 = nib_to_float(hi, 0x7653);
    const float dl0 = d * sc[0], dl1 = d * sc[1], ml0 = dmin * mn[0], ml1 = dmin * mn[1];
    const int e0 = sb * 256 + j * 64 + cw * 4;
#pragma unroll
    for (int m = 0; m < MB; ++m) {
      if (m0 + m >= p.M) continue;
      const __nv_bfloat16* xr = p.x + static_cast<long long>(m0 + m) * p.ldx + e0;
      const uint2 xl = __ldg(reinterpret_cast<const uint2*>(xr));
      const uint2 xh = __ldg(reinterpret_cast<const uint2*>(xr + 32));
      const float2 a0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xl.x));
      const float2 a1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xl.y));
      const float2 b0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xh.x));
      const float2 b1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xh.y));
      const float ql = l0 * a0.x + l1 * a0.y + l2 * a1.x + l3 * a1.y;
      const float qh = h0 * b0.x + h1 * b0.y + h2 * b1.x + h3 * b1.y;
      const float sl = (a0.x + a0.y) + (a1.x + a1.y), sh = (b0.x + b0.y) + (b1.x + b1.y);
      acc[m] += dl0 * ql - ml0 * sl + dl1 * qh - ml1 * sh;
    }
  }
  pdl_launch_dependents();  // the weight stream is done: the next kernel may become resident
#pragma unroll
  for (int m = 0; m < MB; ++m) {
    const float v = warp_sum(acc[m]);
    if (lane == 0 && m0 + m < p.M) mmvq_store(p, n, m0 + m, v);
  }
}

// ---- integer dot-product path (activations pre-quantised to int8 blocks of 32) -------------------
// The fp32 kernels above spend 6-9 instructions per weight and top out near 0.8 TB/s; the HBM
// roofline leaves about 3. With int8 activations a lane multiplies 4 weights per `dp4a`.
__device__ __forceinline__ float int_to_float(int v) {  // |v| < 2^22, two full-rate instructions
  return __int_as_float(0x4B400000 + v) - 12582912.f;
}

__global__ void quant_q8_1_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, int8_t* __restrict__ xq,
                                  float* __restrict__ xd, float* __restrict__ xs, int M, int K) {
  pdl_launch_dependents();
  pdl_wait();  // the activation rows come from the kernel before this one
  const int n_blk = K >> 5;
  const long long wid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= static_cast<long long>(M) * n_blk) return;
  const int row = static_cast<int>(wid / n_blk), blk = static_cast<int>(wid % n_blk);
  const float v = __bfloat162float(x[static_cast<long long>(row) * ldx + blk * 32 + lane]);
  const float amax = warp_max(fabsf(v));
  const float d = amax / 127.f;
  const float inv = amax > 0.f ? 127.f / amax : 0.f;
  const int q = __float2int_rn(v * inv);
  xq[static_cast<long long>(row) * K + blk * 32 + lane] = static_cast<int8_t>(q);
  const float sum = warp_sum(static_cast<float>(q));
  if (lane == 0) {
    xd[static_cast<long long>(row) * n_blk + blk] = d;
    xs[static_cast<long long>(row) * n_blk + blk] = d * sum;
  }
}

// Q4_K x int8: one warp per weight row, four super-blocks per iteration. Lane l: super-block l / 8
// of the four, 16-byte chunk r = l % 8 of its 128 nibble bytes = 16 low-nibble weights of sub-block
// 2j and 16 high-nibble weights of sub-block 2j+1 (j = r / 2). The loop is unrolled so that a warp
// keeps 2 KB of weights in flight; all loads are contiguous across lanes.
// R weight rows per warp: their loads are issued together (more bytes in flight per warp, the
// activation loads are shared).
template <int MB, int R>
__global__ void __launch_bounds__(kRowsPerCta * 32) mmvq_q4k_dp4a_kernel(const MmvqParams p) {
  pdl_wait();  // the activation rows come from the kernel before this one
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_base = (blockIdx.x * kRowsPerCta + warp) * R;
  if (n_base >= p.N) return;
  const int m0 = blockIdx.y * MB;
  const int n_sb = p.K >> 8, n_blk = p.K >> 5;
  const int r = lane & 7, j = r >> 1, c2 = r & 1;
  float acc[R][MB];
#pragma unroll
  for (int t = 0; t < R; ++t)
#pragma unroll
    for (int m = 0; m < MB; ++m) acc[t][m] = 0.f;

#pragma unroll 4
  for (int sb = lane >> 3; sb < n_sb; sb += 4) {
    uint4 q[R];
    uint32_t dm[R], s0[R], s1[R], s2[R];
#pragma unroll
    for (int t = 0; t < R; ++t) {
      const int n = n_base + t < p.N ? n_base + t : p.N - 1;  // a clamped duplicate row is not stored
      const uint8_t* b = p.w + static_cast<long long>(n) * p.row_bytes + static_cast<long long>(sb) * 144;
      q[t] = __ldg(reinterpret_cast<const uint4*>(b + 16) + r);
      const uint4 hdr = __ldg(reinterpret_cast<const uint4*>(b));  // d | dmin | 12 scale bytes
      dm[t] = hdr.x;
      s0[t] = hdr.y;
      s1[t] = hdr.z;
      s2[t] = hdr.w;
    }
    const int e0 = sb * 256 + j * 64 + c2 * 16;
    const int blk = sb * 8 + 2 * j;
    int4 xl[MB], xh[MB];
    float2 dd[MB], ss[MB];
#pragma unroll
    for (int m = 0; m < MB; ++m) {
      const int mm = m0 + m < p.M ? m0 + m : p.M - 1;
      const int8_t* xr = p.xq + static_cast<long long>(mm) * p.K + e0;
      xl[m] = __ldg(reinterpret_cast<const int4*>(xr));
      xh[m] = __ldg(reinterpret_cast<const int4*>(xr + 32));
      dd[m] = __ldg(reinterpret_cast<const float2*>(p.xd + static_cast<long long>(mm) * n_blk + blk));
      ss[m] = __ldg(reinterpret_cast<const float2*>(p.xs + static_cast<long long>(mm) * n_blk + blk));
    }
#pragma unroll
    for (int t = 0; t < R; ++t) {
      const float d = __half2float(__ushort_as_half(static_cast<uint16_t>(dm[t] & 0xFFFFu)));
      const float dmin = __half2float(__ushort_as_half(static_cast<uint16_t>(dm[t] >> 16)));
      int sc[2], mn[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int sub = 2 * j + h;
        if (sub < 4) {
          sc[h] = byte_of3(s0[t], s1[t], s2[t], sub) & 63;
          mn[h] = byte_of3(s0[t], s1[t], s2[t], sub + 4) & 63;
        } else {
          sc[h] = (byte_of3(s0[t], s1[t], s2[t], sub + 4) & 0xF) | ((byte_of3(s0[t], s1[t], s2[t], sub - 4) >> 6) << 4);
          mn[h] = (byte_of3(s0[t], s1[t], s2[t], sub + 4) >> 4) | ((byte_of3(s0[t], s1[t], s2[t], sub) >> 6) << 4);
        }
      }
      const uint32_t qw[4] = {q[t].x, q[t].y, q[t].z, q[t].w};
      const float dl0 = d * sc[0], dl1 = d * sc[1];
      // the `- dmin * mn * sum(x)` term of a sub-block is added once, by the lane that owns its first half
      const float ml0 = c2 == 0 ? dmin * mn[0] : 0.f, ml1 = c2 == 0 ? dmin * mn[1] : 0.f;
#pragma unroll
      for (int m = 0; m < MB; ++m) {
        const int xlw[4] = {xl[m].x, xl[m].y, xl[m].z, xl[m].w}, xhw[4] = {xh[m].x, xh[m].y, xh[m].z, xh[m].w};
        int il = 0, ih = 0;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          il = __dp4a(static_cast<int>(qw[u] & 0x0F0F0F0Fu), xlw[u], il);
          ih = __dp4a(static_cast<int>((qw[u] >> 4) & 0x0F0F0F0Fu), xhw[u], ih);
        }
        acc[t][m] += dl0 * dd[m].x * int_to_float(il) + dl1 * dd[m].y * int_to_float(ih) - ml0 * ss[m].x -
                     ml1 * ss[m].y;
      }
    }
  }
  pdl_launch_dependents();  // the weight stream is done: the next kernel may become resident
#pragma unroll
  for (int t = 0; t < R; ++t)
#pragma unroll
    for (int m = 0; m < MB; ++m) {
      const float v = warp_sum(acc[t][m]);
      if (lane == 0 && m0 + m < p.M && n_base + t < p.N) mmvq_store(p, n_base + t, m0 + m, v);
    }
}

// Q8_0 x int8: a lane takes one 34-byte block (2-byte aligned: 16-bit loads, repacked into words).
template <int MB>
__global__ void __launch_bounds__(kRowsPerCta * 32) mmvq_q8_0_dp4a_kernel(const MmvqParams p) {
  pdl_wait();  // the activation rows come from the kernel before this one
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * kRowsPerCta + warp;
  if (n >= p.N) return;
  const int m0 = blockIdx.y * MB;
  const uint8_t* wrow = p.w + static_cast<long long>(n) * p.row_bytes;
  const int groups = p.K >> 5;
  float acc[MB];
#pragma unroll
  for (int m = 0; m < MB; ++m) acc[m] = 0.f;
#pragma unroll 2
  for (int grp = lane; grp < groups; grp += 32) {
    const uint16_t* b = reinterpret_cast<const uint16_t*>(wrow + static_cast<long long>(grp) * 34);
    const float d = __half2float(__ushort_as_half(__ldg(b)));
    int w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
      w[i] = static_cast<int>(static_cast<uint32_t>(__ldg(b + 1 + 2 * i)) |
                              (static_cast<uint32_t>(__ldg(b + 2 + 2 * i)) << 16));
#pragma unroll
    for (int m = 0; m < MB; ++m) {
      if (m0 + m >= p.M) continue;
      const int4* xr = reinterpret_cast<const int4*>(p.xq + static_cast<long long>(m0 + m) * p.K + grp * 32);
      const int4 a = __ldg(xr), c = __ldg(xr + 1);
      int s = __dp4a(w[0], a.x, 0);
      s = __dp4a(w[1], a.y, s);
      s = __dp4a(w[2], a.z, s);
      s = __dp4a(w[3], a.w, s);
      s = __dp4a(w[4], c.x, s);
      s = __dp4a(w[5], c.y, s);
      s = __dp4a(w[6], c.z, s);
      s = __dp4a(w[7], c.w, s);
      acc[m] += d * __ldg(p.xd + static_cast<long long>(m0 + m) * groups + grp) * int_to_float(s);
    }
  }
  pdl_launch_dependents();  // the weight stream is done: the next kernel may become resident
#pragma unroll
  for (int m = 0; m < MB; ++m) {
    const float v = warp_sum(acc[m]);
    if (lane == 0 && m0 + m < p.M) mmvq_store(p, n, m0 + m, v);
  }
}

// ---- integer path for the other block types ------------------------------------------------------
// A group of 32 weights is rebuilt as eight words of four signed bytes q_j with
//   w_j = dl0 * q_j + ml  (j < 16),   w_j = dl1 * q_j + ml  (j >= 16),
// so a group's share of the dot product is  xd * (dl0 * sum_lo(q x) + dl1 * sum_hi(q x)) + ml * xs
// with eight `dp4a` per activation row. Blocks are read with the widest loads their alignment allows
// (Q4_0 / Q5_0 / Q8_0 / Q6_K blocks are only 2-byte aligned).
// One weight row against MB int8 activation rows; every lane takes the groups lane, lane + 32, ...
template <int T, int MB>
__device__ __forceinline__ void row_dot_int8(const uint8_t* wrow, const MmvqParams& p, int m0, int lane,
                                             float (&acc)[MB]) {
  const int groups = p.K >> 5;
#pragma unroll 2
  for (int grp = lane; grp < groups; grp += 32) {
    uint32_t wq[8];
    float dl0, dl1, ml;
    expand_q8<T>(wrow, grp, wq, dl0, dl1, ml);
#pragma unroll
    for (int m = 0; m < MB; ++m) {
      const int mm = m0 + m < p.M ? m0 + m : p.M - 1;  // a clamped duplicate row is not stored
      const int4* xr = reinterpret_cast<const int4*>(p.xq + static_cast<long long>(mm) * p.K + grp * 32);
      const int4 a = __ldg(xr), c = __ldg(xr + 1);
      int lo = __dp4a(static_cast<int>(wq[0]), a.x, 0);
      lo = __dp4a(static_cast<int>(wq[1]), a.y, lo);
      lo = __dp4a(static_cast<int>(wq[2]), a.z, lo);
      lo = __dp4a(static_cast<int>(wq[3]), a.w, lo);
      int hi = __dp4a(static_cast<int>(wq[4]), c.x, 0);
      hi = __dp4a(static_cast<int>(wq[5]), c.y, hi);
      hi = __dp4a(static_cast<int>(wq[6]), c.z, hi);
      hi = __dp4a(static_cast<int>(wq[7]), c.w, hi);
      const long long bi = static_cast<long long>(mm) * groups + grp;
      acc[m] += __ldg(p.xd + bi) * (dl0 * int_to_float(lo) + dl1 * int_to_float(hi)) + ml * __ldg(p.xs + bi);
    }
  }
}

template <int T, int MB>
__global__ void __launch_bounds__(kRowsPerCta * 32) mmvq_int8_kernel(const MmvqParams p) {
  pdl_wait();  // the activation rows come from the kernel before this one
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * kRowsPerCta + warp;
  if (n >= p.N) return;
  const int m0 = blockIdx.y * MB;
  float acc[MB];
#pragma unroll
  for (int m = 0; m < MB; ++m) acc[m] = 0.f;
  row_dot_int8<T, MB>(p.w + static_cast<long long>(n) * p.row_bytes, p, m0, lane, acc);
  pdl_launch_dependents();  // the weight stream is done: the next kernel may become resident
#pragma unroll
  for (int m = 0; m < MB; ++m) {
    const float v = warp_sum(acc[m]);
    if (lane == 0 && m0 + m < p.M) mmvq_store(p, n, m0 + m, v);
  }
}

// Stacked matrices of different block types (Q|K|V or gate|up of a mixed-precision file) in one
// launch: a warp looks up the segment of its output row; the type switch is uniform per warp.
template <int MB>
__global__ void __launch_bounds__(kRowsPerCta * 32) mmvq_mixed_kernel(const MmvqParams p) {
  pdl_wait();  // the activation rows come from the kernel before this one
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * kRowsPerCta + warp;
  if (n >= p.N) return;
  const int m0 = blockIdx.y * MB;
  int seg = 0, row0 = 0;
#pragma unroll
  for (int i = 0; i < 3; ++i)
    if (seg == i && i + 1 < p.n_seg && n >= p.seg_row_end[i]) {
      row0 = p.seg_row_end[i];
      seg = i + 1;
    }
  const uint8_t* wrow = p.seg_w[seg] + static_cast<long long>(n - row0) * p.seg_row_bytes[seg];
  float acc[MB];
#pragma unroll
  for (int m = 0; m < MB; ++m) acc[m] = 0.f;
  switch (p.seg_type[seg]) {
    case kQ_Q4_0: row_dot_int8<kQ_Q4_0, MB>(wrow, p, m0, lane, acc); break;
    case kQ_Q4_1: row_dot_int8<kQ_Q4_1, MB>(wrow, p, m0, lane, acc); break;
    case kQ_Q5_0: row_dot_int8<kQ_Q5_0, MB>(wrow, p, m0, lane, acc); break;
    case kQ_Q5_1: row_dot_int8<kQ_Q5_1, MB>(wrow, p, m0, lane, acc); break;
    case kQ_Q8_0: row_dot_int8<kQ_Q8_0, MB>(wrow, p, m0, lane, acc); break;
    case kQ_Q4_K: row_dot_int8<kQ_Q4_K, MB>(wrow, p, m0, lane, acc); break;
    case kQ_Q5_K: row_dot_int8<kQ_Q5_K, MB>(wrow, p, m0, lane, acc); break;
    case kQ_Q6_K: row_dot_int8<kQ_Q6_K, MB>(wrow, p, m0, lane, acc); break;
    default: break;
  }
  pdl_launch_dependents();  // the weight stream is done: the next kernel may become resident
#pragma unroll
  for (int m = 0; m < MB; ++m) {
    const float v = warp_sum(acc[m]);
    if (lane == 0 && m0 + m < p.M) mmvq_store(p, n, m0 + m, v);
  }
}

// Q8_0: 34-byte blocks (fp16 scale + 32 int8) are only 2-byte aligned: seventeen 16-bit loads.
template <int MB>
__global__ void __launch_bounds__(kRowsPerCta * 32) mmvq_q8_0_kernel(const MmvqParams p) {
  pdl_wait();  // the activation rows come from the kernel before this one
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * kRowsPerCta + warp;
  if (n >= p.N) return;
  const int m0 = blockIdx.y * MB;
  const uint8_t* wrow = p.w + static_cast<long long>(n) * p.row_bytes;
  const int groups = p.K >> 5;
  float acc[MB];
#pragma unroll
  for (int m = 0; m < MB; ++m) acc[m] = 0.f;

#pragma unroll 2
  for (int grp = lane; grp < groups; grp += 32) {
    const uint16_t* b = reinterpret_cast<const uint16_t*>(wrow + static_cast<long long>(grp) * 34);
    uint16_t q[17];
#pragma unroll
    for (int i = 0; i < 17; ++i) q[i] = __ldg(b + i);
    const float d = __half2float(__ushort_as_half(q[0]));
#pragma unroll
    for (int m = 0; m < MB; ++m) {
      if (m0 + m >= p.M) continue;
      const uint4* xp =
          reinterpret_cast<const uint4*>(p.x + static_cast<long long>(m0 + m) * p.ldx + grp * 32);
      float s = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint4 v = __ldg(xp + c);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const uint16_t w = q[1 + 4 * c + e];
          const float2 f = __bfloat1622float2(h[e]);
          s += static_cast<float>(static_cast<int8_t>(w & 0xFF)) * f.x +
               static_cast<float>(static_cast<int8_t>(w >> 8)) * f.y;
        }
      }
      acc[m] += d * s;
    }
  }
  pdl_launch_dependents();  // the weight stream is done: the next kernel may become resident
#pragma unroll
  for (int m = 0; m < MB; ++m) {
    const float v = warp_sum(acc[m]);
    if (lane == 0 && m0 + m < p.M) mmvq_store(p, n, m0 + m, v);
  }
}

#define OXB_MMVQ_FAST(KERNEL)                                                                  \
  do {                                                                                         \
    const int gx = (p.N + kRowsPerCta - 1) / kRowsPerCta;                                      \
    if (p.M == 1) launch_kernel(KERNEL<1>, dim3(gx, 1), dim3(kRowsPerCta * 32), 0, s, /*pdl=*/true, false, p);                       \
    else if (p.M == 2) launch_kernel(KERNEL<2>, dim3(gx, 1), dim3(kRowsPerCta * 32), 0, s, /*pdl=*/true, false, p);                  \
    else if (p.M <= 4) launch_kernel(KERNEL<4>, dim3(gx, 1), dim3(kRowsPerCta * 32), 0, s, /*pdl=*/true, false, p);                  \
    else launch_kernel(KERNEL<8>, dim3(gx, (p.M + 7) / 8), dim3(kRowsPerCta * 32), 0, s, /*pdl=*/true, false, p);                    \
  } while (0)

// Alignment that expand_q8 of a type needs: 16 bytes for the K-quants read with uint4 loads, 4 for
// Q4_1 / Q5_1, 2 for the rest; the int8 activations are read with 16-byte loads.
bool int8_operands_ok(int type, const uint8_t* w, long long row_bytes, const MmvqParams& p) {
  const uintptr_t need = (type == kQ_Q4_K || type == kQ_Q5_K) ? 16 : ((type == kQ_Q4_1 || type == kQ_Q5_1) ? 4 : 2);
  const int qk = (type == kQ_Q4_K || type == kQ_Q5_K || type == kQ_Q6_K) ? 256 : 32;
  return (reinterpret_cast<uintptr_t>(w) % need) == 0 && (row_bytes % static_cast<long long>(need)) == 0 &&
         (p.K % qk) == 0 && (reinterpret_cast<uintptr_t>(p.xq) & 15) == 0 && p.xd != nullptr && p.xs != nullptr;
}

template <int T>
void mmvq_dispatch(const MmvqParams& p, cudaStream_t s) {
  // vector-load fast paths need 16-byte aligned rows (weights and activations)
  const bool aligned = (reinterpret_cast<uintptr_t>(p.w) & 15) == 0 && (p.row_bytes & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(p.x) & 15) == 0 && (p.ldx & 7) == 0;
  if constexpr (T == kQ_Q4_K) {
    if (p.xq != nullptr && aligned && (p.K & 255) == 0 && (reinterpret_cast<uintptr_t>(p.xq) & 15) == 0) {
      if (p.M == 1) {
        const int gx = (p.N + 2 * kRowsPerCta - 1) / (2 * kRowsPerCta);
        launch_kernel(mmvq_q4k_dp4a_kernel<1, 2>, dim3(gx, 1), dim3(kRowsPerCta * 32), 0, s, /*pdl=*/true, false, p);
      } else {
        const int gx = (p.N + kRowsPerCta - 1) / kRowsPerCta;
        if (p.M == 2) launch_kernel(mmvq_q4k_dp4a_kernel<2, 1>, dim3(gx, 1), dim3(kRowsPerCta * 32), 0, s, /*pdl=*/true, false, p);
        else if (p.M <= 4) launch_kernel(mmvq_q4k_dp4a_kernel<4, 1>, dim3(gx, 1), dim3(kRowsPerCta * 32), 0, s, /*pdl=*/true, false, p);
        else launch_kernel(mmvq_q4k_dp4a_kernel<8, 1>, dim3(gx, (p.M + 7) / 8), dim3(kRowsPerCta * 32), 0, s, /*pdl=*/true, false, p);
      }
      return;
    }
    if (aligned && (p.K & 255) == 0) {
      OXB_MMVQ_FAST(mmvq_q4k_kernel);
      return;
    }
  }
  if constexpr (T == kQ_Q8_0) {
    if (p.xq != nullptr && (reinterpret_cast<uintptr_t>(p.w) & 1) == 0 && (p.row_bytes & 1) == 0 &&
        (reinterpret_cast<uintptr_t>(p.xq) & 15) == 0) {
      OXB_MMVQ_FAST(mmvq_q8_0_dp4a_kernel);
      return;
    }
    if ((reinterpret_cast<uintptr_t>(p.w) & 1) == 0 && (p.row_bytes & 1) == 0 &&
        (reinterpret_cast<uintptr_t>(p.x) & 15) == 0 && (p.ldx & 7) == 0) {
      OXB_MMVQ_FAST(mmvq_q8_0_kernel);
      return;
    }
  }
  if constexpr (HasInt8Path<T>::value && T != kQ_Q4_K && T != kQ_Q8_0) {
    if (p.xq != nullptr && int8_operands_ok(T, p.w, p.row_bytes, p)) {
      const int gx = (p.N + kRowsPerCta - 1) / kRowsPerCta;
      if (p.M == 1) launch_kernel(mmvq_int8_kernel<T, 1>, dim3(gx, 1), dim3(kRowsPerCta * 32), 0, s, /*pdl=*/true, false, p);
      else if (p.M == 2) launch_kernel(mmvq_int8_kernel<T, 2>, dim3(gx, 1), dim3(kRowsPerCta * 32), 0, s, /*pdl=*/true, false, p);
      else if (p.M <= 4) launch_kernel(mmvq_int8_kernel<T, 4>, dim3(gx, 1), dim3(kRowsPerCta * 32), 0, s, /*pdl=*/true, false, p);
      else launch_kernel(mmvq_int8_kernel<T, 8>, dim3(gx, (p.M + 7) / 8), dim3(kRowsPerCta * 32), 0, s, /*pdl=*/true, false, p);
      return;
    }
  }
  const int gx = (p.N + kRowsPerCta - 1) / kRowsPerCta;
  if (p.M == 1) {
    launch_kernel(mmvq_kernel<T, 1>, dim3(gx, 1), dim3(kRowsPerCta * 32), 0, s, /*pdl=*/true, false, p);
  } else if (p.M == 2) {
    launch_kernel(mmvq_kernel<T, 2>, dim3(gx, 1), dim3(kRowsPerCta * 32), 0, s, /*pdl=*/true, false, p);
  } else if (p.M <= 4) {
    launch_kernel(mmvq_kernel<T, 4>, dim3(gx, 1), dim3(kRowsPerCta * 32), 0, s, /*pdl=*/true, false, p);
  } else {
    launch_kernel(mmvq_kernel<T, 8>, dim3(gx, (p.M + 7) / 8), dim3(kRowsPerCta * 32), 0, s, /*pdl=*/true, false, p);
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

void launch_quant_q8_1(const __nv_bfloat16* x, long long ldx, int8_t* xq, float* xd, float* xs, int M,
                       int K, cudaStream_t stream) {
  const long long warps = static_cast<long long>(M) * (K >> 5);
  if (warps <= 0) return;
  const int threads = 256;
  launch_kernel(quant_q8_1_kernel, dim3(static_cast<unsigned>((warps * 32 + threads - 1) / threads)), dim3(threads), 0,
                stream, /*pdl=*/true, false, x, ldx, xq, xd, xs, M, K);
}

bool launch_mmvq(int qtype, const MmvqParams& p, cudaStream_t stream) {
  if (p.M <= 0 || p.N <= 0) return true;
#define CALL(T) mmvq_dispatch<T>(p, stream)
  OXB_QDISPATCH(qtype, CALL)
#undef CALL
  return true;
}

bool mmvq_has_int8_path(int qtype) {
  switch (qtype) {
    case kQ_Q4_0: case kQ_Q4_1: case kQ_Q5_0: case kQ_Q5_1: case kQ_Q8_0: case kQ_Q4_K: case kQ_Q5_K: case kQ_Q6_K:
      return true;
    default:
      return false;
  }
}

bool launch_mmvq_mixed(const MmvqParams& p, cudaStream_t stream) {
  if (p.M <= 0 || p.N <= 0) return true;
  if (p.n_seg < 1 || p.n_seg > 4 || p.xq == nullptr) return false;
  for (int i = 0; i < p.n_seg; ++i)
    if (!mmvq_has_int8_path(p.seg_type[i]) || !int8_operands_ok(p.seg_type[i], p.seg_w[i], p.seg_row_bytes[i], p))
      return false;
  const int gx = (p.N + kRowsPerCta - 1) / kRowsPerCta;
  if (p.M == 1) launch_kernel(mmvq_mixed_kernel<1>, dim3(gx, 1), dim3(kRowsPerCta * 32), 0, stream, /*pdl=*/true, false, p);
  else if (p.M == 2) launch_kernel(mmvq_mixed_kernel<2>, dim3(gx, 1), dim3(kRowsPerCta * 32), 0, stream, /*pdl=*/true, false, p);
  else if (p.M <= 4) launch_kernel(mmvq_mixed_kernel<4>, dim3(gx, 1), dim3(kRowsPerCta * 32), 0, stream, /*pdl=*/true, false, p);
  else launch_kernel(mmvq_mixed_kernel<8>, dim3(gx, (p.M + 7) / 8), dim3(kRowsPerCta * 32), 0, stream, /*pdl=*/true, false, p);
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
