// Integer expansion of GGUF blocks, shared by the quantised GEMV kernels and the GEMM whose weight
// operand is unpacked in the kernel.
//
// A group of 32 weights is rebuilt as eight words of four signed bytes q_j with
//   w_j = dl0 * q_j + ml  (j < 16),   w_j = dl1 * q_j + ml  (j >= 16).
// Blocks are read with the widest loads their alignment allows (Q4_0 / Q5_0 / Q8_0 / Q6_K blocks
// are only 2-byte aligned, Q4_1 / Q5_1 4-byte, the K-quants read with 16-byte loads need 16).
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

#include "quant_blocks.cuh"

namespace oxb {

__device__ __forceinline__ uint32_t byte_of3(uint32_t s0, uint32_t s1, uint32_t s2, int k) {
  const uint32_t w = k < 4 ? s0 : (k < 8 ? s1 : s2);
  return (w >> (8 * (k & 3))) & 0xFFu;
}

__device__ __forceinline__ uint32_t ldg_u16(const uint8_t* p) {
  return __ldg(reinterpret_cast<const uint16_t*>(p));
}
__device__ __forceinline__ uint32_t ldg_u32_a2(const uint8_t* p) { return ldg_u16(p) | (ldg_u16(p + 2) << 16); }
__device__ __forceinline__ uint32_t ldg_u32(const uint8_t* p) { return __ldg(reinterpret_cast<const uint32_t*>(p)); }
// N consecutive 32-bit words from a 2-byte aligned address: aligned loads, re-joined with a funnel
// shift when the address is 2 mod 4 (N + 1 loads instead of 2 N halfword loads). Reads at most 2 bytes
// before and after the N words, which callers keep inside the block.
template <int N>
__device__ __forceinline__ void ldg_words_a2(const uint8_t* p, uint32_t (&w)[N]) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(p);
  const uint32_t* q = reinterpret_cast<const uint32_t*>(a & ~uintptr_t(3));
  if ((a & 2) == 0) {
#pragma unroll
    for (int i = 0; i < N; ++i) w[i] = __ldg(q + i);
  } else {
    uint32_t prev = __ldg(q);
#pragma unroll
    for (int i = 0; i < N; ++i) {
      const uint32_t nxt = __ldg(q + i + 1);
      w[i] = __funnelshift_r(prev, nxt, 16);
      prev = nxt;
    }
  }
}
__device__ __forceinline__ float half_bits(uint32_t v) {
  return __half2float(__ushort_as_half(static_cast<uint16_t>(v & 0xFFFFu)));
}
// bits 0..3 of x -> bit 4 of bytes 0..3
__device__ __forceinline__ uint32_t spread_bit4(uint32_t x) {
  return (((x & 0xFu) * 0x00204081u) & 0x01010101u) << 4;
}

template <int T>
struct HasInt8Path {
  static constexpr bool value = T == kQ_Q4_0 || T == kQ_Q4_1 || T == kQ_Q5_0 || T == kQ_Q5_1 || T == kQ_Q8_0 ||
                                T == kQ_Q4_K || T == kQ_Q5_K || T == kQ_Q6_K;
};

template <int T>
__device__ __forceinline__ void expand_q8(const uint8_t* row, int grp, uint32_t (&wq)[8], float& dl0, float& dl1,
                                          float& ml) {
  if constexpr (T == kQ_Q4_0) {
    const uint8_t* b = row + static_cast<long long>(grp) * 18;
    const float d = half_bits(ldg_u16(b));
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const uint32_t w = ldg_u32_a2(b + 2 + 4 * u);
      wq[u] = w & 0x0F0F0F0Fu;
      wq[4 + u] = (w >> 4) & 0x0F0F0F0Fu;
    }
    dl0 = dl1 = d;
    ml = -8.f * d;
  } else if constexpr (T == kQ_Q4_1) {
    const uint8_t* b = row + static_cast<long long>(grp) * 20;
    const uint32_t hdr = ldg_u32(b);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const uint32_t w = ldg_u32(b + 4 + 4 * u);
      wq[u] = w & 0x0F0F0F0Fu;
      wq[4 + u] = (w >> 4) & 0x0F0F0F0Fu;
    }
    dl0 = dl1 = half_bits(hdr);
    ml = half_bits(hdr >> 16);
  } else if constexpr (T == kQ_Q5_0) {
    const uint8_t* b = row + static_cast<long long>(grp) * 22;
    const float d = half_bits(ldg_u16(b));
    const uint32_t qh = ldg_u32_a2(b + 2);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const uint32_t w = ldg_u32_a2(b + 6 + 4 * u);
      wq[u] = (w & 0x0F0F0F0Fu) | spread_bit4(qh >> (4 * u));
      wq[4 + u] = ((w >> 4) & 0x0F0F0F0Fu) | spread_bit4(qh >> (16 + 4 * u));
    }
    dl0 = dl1 = d;
    ml = -16.f * d;
  } else if constexpr (T == kQ_Q5_1) {
    const uint8_t* b = row + static_cast<long long>(grp) * 24;
    const uint32_t hdr = ldg_u32(b);
    const uint32_t qh = ldg_u32(b + 4);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const uint32_t w = ldg_u32(b + 8 + 4 * u);
      wq[u] = (w & 0x0F0F0F0Fu) | spread_bit4(qh >> (4 * u));
      wq[4 + u] = ((w >> 4) & 0x0F0F0F0Fu) | spread_bit4(qh >> (16 + 4 * u));
    }
    dl0 = dl1 = half_bits(hdr);
    ml = half_bits(hdr >> 16);
  } else if constexpr (T == kQ_Q8_0) {
    const uint8_t* b = row + static_cast<long long>(grp) * 34;
    const float d = half_bits(ldg_u16(b));
#pragma unroll
    for (int u = 0; u < 8; ++u) wq[u] = ldg_u32_a2(b + 2 + 4 * u);
    dl0 = dl1 = d;
    ml = 0.f;
  } else if constexpr (T == kQ_Q4_K || T == kQ_Q5_K) {
    // Q4_K: d | dmin | scales[12] | qs[128];  Q5_K: d | dmin | scales[12] | qh[32] | qs[128]
    constexpr int kBytes = T == kQ_Q4_K ? 144 : 176;
    constexpr int kQs = T == kQ_Q4_K ? 16 : 48;
    const uint8_t* b = row + static_cast<long long>(grp >> 3) * kBytes;
    const int sub = grp & 7;
    const uint4 hdr = __ldg(reinterpret_cast<const uint4*>(b));
    int sc, mn;
    if (sub < 4) {
      sc = byte_of3(hdr.y, hdr.z, hdr.w, sub) & 63;
      mn = byte_of3(hdr.y, hdr.z, hdr.w, sub + 4) & 63;
    } else {
      sc = (byte_of3(hdr.y, hdr.z, hdr.w, sub + 4) & 0xF) | ((byte_of3(hdr.y, hdr.z, hdr.w, sub - 4) >> 6) << 4);
      mn = (byte_of3(hdr.y, hdr.z, hdr.w, sub + 4) >> 4) | ((byte_of3(hdr.y, hdr.z, hdr.w, sub) >> 6) << 4);
    }
    const uint4* q = reinterpret_cast<const uint4*>(b + kQs + (sub >> 1) * 32);
    const uint4 qa = __ldg(q), qb = __ldg(q + 1);
    const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
    const int shift = (sub & 1) * 4;
    if constexpr (T == kQ_Q4_K) {
#pragma unroll
      for (int u = 0; u < 8; ++u) wq[u] = (w[u] >> shift) & 0x0F0F0F0Fu;
    } else {
      const uint4* hp = reinterpret_cast<const uint4*>(b + 16);
      const uint4 ha = __ldg(hp), hb = __ldg(hp + 1);
      const uint32_t h[8] = {ha.x, ha.y, ha.z, ha.w, hb.x, hb.y, hb.z, hb.w};
#pragma unroll
      for (int u = 0; u < 8; ++u)
        wq[u] = ((w[u] >> shift) & 0x0F0F0F0Fu) | (((h[u] >> sub) & 0x01010101u) << 4);
    }
    dl0 = dl1 = half_bits(hdr.x) * static_cast<float>(sc);
    ml = -half_bits(hdr.x >> 16) * static_cast<float>(mn);
  } else if constexpr (T == kQ_Q6_K) {
    // ql[128] | qh[64] | scales[16] | d ; 210 bytes, 2-byte aligned
    const uint8_t* b = row + static_cast<long long>(grp >> 3) * 210;
    const int sub = grp & 7, half = sub >> 2, quarter = sub & 3;
    const int nib = (quarter >> 1) * 4, hs = 2 * quarter;
    uint32_t lw[8], hw[8];
    ldg_words_a2<8>(b + half * 64 + (quarter & 1) * 32, lw);
    ldg_words_a2<8>(b + 128 + half * 32, hw);
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const uint32_t lo = (lw[u] >> nib) & 0x0F0F0F0Fu;
      const uint32_t hi = ((hw[u] >> hs) & 0x03030303u) << 4;
      wq[u] = __vsub4(lo | hi, 0x20202020u);
    }
    const uint32_t sc = ldg_u16(b + 192 + half * 8 + quarter * 2);
    const float d = half_bits(ldg_u16(b + 208));
    dl0 = d * static_cast<float>(static_cast<int8_t>(sc & 0xFF));
    dl1 = d * static_cast<float>(static_cast<int8_t>(sc >> 8));
    ml = 0.f;
  }
}

// Both groups of one 64-value k block (groups 2 kb and 2 kb + 1) of a row. The K-quants keep the two
// groups in the same bytes (low / high nibbles, neighbouring bit planes), so their blocks are read once.
template <int T>
__device__ __forceinline__ void expand_q8_pair(const uint8_t* row, int kb, uint32_t (&wq)[2][8], float (&dl0)[2],
                                               float (&dl1)[2], float (&ml)[2]) {
  if constexpr (T == kQ_Q4_K || T == kQ_Q5_K) {
    constexpr int kBytes = T == kQ_Q4_K ? 144 : 176;
    constexpr int kQs = T == kQ_Q4_K ? 16 : 48;
    const uint8_t* b = row + static_cast<long long>(kb >> 2) * kBytes;
    const int j = kb & 3;
    const uint4 hdr = __ldg(reinterpret_cast<const uint4*>(b));
    const uint4* q = reinterpret_cast<const uint4*>(b + kQs + j * 32);
    const uint4 qa = __ldg(q), qb = __ldg(q + 1);
    const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
    uint32_t h[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if constexpr (T == kQ_Q5_K) {
      const uint4* hp = reinterpret_cast<const uint4*>(b + 16);
      const uint4 ha = __ldg(hp), hb = __ldg(hp + 1);
      h[0] = ha.x, h[1] = ha.y, h[2] = ha.z, h[3] = ha.w, h[4] = hb.x, h[5] = hb.y, h[6] = hb.z, h[7] = hb.w;
    }
    const float d = half_bits(hdr.x), dmin = half_bits(hdr.x >> 16);
#pragma unroll
    for (int g = 0; g < 2; ++g) {
      const int sub = 2 * j + g;
      int sc, mn;
      if (sub < 4) {
        sc = byte_of3(hdr.y, hdr.z, hdr.w, sub) & 63;
        mn = byte_of3(hdr.y, hdr.z, hdr.w, sub + 4) & 63;
      } else {
        sc = (byte_of3(hdr.y, hdr.z, hdr.w, sub + 4) & 0xF) | ((byte_of3(hdr.y, hdr.z, hdr.w, sub - 4) >> 6) << 4);
        mn = (byte_of3(hdr.y, hdr.z, hdr.w, sub + 4) >> 4) | ((byte_of3(hdr.y, hdr.z, hdr.w, sub) >> 6) << 4);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        wq[g][u] = (w[u] >> (4 * g)) & 0x0F0F0F0Fu;
        if constexpr (T == kQ_Q5_K) wq[g][u] |= ((h[u] >> sub) & 0x01010101u) << 4;
      }
      dl0[g] = dl1[g] = d * static_cast<float>(sc);
      ml[g] = -dmin * static_cast<float>(mn);
    }
  } else if constexpr (T == kQ_Q6_K) {
    const uint8_t* b = row + static_cast<long long>(kb >> 2) * 210;
    const int half = (kb >> 1) & 1, pi = kb & 1;  // quarters 2 pi and 2 pi + 1 of this half
    uint32_t lw[16], hw[8], sw[1];
    ldg_words_a2<16>(b + half * 64, lw);
    ldg_words_a2<8>(b + 128 + half * 32, hw);
    ldg_words_a2<1>(b + 192 + half * 8 + pi * 4, sw);
    const float d = half_bits(ldg_u16(b + 208));
#pragma unroll
    for (int g = 0; g < 2; ++g) {
      const int hs = 4 * pi + 2 * g;
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const uint32_t lo = (lw[8 * g + u] >> (4 * pi)) & 0x0F0F0F0Fu;
        const uint32_t hi = ((hw[u] >> hs) & 0x03030303u) << 4;
        wq[g][u] = __vsub4(lo | hi, 0x20202020u);
      }
      dl0[g] = d * static_cast<float>(static_cast<int8_t>((sw[0] >> (16 * g)) & 0xFF));
      dl1[g] = d * static_cast<float>(static_cast<int8_t>((sw[0] >> (16 * g + 8)) & 0xFF));
      ml[g] = 0.f;
    }
  } else {
    expand_q8<T>(row, 2 * kb, wq[0], dl0[0], dl1[0], ml[0]);
    expand_q8<T>(row, 2 * kb + 1, wq[1], dl0[1], dl1[1], ml[1]);
  }
}

}  // namespace oxb
