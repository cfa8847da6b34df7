// GGML-exact block layouts of the GGUF weight types and per-type device decoders.
// Each decoder expands one group of 32 consecutive weights of a row into fp32.
// Layouts follow the GGUF files written by llama.cpp-compatible tools (the reference's
// CUDA kernels decode the same layouts: quant_gemv_standard.cu:16-64,182-338,452-612,753-804;
// quant_gemv_kquants.cu:1189-1376; block sizes norms_rope.cu:323-388).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace oxb {

// GGUF tensor type codes (subset with device decoders)
enum QuantType : int {
  kQ_F32 = 0,
  kQ_F16 = 1,
  kQ_Q4_0 = 2,
  kQ_Q4_1 = 3,
  kQ_Q5_0 = 6,
  kQ_Q5_1 = 7,
  kQ_Q8_0 = 8,
  kQ_Q2_K = 10,
  kQ_Q3_K = 11,
  kQ_Q4_K = 12,
  kQ_Q5_K = 13,
  kQ_Q6_K = 14,
  kQ_IQ4_NL = 20,
  kQ_BF16 = 30,
  kQ_TQ2_0 = 35,
  kQ_NVFP4 = 144,
};

template <int T> struct QInfo;
template <> struct QInfo<kQ_Q4_0> { static constexpr int qk = 32, bytes = 18; };
template <> struct QInfo<kQ_Q4_1> { static constexpr int qk = 32, bytes = 20; };
template <> struct QInfo<kQ_Q5_0> { static constexpr int qk = 32, bytes = 22; };
template <> struct QInfo<kQ_Q5_1> { static constexpr int qk = 32, bytes = 24; };
template <> struct QInfo<kQ_Q8_0> { static constexpr int qk = 32, bytes = 34; };
template <> struct QInfo<kQ_Q2_K> { static constexpr int qk = 256, bytes = 84; };
template <> struct QInfo<kQ_Q3_K> { static constexpr int qk = 256, bytes = 110; };
template <> struct QInfo<kQ_Q4_K> { static constexpr int qk = 256, bytes = 144; };
template <> struct QInfo<kQ_Q5_K> { static constexpr int qk = 256, bytes = 176; };
template <> struct QInfo<kQ_Q6_K> { static constexpr int qk = 256, bytes = 210; };
template <> struct QInfo<kQ_IQ4_NL> { static constexpr int qk = 32, bytes = 18; };
template <> struct QInfo<kQ_TQ2_0> { static constexpr int qk = 256, bytes = 66; };
// 16 weights: e4m3 scale at byte 0, 8 nibble bytes at 1..8, padded to a 16-byte stride
template <> struct QInfo<kQ_NVFP4> { static constexpr int qk = 16, bytes = 16; };

__device__ __forceinline__ float ld_half(const uint8_t* p) {
  const uint16_t v = static_cast<uint16_t>(p[0]) | (static_cast<uint16_t>(p[1]) << 8);
  return __half2float(__ushort_as_half(v));
}

__device__ __forceinline__ float e4m3_to_float(uint8_t v) {
  const int s = v >> 7, e = (v >> 3) & 0xF, m = v & 7;
  float r;
  if (e == 0) {
    r = ldexpf(static_cast<float>(m), -9);
  } else if (e == 15 && m == 7) {
    r = 0.f;  // NaN encoding never produced by the writer; decoded as 0
  } else {
    r = ldexpf(1.f + static_cast<float>(m) * 0.125f, e - 7);
  }
  return s ? -r : r;
}

__device__ __constant__ int8_t kIq4nlValues[16] = {-127, -104, -83, -65, -49, -35, -22, -10,
                                                   1,    13,   25,  38,  53,  69,  89,  113};
__device__ __constant__ float kE2M1[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};

__device__ __forceinline__ void scale_min_k4(int j, const uint8_t* q, int& sc, int& mn) {
  if (j < 4) {
    sc = q[j] & 63;
    mn = q[j + 4] & 63;
  } else {
    sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
    mn = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
  }
}

// Expands weights [32*grp, 32*grp+32) of the row starting at `row` into w[32].
template <int T>
__device__ __forceinline__ void dequant32(const uint8_t* row, int grp, float (&w)[32]) {
  if constexpr (T == kQ_Q4_0) {
    const uint8_t* b = row + static_cast<long long>(grp) * 18;
    const float d = ld_half(b);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int q = b[2 + j];
      w[j] = static_cast<float>((q & 0xF) - 8) * d;
      w[j + 16] = static_cast<float>((q >> 4) - 8) * d;
    }
  } else if constexpr (T == kQ_Q4_1) {
    const uint8_t* b = row + static_cast<long long>(grp) * 20;
    const float d = ld_half(b), m = ld_half(b + 2);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int q = b[4 + j];
      w[j] = static_cast<float>(q & 0xF) * d + m;
      w[j + 16] = static_cast<float>(q >> 4) * d + m;
    }
  } else if constexpr (T == kQ_Q5_0) {
    const uint8_t* b = row + static_cast<long long>(grp) * 22;
    const float d = ld_half(b);
    const uint32_t qh = static_cast<uint32_t>(b[2]) | (static_cast<uint32_t>(b[3]) << 8) |
                        (static_cast<uint32_t>(b[4]) << 16) | (static_cast<uint32_t>(b[5]) << 24);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int q = b[6 + j];
      const int h0 = ((qh >> j) << 4) & 0x10;
      const int h1 = (qh >> (j + 12)) & 0x10;
      w[j] = static_cast<float>(((q & 0xF) | h0) - 16) * d;
      w[j + 16] = static_cast<float>(((q >> 4) | h1) - 16) * d;
    }
  } else if constexpr (T == kQ_Q5_1) {
    const uint8_t* b = row + static_cast<long long>(grp) * 24;
    const float d = ld_half(b), m = ld_half(b + 2);
    const uint32_t qh = static_cast<uint32_t>(b[4]) | (static_cast<uint32_t>(b[5]) << 8) |
                        (static_cast<uint32_t>(b[6]) << 16) | (static_cast<uint32_t>(b[7]) << 24);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int q = b[8 + j];
      const int h0 = ((qh >> j) << 4) & 0x10;
      const int h1 = (qh >> (j + 12)) & 0x10;
      w[j] = static_cast<float>((q & 0xF) | h0) * d + m;
      w[j + 16] = static_cast<float>((q >> 4) | h1) * d + m;
    }
  } else if constexpr (T == kQ_Q8_0) {
    const uint8_t* b = row + static_cast<long long>(grp) * 34;
    const float d = ld_half(b);
#pragma unroll
    for (int j = 0; j < 32; ++j) w[j] = static_cast<float>(static_cast<int8_t>(b[2 + j])) * d;
  } else if constexpr (T == kQ_IQ4_NL) {
    const uint8_t* b = row + static_cast<long long>(grp) * 18;
    const float d = ld_half(b);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int q = b[2 + j];
      w[j] = static_cast<float>(kIq4nlValues[q & 0xF]) * d;
      w[j + 16] = static_cast<float>(kIq4nlValues[q >> 4]) * d;
    }
  } else if constexpr (T == kQ_Q2_K) {
    // scales[16] | qs[64] | d | dmin
    const uint8_t* b = row + static_cast<long long>(grp >> 3) * 84;
    const int sub = grp & 7, n = sub >> 2, j = sub & 3;
    const float d = ld_half(b + 80), dmin = ld_half(b + 82);
    const uint8_t* q = b + 16 + n * 32;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int sc = b[n * 8 + j * 2 + half];
      const float dl = d * static_cast<float>(sc & 0xF), ml = dmin * static_cast<float>(sc >> 4);
#pragma unroll
      for (int l = 0; l < 16; ++l)
        w[half * 16 + l] = dl * static_cast<float>((q[half * 16 + l] >> (2 * j)) & 3) - ml;
    }
  } else if constexpr (T == kQ_Q3_K) {
    // hmask[32] | qs[64] | scales[12] | d
    const uint8_t* b = row + static_cast<long long>(grp >> 3) * 110;
    const int sub = grp & 7, n = sub >> 2, j = sub & 3;
    const float d_all = ld_half(b + 108);
    const uint8_t* sc12 = b + 96;
    uint32_t aux[4];
    aux[0] = sc12[0] | (sc12[1] << 8) | (sc12[2] << 16) | (static_cast<uint32_t>(sc12[3]) << 24);
    aux[1] = sc12[4] | (sc12[5] << 8) | (sc12[6] << 16) | (static_cast<uint32_t>(sc12[7]) << 24);
    const uint32_t tmp =
        sc12[8] | (sc12[9] << 8) | (sc12[10] << 16) | (static_cast<uint32_t>(sc12[11]) << 24);
    const uint32_t km1 = 0x03030303u, km2 = 0x0f0f0f0fu;
    const uint32_t a0 = aux[0], a1 = aux[1];
    aux[2] = ((a0 >> 4) & km2) | (((tmp >> 4) & km1) << 4);
    aux[3] = ((a1 >> 4) & km2) | (((tmp >> 6) & km1) << 4);
    aux[0] = (a0 & km2) | (((tmp >> 0) & km1) << 4);
    aux[1] = (a1 & km2) | (((tmp >> 2) & km1) << 4);
    const uint8_t* q = b + 32 + n * 32;
    const uint8_t* hm = b;
    const int mbit = 1 << (n * 4 + j);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int is = n * 8 + j * 2 + half;
      const int sc = static_cast<int8_t>((aux[is >> 2] >> (8 * (is & 3))) & 0xFF) - 32;
      const float dl = d_all * static_cast<float>(sc);
#pragma unroll
      for (int l = 0; l < 16; ++l) {
        const int idx = half * 16 + l;
        const int v = ((q[idx] >> (2 * j)) & 3) - ((hm[idx] & mbit) ? 0 : 4);
        w[idx] = dl * static_cast<float>(v);
      }
    }
  } else if constexpr (T == kQ_Q4_K) {
    // d | dmin | scales[12] | qs[128]
    const uint8_t* b = row + static_cast<long long>(grp >> 3) * 144;
    const int sub = grp & 7;
    const float d = ld_half(b), dmin = ld_half(b + 2);
    int sc, mn;
    scale_min_k4(sub, b + 4, sc, mn);
    const float dl = d * static_cast<float>(sc), ml = dmin * static_cast<float>(mn);
    const uint8_t* q = b + 16 + (sub >> 1) * 32;
    const int shift = (sub & 1) * 4;
#pragma unroll
    for (int l = 0; l < 32; ++l) w[l] = dl * static_cast<float>((q[l] >> shift) & 0xF) - ml;
  } else if constexpr (T == kQ_Q5_K) {
    // d | dmin | scales[12] | qh[32] | qs[128]
    const uint8_t* b = row + static_cast<long long>(grp >> 3) * 176;
    const int sub = grp & 7;
    const float d = ld_half(b), dmin = ld_half(b + 2);
    int sc, mn;
    scale_min_k4(sub, b + 4, sc, mn);
    const float dl = d * static_cast<float>(sc), ml = dmin * static_cast<float>(mn);
    const uint8_t* qh = b + 16;
    const uint8_t* q = b + 48 + (sub >> 1) * 32;
    const int shift = (sub & 1) * 4;
#pragma unroll
    for (int l = 0; l < 32; ++l) {
      const int hi = (qh[l] >> sub) & 1;
      w[l] = dl * static_cast<float>(((q[l] >> shift) & 0xF) + (hi << 4)) - ml;
    }
  } else if constexpr (T == kQ_Q6_K) {
    // ql[128] | qh[64] | scales[16] | d
    const uint8_t* b = row + static_cast<long long>(grp >> 3) * 210;
    const int sub = grp & 7, half = sub >> 2, quarter = sub & 3;
    const float d = ld_half(b + 208);
    const uint8_t* ql = b + half * 64 + (quarter & 1) * 32;
    const uint8_t* qh = b + 128 + half * 32;
    const int8_t* sc = reinterpret_cast<const int8_t*>(b + 192) + half * 8 + quarter * 2;
    const int nib = (quarter >> 1) * 4;
#pragma unroll
    for (int l = 0; l < 32; ++l) {
      const int q = ((ql[l] >> nib) & 0xF) | (((qh[l] >> (2 * quarter)) & 3) << 4);
      w[l] = d * static_cast<float>(sc[l >> 4]) * static_cast<float>(q - 32);
    }
  } else if constexpr (T == kQ_TQ2_0) {
    // qs[64] | d
    const uint8_t* b = row + static_cast<long long>(grp >> 3) * 66;
    const int sub = grp & 7, j = sub >> 2, l = sub & 3;
    const float d = ld_half(b + 64);
    const uint8_t* q = b + j * 32;
#pragma unroll
    for (int m = 0; m < 32; ++m) w[m] = static_cast<float>(((q[m] >> (2 * l)) & 3) - 1) * d;
  } else if constexpr (T == kQ_NVFP4) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint8_t* b = row + (static_cast<long long>(grp) * 2 + h) * 16;
      const float s = e4m3_to_float(b[0]);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int q = b[1 + i];
        const float lo = kE2M1[q & 7], hi = kE2M1[(q >> 4) & 7];
        w[h * 16 + i] = ((q & 8) ? -lo : lo) * s;
        w[h * 16 + i + 8] = ((q & 0x80) ? -hi : hi) * s;
      }
    }
  }
}

}  // namespace oxb
