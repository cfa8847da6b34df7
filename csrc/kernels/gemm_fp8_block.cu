// tcgen05 fp8 GEMM with DeepSeek-style block scales for sm_100a.
//
//   C[m, n] = sum_kb  sa[m, kb] * sw[n / 128, kb] * sum_{k in block kb} A8[m, k] * W8[n, k]
//
// One CTA computes a 128 x 128 output tile. K advances in blocks of 128 fp8 values (128 bytes =
// one swizzle atom row). Every K block is one fresh accumulation (`kind::f8f6f4`, four K=32
// instructions) into one of two TMEM buffers; the four epilogue warps read that buffer back,
// multiply by the two scales of the block and add into fp32 registers (the "promotion" that keeps
// the scales outside the tensor core), while the MMA warp already fills the other buffer.
// Warp 0 feeds a TMA ring, warp 1 issues the MMAs; every wait is bounded.
//
// Reference counterpart: the e4m3 codec and the scaled fp8 block of crates/oxide-quant/src/fp8.rs
// (Fp8E4M3 :13-98, BlockFp8E4M3 quantize / dequantize / dot_product :185-245). The reference has no
// fp8 tensor-core GEMM; the 1x128 activation / 128x128 weight scale grid here is the usual layout of
// block-scaled fp8 checkpoints.
#include "gemm_fp8_block.cuh"

#include <cuda_fp8.h>

#include "../common/device_info.h"
#include "../common/sm100.cuh"

namespace oxb {

namespace {

constexpr int BM = 128, BN = 128, BKB = 128;  // BKB: bytes = fp8 elements per K block
constexpr int STAGES = 5;
constexpr int kTileBytes = 128 * BKB;  // A tile = B tile = 16 KB
constexpr int kThreads = 192;
constexpr int kBarOffset = STAGES * 2 * kTileBytes;
constexpr int kSmemTotal = kBarOffset + 256 + 1024;

__global__ void __launch_bounds__(kThreads, 1)
gemm_fp8_block_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const Fp8GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem =
      reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * kTileBytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kBarOffset);
  uint64_t* empty = full + STAGES;
  uint64_t* tmem_full = empty + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
  const int n_kb = (p.K + BKB - 1) / BKB;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(&tmem_full[0], 1);
    mbar_init(&tmem_full[1], 1);
    mbar_init(&tmem_empty[0], 4);
    mbar_init(&tmem_empty[1], 4);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      for (int kb = 0; kb < n_kb; ++kb) {
        const int s = kb % STAGES;
        if (kb >= STAGES && !mbar_wait(&empty[s], ((kb / STAGES) & 1) ^ 1)) {
          set_status_once(p.status, kStatusMbarTimeoutProducer);
          break;
        }
        mbar_arrive_expect_tx(&full[s], 2 * kTileBytes);
        tma_load_2d(sB + s * kTileBytes, &tmB, &full[s], kb * BKB, n0);
        tma_load_2d(sA + s * kTileBytes, &tmA, &full[s], kb * BKB, m0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(kFmtE4M3, kFmtE4M3, BM, BN);
      for (int kb = 0; kb < n_kb; ++kb) {
        const int s = kb % STAGES;
        const uint32_t buf = kb & 1;
        if (kb >= 2 && !mbar_wait(&tmem_empty[buf], ((kb >> 1) & 1) ^ 1)) {
          set_status_once(p.status, kStatusMbarTimeoutMma);
          break;
        }
        if (!mbar_wait(&full[s], (kb / STAGES) & 1)) {
          set_status_once(p.status, kStatusMbarTimeoutMma);
          break;
        }
        tc_fence_after_sync();
        const uint32_t a_addr = smem_u32(sA + s * kTileBytes);
        const uint32_t b_addr = smem_u32(sB + s * kTileBytes);
#pragma unroll
        for (int k = 0; k < BKB / 32; ++k)
          tc_mma_f8(tmem_base + buf * BN, make_desc_kmajor_sw128(a_addr + k * 32),
                    make_desc_kmajor_sw128(b_addr + k * 32), idesc, k != 0 ? 1u : 0u);
        tc_commit(&empty[s]);
        tc_commit(&tmem_full[buf]);
      }
    }
  } else {
    const int q = warp & 3;
    const int row = m0 + q * 32 + lane;
    const bool row_ok = row < p.M;
    const int kb_cols = n_kb;
    const float* sw_row = p.sw + static_cast<long long>(blockIdx.y) * kb_cols;
    float acc[BN];
#pragma unroll
    for (int j = 0; j < BN; ++j) acc[j] = 0.f;
    bool ok = true;
    for (int kb = 0; kb < n_kb; ++kb) {
      const uint32_t buf = kb & 1;
      if (ok && !mbar_wait(&tmem_full[buf], (kb >> 1) & 1)) {
        if (lane == 0) set_status_once(p.status, kStatusMbarTimeoutEpilogue);
        ok = false;
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const float sc = (row_ok ? __ldg(p.sa_t + static_cast<long long>(kb) * p.sa_ld + row) : 0.f) *
                       __ldg(sw_row + kb);
      const uint32_t lane_addr = tmem_base + buf * BN + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(lane_addr + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[c * 32 + j] = fmaf(__uint_as_float(r[j]), sc, acc[c * 32 + j]);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[buf]);
    }
    if (ok && row_ok) {
      __nv_bfloat16* d = p.C + static_cast<long long>(row) * p.ldc + n0;
      long long ld = p.ldc;
      if (p.n_owners > 0) {
        int owner = row / p.rows_per_owner;
        if (owner >= p.n_owners) owner = p.n_owners - 1;
        __nv_bfloat16* base = nullptr;
#pragma unroll
        for (int o = 0; o < 8; ++o)
          if (o == owner) base = p.slab[o];
        d = base + (static_cast<long long>(p.my_rank) * p.rows_per_owner + (row - owner * p.rows_per_owner)) * p.slab_ld + n0;
        ld = p.slab_ld;
      }
      const bool vec = (ld & 7) == 0 && n0 + BN <= p.N;
#pragma unroll
      for (int j = 0; j < BN; j += 8) {
        float v[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          v[e] = acc[j + e];
          if (p.bias != nullptr && n0 + j + e < p.N) v[e] += __bfloat162float(p.bias[n0 + j + e]);
        }
        if (vec) {
          uint4 o4;
          o4.x = pack_bf16x2(v[0], v[1]);
          o4.y = pack_bf16x2(v[2], v[3]);
          o4.z = pack_bf16x2(v[4], v[5]);
          o4.w = pack_bf16x2(v[6], v[7]);
          *reinterpret_cast<uint4*>(d + j) = o4;
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e)
            if (n0 + j + e < p.N) d[j + e] = __float2bfloat16(v[e]);
        }
      }
    }
    tc_fence_before_sync();
    if (p.done_ticket != nullptr) {
      // one system-scope fence per CTA after the barrier, then the grid-wide ticket; the last CTA
      // signals every owner with relaxed adds (see the bf16 GEMM for the reasoning)
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (warp == 2 && lane == 0) {
        __threadfence_system();
        const uint32_t total = gridDim.x * gridDim.y;
        const uint32_t old = atomicAdd(p.done_ticket, 1u);
        if (old == total - 1) {
          *p.done_ticket = 0;
          __threadfence_system();
#pragma unroll
          for (int o = 0; o < 8; ++o)
            if (o < p.n_owners && p.arrive[o] != nullptr)
              asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p.arrive[o]), "r"(1u) : "memory");
        }
      }
    }
  }

  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

// One warp per (row, 128-wide block).
__global__ void quant_act_fp8_kernel(const __nv_bfloat16* x, long long x_ld, uint8_t* __restrict__ q,
                                     long long q_ld, float* __restrict__ sa_t, int sa_ld, int M, int K,
                                     const QuantActWait w) {
  const int n_kb = (K + 127) / 128;
  const long long wid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w.flags != nullptr) {
    // The input rows are pushed by peers (all-gather): wait, bounded, for the sources of the rows
    // this CTA touches, then pass the grid-wide gate whose last passer re-arms the flags.
    __shared__ int s_ok;
    if (threadIdx.x == 0) {
      const long long w0 = (static_cast<long long>(blockIdx.x) * blockDim.x) >> 5;
      long long w1 = w0 + (blockDim.x >> 5) - 1;
      const long long w_max = static_cast<long long>(M) * n_kb - 1;
      if (w1 > w_max) w1 = w_max;
      int s_lo = 0, s_hi = w.n_src - 1;
      if (w.rows_per_src > 0 && w0 <= w_max) {
        s_lo = static_cast<int>(w0 / n_kb) / w.rows_per_src;
        s_hi = static_cast<int>(w1 / n_kb) / w.rows_per_src;
        if (s_hi >= w.n_src) s_hi = w.n_src - 1;
        if (s_lo > s_hi) s_lo = s_hi;
      }
      int ok = 1;
      for (int s = s_lo; s <= s_hi && ok; ++s) {
        uint32_t it = 0, v;
        do {
          asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(w.flags + s) : "memory");
          if (v >= w.expected) break;
        } while (++it <= OXB_SPIN_LIMIT);
        if (v < w.expected) {
          set_status_peer_timeout(w.status);
          ok = 0;
        }
      }
      const uint32_t old = atomicAdd(w.ticket, 1u);
      if (old == gridDim.x - 1) {
        for (int s = 0; s < w.n_src; ++s) const_cast<uint32_t*>(w.flags)[s] = 0;
        __threadfence();
        *w.ticket = 0;
      }
      s_ok = ok;
    }
    __syncthreads();
    if (!s_ok) return;
  }
  if (wid >= static_cast<long long>(M) * n_kb) return;
  const int row = static_cast<int>(wid / n_kb), kb = static_cast<int>(wid % n_kb);
  const int k0 = kb * 128 + lane * 4;
  float v[4];
  const __nv_bfloat16* xr = x + static_cast<long long>(row) * x_ld + k0;
  if (k0 + 3 < K && (reinterpret_cast<uintptr_t>(xr) & 7) == 0) {
    // L2 load: the rows may have been written by a peer GPU moments ago
    const uint2 raw = __ldcg(reinterpret_cast<const uint2*>(xr));
    const __nv_bfloat16* e4 = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) v[e] = __bfloat162float(e4[e]);
  } else {
#pragma unroll
    for (int e = 0; e < 4; ++e)
      v[e] = k0 + e < K
                 ? __bfloat162float(__ushort_as_bfloat16(__ldcg(reinterpret_cast<const unsigned short*>(xr + e))))
                 : 0.f;
  }
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
  amax = warp_max(amax);
  const float scale = fmaxf(amax, 1e-10f) / 448.f;
  const float inv = 1.f / scale;
  if (lane == 0) sa_t[static_cast<long long>(kb) * sa_ld + row] = scale;
#pragma unroll
  for (int e = 0; e < 4; ++e)
    if (k0 + e < K)
      q[static_cast<long long>(row) * q_ld + k0 + e] =
          static_cast<uint8_t>(__nv_cvt_float_to_fp8(v[e] * inv, __NV_SATFINITE, __NV_E4M3));
}

}  // namespace

void launch_gemm_fp8_block(const CUtensorMap& tmA, const CUtensorMap& tmB, const Fp8GemmParams& p,
                           cudaStream_t stream) {
  ensure_dynamic_smem(gemm_fp8_block_kernel, kSmemTotal);
  dim3 grid((p.M + BM - 1) / BM, (p.N + BN - 1) / BN);
  gemm_fp8_block_kernel<<<grid, kThreads, kSmemTotal, stream>>>(tmA, tmB, p);
}

void launch_quant_act_fp8(const __nv_bfloat16* x, long long x_ld, uint8_t* q, long long q_ld,
                          float* sa_t, int sa_ld, int M, int K, const QuantActWait& wait,
                          cudaStream_t stream) {
  const long long warps = static_cast<long long>(M) * ((K + 127) / 128);
  const int threads = 256;
  const long long blocks = (warps * 32 + threads - 1) / threads;
  quant_act_fp8_kernel<<<static_cast<unsigned>(blocks), threads, 0, stream>>>(x, x_ld, q, q_ld, sa_t,
                                                                             sa_ld, M, K, wait);
}

}  // namespace oxb
