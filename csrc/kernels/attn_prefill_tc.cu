// Paged causal flash-attention for prefill chunks on the 5th-generation tensor cores (sm_100a).
//
// One CTA = one 128-row query tile of one (sequence, query head). KV is streamed in tiles of 128
// tokens (8 pages of the block table), each page fetched by TMA straight from the paged cache into
// 128B-swizzled shared memory. Per KV tile:
//     S  = Q K^T          tcgen05.mma, fp32 accumulator in TMEM (double buffered)
//     P  = exp2(S - m)    softmax warps: one thread per query row reads its row with tcgen05.ld, so
//                         row max / row sum need no cross-thread reduction; P goes back to shared
//                         memory in the swizzled K-major layout the next MMA expects
//     O += P V            tcgen05.mma with V as an MN-major operand, accumulator in TMEM
// The running maximum is updated lazily (O is rescaled in TMEM only when a row's maximum grows by
// more than 2^8), causal / sliding-window masks are applied from absolute positions, and the
// tiles above the diagonal are skipped. Warp roles: warp 0 = TMA producer, warp 1 = MMA issuer,
// warps 2..5 = softmax + epilogue. Every wait is bounded.
//
// Replaces flash_causal_batched_prefill_kernel
// (oxide-backend-cuda/src/kernels/flash_attn.cu:536-781), an O(S^2) scalar kernel over a
// contiguous slot cache.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/device_info.h"
#include "../common/sm100.cuh"
#include "attn.cuh"

namespace oxb {

namespace {

constexpr int BQ = 128;
constexpr int BKV = 128;
constexpr int kHalfBytes = 128 * 64 * 2;  // one [128 x 64] bf16 sub-tile (16 KB)
constexpr int kThreads = 192;

__device__ __forceinline__ float ex2a(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int D>
struct Smem {
  static constexpr int DH = D / 64;
  static constexpr int kQ = 0;
  static constexpr int kK = kQ + DH * kHalfBytes;           // 2 stages
  static constexpr int kV = kK + 2 * DH * kHalfBytes;       // 2 stages
  static constexpr int kP = kV + 2 * DH * kHalfBytes;       // [128 x 128] as two halves
  static constexpr int kBar = kP + 2 * kHalfBytes;
  static constexpr int kTotal = kBar + 256 + 1024;
};

template <int D>
__global__ void __launch_bounds__(kThreads, 1)
prefill_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const PrefillAttnParams p, int* status) {
  using L = Smem<D>;
  constexpr int DH = D / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem =
      reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + L::kQ;
  uint8_t* sK = smem + L::kK;
  uint8_t* sV = smem + L::kV;
  uint8_t* sP = smem + L::kP;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBar);
  uint64_t* q_full = bars;           // 1
  uint64_t* k_full = bars + 1;       // 2
  uint64_t* v_full = bars + 3;       // 2
  uint64_t* kv_empty = bars + 5;     // 2
  uint64_t* s_full = bars + 7;       // 2
  uint64_t* s_empty = bars + 9;      // 2
  uint64_t* p_full = bars + 11;      // 1
  uint64_t* pv_done = bars + 12;     // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);

  const int tile = blockIdx.x;
  const int head = blockIdx.y;
  const int q0 = p.tile_q0[tile];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int seq = p.tile_seq[tile];
  const int q_len = p.q_lens[seq];
  const int ctx = p.ctx_lens[seq];
  const int row_base = p.q_start[seq];
  const int pos_off = ctx - q_len;
  const int G = p.Hq / p.Hkv;
  const int kvh = head / G;

  int last_row = q0 + BQ - 1;
  if (last_row > q_len - 1) last_row = q_len - 1;
  const int max_pos = pos_off + last_row;
  int first_tile = 0;
  if (p.window > 0) {
    const int lo = pos_off + q0 - p.window + 1;
    if (lo > 0) first_tile = lo / BKV;
  }
  const int n_tiles = max_pos / BKV + 1 - first_tile;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&kv_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 4);
    }
    mbar_init(p_full, 4);
    mbar_init(pv_done, 1);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s0 = tmem_base;        // S buffers: columns [0,128) and [128,256)
  const uint32_t tmem_o = tmem_base + 256;   // O: D columns

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    // The whole warp issues: a KV tile is 8 pages x DH halves x {K, V} = up to 32 boxes of 2 KB,
    // and copies issued by ONE thread complete about one per memory round trip (their rate grows
    // with the number of issuing threads, not with the number in flight), which would bound a tile
    // at several microseconds against half a microsecond of MMA work. Lane = (tensor, page, half).
    {
      if (lane == 0) mbar_arrive_expect_tx(q_full, DH * kHalfBytes);
      __syncwarp();
      if (lane < DH) tma_load_2d(sQ + lane * kHalfBytes, &tmQ, q_full, head * D + lane * 64, row_base + q0);
      const int* bt = p.block_tables + static_cast<long long>(seq) * p.max_blocks;
      constexpr int kOps = 2 * (BKV / 16) * DH;  // 32 (D = 128) or 16 (D = 64)
      const bool issuer = lane < kOps;
      const int is_v = lane / (kOps / 2);
      const int pg = (lane % (kOps / 2)) / DH;
      const int hf = lane % DH;
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j & 1;
        if (j >= 2 && !mbar_wait(&kv_empty[s], ((j >> 1) - 1) & 1)) ok = false;
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) set_status_once(status, kStatusMbarTimeoutProducer);
          break;
        }
        if (lane == 0) {
          mbar_arrive_expect_tx(&k_full[s], DH * kHalfBytes);
          mbar_arrive_expect_tx(&v_full[s], DH * kHalfBytes);
        }
        __syncwarp();
        if (issuer) {
          const int pi = (first_tile + j) * (BKV / 16) + pg;
          int blk = pi < p.max_blocks ? bt[pi] : 0;
          if (p.num_blocks > 0 && static_cast<unsigned>(blk) >= static_cast<unsigned>(p.num_blocks)) {
            set_status_once(status, kStatusBadIndex);
            blk = 0;
          }
          const int row = (blk * p.Hkv + kvh) * 16;
          if (is_v)
            tma_load_2d(sV + (s * DH + hf) * kHalfBytes + pg * 2048, &tmV, &v_full[s], hf * 64, row);
          else
            tma_load_2d(sK + (s * DH + hf) * kHalfBytes + pg * 2048, &tmK, &k_full[s], hf * 64, row);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(kFmtBF16, kFmtBF16, BQ, BKV);
      constexpr uint32_t idesc_o = make_idesc(kFmtBF16, kFmtBF16, BQ, D, 0, 1);  // V is MN-major
      bool ok = mbar_wait(q_full, 0);
      if (!ok) set_status_once(status, kStatusMbarTimeoutMma);
      auto issue_s = [&](int j) -> bool {
        const int s = j & 1;
        if (!mbar_wait(&k_full[s], (j >> 1) & 1)) return false;
        if (j >= 2 && !mbar_wait(&s_empty[s], ((j >> 1) - 1) & 1)) return false;
        tc_fence_after_sync();
        const uint32_t qa = smem_u32(sQ);
        const uint32_t kb = smem_u32(sK + s * DH * kHalfBytes);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * kHalfBytes + (kk & 3) * 32;
          tc_mma_f16(tmem_s0 + s * BKV, make_desc_kmajor_sw128(qa + off), make_desc_kmajor_sw128(kb + off),
                     idesc_s, kk != 0 ? 1u : 0u);
        }
        tc_commit(&s_full[s]);
        return true;
      };
      if (ok && n_tiles > 0) ok = issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j & 1;
        if (j + 1 < n_tiles) ok = issue_s(j + 1);
        if (!ok) break;
        if (!mbar_wait(p_full, j & 1) || !mbar_wait(&v_full[s], (j >> 1) & 1)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t pa = smem_u32(sP);
        const uint32_t vb = smem_u32(sV + s * DH * kHalfBytes);
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
          const uint32_t aoff = (kk >> 2) * kHalfBytes + (kk & 3) * 32;
          tc_mma_f16(tmem_o, make_desc_kmajor_sw128(pa + aoff),
                     make_desc_mnmajor_sw128(vb + kk * 2048, kHalfBytes, 1024), idesc_o,
                     (j | kk) != 0 ? 1u : 0u);
        }
        tc_commit(&kv_empty[s]);
        tc_commit(pv_done);
      }
      if (!ok) set_status_once(status, kStatusMbarTimeoutMma);
    }
  } else {
    // ------------------------------ softmax + epilogue ------------------------
    const int q = warp & 3;
    const int r = q * 32 + lane;  // query row of this thread == TMEM lane
    const int qi = q0 + r;
    const bool row_valid = qi < q_len;
    const int pos = pos_off + (row_valid ? qi : q_len - 1);
    const uint32_t lane_sel = static_cast<uint32_t>(q * 32) << 16;
    float m_used = -INFINITY, l_sum = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int b = j & 1;
      if (ok && !mbar_wait(&s_full[b], (j >> 1) & 1)) ok = false;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t s_addr = tmem_s0 + b * BKV + lane_sel;
      const int t0 = (first_tile + j) * BKV;
      // ---- pass 1: row maximum over the unmasked scores ----
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < BKV / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(s_addr + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int t = t0 + c * 32 + i;
          const bool keep = t <= pos && (p.window <= 0 || t > pos - p.window);
          if (keep) mx = fmaxf(mx, __uint_as_float(v[i]));
        }
      }
      mx *= p.scale_log2;
      float alpha = 1.f;
      bool grow = false;
      if (mx > m_used + 8.f || (m_used == -INFINITY && mx > -INFINITY)) {
        alpha = m_used == -INFINITY ? 0.f : ex2a(m_used - mx);
        m_used = mx;
        grow = true;
      }
      // PV of the previous tile must be complete before P or O are touched
      if (j > 0) {
        if (ok && !mbar_wait(pv_done, (j - 1) & 1)) ok = false;
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
      }
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
        // lazy rescale of this warp's 32 accumulator rows in TMEM
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(tmem_o + lane_sel + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
          tmem_st_32x32b_x32(tmem_o + lane_sel + c * 32, v);
        }
        tmem_st_wait();
      }
      l_sum *= alpha;
      const float m_sub = m_used == -INFINITY ? 0.f : m_used;
      // ---- pass 2: P = exp2(S * scale - m), row sum, swizzled K-major store ----
#pragma unroll 1
      for (int c = 0; c < BKV / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(s_addr + c * 32, v);
        tmem_ld_wait();
        float pv[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int t = t0 + c * 32 + i;
          const bool keep = t <= pos && (p.window <= 0 || t > pos - p.window);
          pv[i] = keep ? ex2a(__uint_as_float(v[i]) * p.scale_log2 - m_sub) : 0.f;
          l_sum += pv[i];
        }
        uint8_t* base = sP + (c >> 1) * kHalfBytes + (r >> 3) * 1024 + (r & 7) * 128;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int ch = (c & 1) * 4 + i;
          uint4 o4;
          o4.x = pack_bf16x2(pv[i * 8 + 0], pv[i * 8 + 1]);
          o4.y = pack_bf16x2(pv[i * 8 + 2], pv[i * 8 + 3]);
          o4.z = pack_bf16x2(pv[i * 8 + 4], pv[i * 8 + 5]);
          o4.w = pack_bf16x2(pv[i * 8 + 6], pv[i * 8 + 7]);
          *reinterpret_cast<uint4*>(base + ((ch ^ (r & 7)) * 16)) = o4;
        }
      }
      // S buffer may be overwritten; P is ready for the tensor core
      tc_fence_before_sync();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&s_empty[b]);
        mbar_arrive(p_full);
      }
    }
    // ---- epilogue: O / l -> bf16 rows ----
    if (ok && n_tiles > 0) {
      if (!mbar_wait(pv_done, (n_tiles - 1) & 1)) ok = false;
      ok = __all_sync(0xffffffffu, ok);
    }
    if (!ok && lane == 0) set_status_once(status, kStatusMbarTimeoutEpilogue);
    if (ok && n_tiles > 0) {
      tc_fence_after_sync();
      const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
      __nv_bfloat16* orow = p.out + static_cast<long long>(row_base + qi) * p.out_stride + head * D;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_o + lane_sel + c * 32, v);
        tmem_ld_wait();
        if (row_valid) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 o4;
            o4.x = pack_bf16x2(__uint_as_float(v[i]) * inv, __uint_as_float(v[i + 1]) * inv);
            o4.y = pack_bf16x2(__uint_as_float(v[i + 2]) * inv, __uint_as_float(v[i + 3]) * inv);
            o4.z = pack_bf16x2(__uint_as_float(v[i + 4]) * inv, __uint_as_float(v[i + 5]) * inv);
            o4.w = pack_bf16x2(__uint_as_float(v[i + 6]) * inv, __uint_as_float(v[i + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 32 + i) = o4;
          }
        }
      }
    }
    tc_fence_before_sync();
  }

  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int D>
void launch_tc(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV,
               const PrefillAttnParams& p, int n_tiles, int* status, cudaStream_t stream) {
  using L = Smem<D>;
  auto kern = prefill_tc_kernel<D>;
  ensure_dynamic_smem(kern, L::kTotal);
  dim3 grid(n_tiles, p.Hq);
  kern<<<grid, kThreads, L::kTotal, stream>>>(tmQ, tmK, tmV, p, status);
}

}  // namespace

void launch_paged_prefill_tc(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV,
                             const PrefillAttnParams& p, int n_tiles, int head_dim, int* status,
                             cudaStream_t stream) {
  if (n_tiles <= 0) return;
  if (head_dim == 128)
    launch_tc<128>(tmQ, tmK, tmV, p, n_tiles, status, stream);
  else
    launch_tc<64>(tmQ, tmK, tmV, p, n_tiles, status, stream);
}

}  // namespace oxb
