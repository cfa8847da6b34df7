// tcgen05 bf16 GEMM for sm_100a:  C[g][M,N] (+)= A[g][M,K] * B[g][N,K]^T, fp32 accumulation in TMEM.
//
// One CTA computes one 128 x BN output tile over a slice of K (grid.z = split-K).
// Warp roles: warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer, warps 2..5 =
// epilogue (one TMEM lane quarter each). Operands are staged by TMA into a ring of
// 128B-swizzled shared-memory tiles; completion is tracked by mbarriers, and every
// wait is bounded (a spin that runs out writes a status code and unwinds).
//
// Fused collectives, all issued by this kernel over NVLink peer mappings:
//  * kEpiRedF32 routes each output row to the fp32 accumulator of the rank that owns it
//    (`red.global.add.v4.f32` into local or peer memory). With one owner this is split-K; with
//    tp owners it is the reduce-scatter of a row-parallel projection; with a RowMeta table it is
//    the MoE combine (weighted scatter-add of expert outputs back to the token's home rank).
//    The last CTA to finish (ticket) bumps an arrival counter on every owner with a
//    system-scope release, so the consumer kernel on each owner needs one bounded wait.
//  * The A operand may be an all-gather / dispatch buffer that peers fill: the producer waits
//    (bounded) on per-source counters before its first A load, weights are prefetched first.
//  * Grouped mode walks a device-side table of per-expert row counts, so the grid is static
//    (CUDA-graph friendly) while the work is data dependent.
//
// Replaces the reference's cuBLAS prefill path (cublas_ops.cu:242-260), the `*_fused_add`
// output projections (launch_wrappers.cu:202-247) and the host-loop grouped expert GEMM
// (oxide-engine/src/moe_gemm.rs:208-345); the reference's all-reduce
// (oxide-backend-cuda/src/nccl.rs:18-29) is a no-op.
#include "gemm_bf16.cuh"

#include "../common/sm100.cuh"

namespace oxb {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = 128 bytes = one swizzle atom row
constexpr int kThreads = 192;

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_add_v4_f32(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c),
               "f"(d)
               : "memory");
}
__device__ __forceinline__ float act_fn(float x, int act) {
  if (act == 0) return x / (1.f + __expf(-x));
  return 0.5f * x * (1.f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
}

// Waits until the source counters [s_lo, s_hi] reach the expected value, then lets the last
// CTA of the grid re-arm them. Returns false when the budget ran out.
__device__ bool wait_sources(const GemmParams& p, int s_lo, int s_hi) {
  bool ok = true;
  for (int s = s_lo; s <= s_hi && ok; ++s) {
    uint32_t it = 0;
    while (ld_acquire_sys(p.ag_flags + s) < p.ag_expected) {
      if (++it > OXB_SPIN_LIMIT) {
        atomicExch(p.status, kStatusPeerFlagTimeout);
        ok = false;
        break;
      }
    }
  }
  // Peer stores went through the generic proxy; TMA reads through the async proxy.
  asm volatile("fence.proxy.async;" ::: "memory");
  const uint32_t total = gridDim.x * gridDim.y * gridDim.z;
  const uint32_t old = atomicAdd(p.ag_ticket, 1u);
  if (old == total - 1) {
    for (int s = 0; s < p.ag_n_src; ++s) const_cast<uint32_t*>(p.ag_flags)[s] = 0;
    __threadfence();
    *p.ag_ticket = 0;
  }
  return ok;
}

template <int BN, int STAGES>
struct SmemLayout {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kBarOffset = STAGES * (kABytes + kBBytes);
  static constexpr int kTotal = kBarOffset + 256 + 1024;  // + barriers + alignment slack
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const GemmParams p) {
  using L = SmemLayout<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem =
      reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * L::kABytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* empty = full + STAGES;
  uint64_t* tmem_full = empty + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_full + 1);
  int* s_info = reinterpret_cast<int*>(tmem_slot + 1);  // [0]=group [1]=m tile [2]=rows [3]=active

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BN;
  const int total_kb = (p.K + BK - 1) / BK;
  const int kb0 = blockIdx.z * p.kb_per_split;
  int nkb = total_kb - kb0;
  if (nkb > p.kb_per_split) nkb = p.kb_per_split;
  const bool grouped = p.group_counts != nullptr;
  // Each CTA walks its k-blocks from a different starting point: the CTAs of one wave would
  // otherwise all ask L2 for the same activation tile at the same moment.
  const int k_rot = (p.k_stagger && nkb > 1) ? static_cast<int>((blockIdx.x * 5u + blockIdx.y * 3u) % static_cast<unsigned>(nkb)) : 0;

  constexpr uint32_t kTmemCols = BN < 32 ? 32 : BN;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(tmem_full, 1);
    fence_mbar_init();
    int group = 0, mtile = blockIdx.y, rows = p.M, active = 1;
    if (grouped) {
      // The per-group row counts are final only once every source has finished dispatching.
      if (p.ag_flags != nullptr) active = wait_sources(p, 0, p.ag_n_src - 1) ? 1 : 0;
      int t = blockIdx.y;
      group = -1;
      for (int e = 0; e < p.n_groups; ++e) {
        const int cnt = static_cast<int>(__ldcg(p.group_counts + e));
        const int tiles = (cnt + BM - 1) / BM;
        if (t < tiles) {
          group = e;
          rows = cnt;
          break;
        }
        t -= tiles;
      }
      mtile = t;
      if (group < 0) active = 0;
    }
    if (nkb <= 0) active = 0;
    s_info[0] = group;
    s_info[1] = mtile;
    s_info[2] = rows;
    s_info[3] = active;
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const int group = s_info[0];
  const int m0 = s_info[1] * BM;
  const int rows = s_info[2];
  const bool active = s_info[3] != 0;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0 && active) {
      const int pre = nkb < STAGES ? nkb : STAGES;
      // Weights do not depend on any peer: start them before waiting for the gathered rows.
      for (int kb = 0; kb < pre; ++kb) {
        mbar_arrive_expect_tx(&full[kb], L::kABytes + L::kBBytes);
        tma_load_3d(sB + kb * L::kBBytes, &tmB, &full[kb], (kb0 + (kb + k_rot) % nkb) * BK, n0, group);
      }
      bool ok = true;
      if (p.ag_flags != nullptr && !grouped) {
        int s_lo = 0, s_hi = p.ag_n_src - 1;  // rows_per_src <= 0: rows are not grouped by source
        if (p.ag_rows_per_src > 0) {
          const int m_end = m0 + BM < rows ? m0 + BM : rows;
          s_lo = m0 / p.ag_rows_per_src;
          s_hi = (m_end - 1) / p.ag_rows_per_src;
          if (s_hi >= p.ag_n_src) s_hi = p.ag_n_src - 1;
          if (s_lo > s_hi) s_lo = s_hi;
        }
        ok = wait_sources(p, s_lo, s_hi);
      }
      for (int kb = 0; kb < nkb && ok; ++kb) {
        const int s = kb % STAGES;
        if (kb >= pre) {
          const uint32_t ph = (kb / STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1)) {
            atomicExch(p.status, kStatusMbarTimeoutProducer);
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&full[s], L::kABytes + L::kBBytes);
          tma_load_3d(sB + s * L::kBBytes, &tmB, &full[s], (kb0 + (kb + k_rot) % nkb) * BK, n0, group);
        }
        tma_load_3d(sA + s * L::kABytes, &tmA, &full[s], (kb0 + (kb + k_rot) % nkb) * BK, m0, group);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0 && active) {
      constexpr uint32_t idesc = make_idesc(kFmtBF16, kFmtBF16, BM, BN);
      bool ok = true;
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % STAGES;
        const uint32_t ph = (kb / STAGES) & 1;
        if (!mbar_wait(&full[s], ph)) {
          atomicExch(p.status, kStatusMbarTimeoutMma);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t a_addr = smem_u32(sA + s * L::kABytes);
        const uint32_t b_addr = smem_u32(sB + s * L::kBBytes);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k) {
          tc_mma_f16(tmem_base, make_desc_kmajor_sw128(a_addr + k * 32),
                     make_desc_kmajor_sw128(b_addr + k * 32), idesc, (kb | k) != 0 ? 1u : 0u);
        }
        tc_commit(&empty[s]);  // frees this smem stage once the MMAs above have read it
      }
      if (ok) tc_commit(tmem_full);
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const int row = m0 + q * 32 + lane;
    bool ok = active;
    if (ok && !mbar_wait(tmem_full, 0)) {
      if (lane == 0) atomicExch(p.status, kStatusMbarTimeoutEpilogue);
      ok = false;
    }
    ok = __all_sync(0xffffffffu, ok);  // tcgen05.ld below is warp-collective
    tc_fence_after_sync();
    if (ok) {
      const bool row_ok = row < rows;
      const bool vec_ok = (p.N & 7) == 0;
      const __nv_bfloat16* bias = p.bias != nullptr ? p.bias + static_cast<long long>(group) * p.N
                                                    : nullptr;
      const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);

      if (p.epi == kEpiRedF32) {
        int owner = 0, row_local = row;
        float wgt = 1.f;
        if (p.row_meta != nullptr) {
          if (row_ok) {
            const RowMeta m = p.row_meta[static_cast<long long>(group) * p.meta_group_stride + row];
            owner = m.rank;
            row_local = m.row;
            wgt = m.weight;
          }
        } else {
          owner = row / p.rows_per_owner;
          if (owner >= p.n_owners) owner = p.n_owners - 1;
          row_local = row - owner * p.rows_per_owner;
        }
        float* red_base = nullptr;
        // avoid a dynamically indexed parameter array (it would be copied to local memory)
#pragma unroll
        for (int o = 0; o < kMaxRanks; ++o)
          if (o == owner) red_base = p.dst[o];
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(lane_addr + c * 32, r);
          tmem_ld_wait();
          const int col0 = n0 + c * 32;
          if (!row_ok || col0 >= p.N || red_base == nullptr) continue;
          float* d = red_base + static_cast<long long>(row_local) * p.dst_ld + col0;
          if (vec_ok && col0 + 32 <= p.N) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              red_add_v4_f32(d + j, wgt * __uint_as_float(r[j]), wgt * __uint_as_float(r[j + 1]),
                             wgt * __uint_as_float(r[j + 2]), wgt * __uint_as_float(r[j + 3]));
          } else {
            for (int j = 0; j < 32 && col0 + j < p.N; ++j)
              atomicAdd(d + j, wgt * __uint_as_float(r[j]));
          }
        }
      } else if (p.epi == kEpiStoreF32) {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(lane_addr + c * 32, r);
          tmem_ld_wait();
          const int col0 = n0 + c * 32;
          if (!row_ok || col0 >= p.N) continue;
          float* d = reinterpret_cast<float*>(p.C) + static_cast<long long>(group) * p.c_group_stride +
                     static_cast<long long>(row) * p.ldc + col0;
          if ((p.ldc & 3) == 0 && vec_ok && col0 + 32 <= p.N) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              float4 o4;
              o4.x = __uint_as_float(r[j]);
              o4.y = __uint_as_float(r[j + 1]);
              o4.z = __uint_as_float(r[j + 2]);
              o4.w = __uint_as_float(r[j + 3]);
              if (bias) {
                o4.x += __bfloat162float(bias[col0 + j]);
                o4.y += __bfloat162float(bias[col0 + j + 1]);
                o4.z += __bfloat162float(bias[col0 + j + 2]);
                o4.w += __bfloat162float(bias[col0 + j + 3]);
              }
              *reinterpret_cast<float4*>(d + j) = o4;
            }
          } else {
            for (int j = 0; j < 32 && col0 + j < p.N; ++j) {
              float v = __uint_as_float(r[j]);
              if (bias) v += __bfloat162float(bias[col0 + j]);
              d[j] = v;
            }
          }
        }
      } else {
        // ---- bf16 outputs (plain store, SwiGLU, routed slab store): TMEM -> registers -> a
        // padded shared-memory tile (the operand ring is free once tmem_full has fired) ->
        // row-contiguous 16-byte stores, so local HBM and NVLink both see full lines. Each
        // warp stages and writes only its own 32 rows, a __syncwarp is all it needs.
        const bool swiglu = p.epi == kEpiSwigluBf16;
        constexpr int kOutColsMax = BN;
        constexpr int kPitch = kOutColsMax * 2 + 16;  // bytes; 16-byte skew keeps stores conflict-free
        uint8_t* stage = smem + static_cast<size_t>(q) * 32 * kPitch;
        uint8_t* my_row = stage + static_cast<size_t>(lane) * kPitch;
        const int out_cols = swiglu ? BN / 2 : BN;  // columns of this tile in the output
        if (swiglu) {
#pragma unroll 1
          for (int c = 0; c < BN / 64; ++c) {
            uint32_t gt[32], up[32];
            tmem_ld_32x32b_x32(lane_addr + c * 64, gt);
            tmem_ld_32x32b_x32(lane_addr + c * 64 + 32, up);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              float v[8];
#pragma unroll
              for (int t = 0; t < 8; ++t)
                v[t] = act_fn(__uint_as_float(gt[j + t]), p.act) * __uint_as_float(up[j + t]);
              uint4 o4;
              o4.x = pack_bf16x2(v[0], v[1]);
              o4.y = pack_bf16x2(v[2], v[3]);
              o4.z = pack_bf16x2(v[4], v[5]);
              o4.w = pack_bf16x2(v[6], v[7]);
              *reinterpret_cast<uint4*>(my_row + (c * 32 + j) * 2) = o4;
            }
          }
        } else {
#pragma unroll 1
          for (int c = 0; c < BN / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(lane_addr + c * 32, r);
            tmem_ld_wait();
            const int col0 = n0 + c * 32;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              float v[8];
#pragma unroll
              for (int t = 0; t < 8; ++t) {
                v[t] = __uint_as_float(r[j + t]);
                if (bias != nullptr && col0 + j + t < p.N) v[t] += __bfloat162float(bias[col0 + j + t]);
              }
              uint4 o4;
              o4.x = pack_bf16x2(v[0], v[1]);
              o4.y = pack_bf16x2(v[2], v[3]);
              o4.z = pack_bf16x2(v[4], v[5]);
              o4.w = pack_bf16x2(v[6], v[7]);
              *reinterpret_cast<uint4*>(my_row + (c * 32 + j) * 2) = o4;
            }
          }
        }
        __syncwarp();
        // copy-out: lanes sweep the row's 16-byte chunks; several rows per instruction
        const int n_total = swiglu ? (p.N >> 1) : p.N;       // output row length
        const int oc0 = swiglu ? (n0 >> 1) : n0;             // first output column of this tile
        const int chunks = out_cols / 8;                     // 16-byte chunks per staged row
        const int rows_per_it = 32 / chunks > 0 ? 32 / chunks : 1;
        const bool out_vec = (n_total & 7) == 0;
        for (int r0 = 0; r0 < 32; r0 += rows_per_it) {
          for (int ch0 = 0; ch0 < chunks; ch0 += 32) {
            const int rr = r0 + (chunks >= 32 ? 0 : lane / chunks);
            const int ch = chunks >= 32 ? ch0 + lane : lane % chunks;
            const int grow = m0 + q * 32 + rr;
            const int gcol = oc0 + ch * 8;
            if (rr >= 32 || ch >= chunks || grow >= rows || gcol >= n_total) continue;
            __nv_bfloat16* drow;
            if (p.epi == kEpiSlabBf16) {
              int owner = grow / p.rows_per_owner;
              if (owner >= p.n_owners) owner = p.n_owners - 1;
              const int row_local = grow - owner * p.rows_per_owner;
              __nv_bfloat16* base = nullptr;
#pragma unroll
              for (int o = 0; o < kMaxRanks; ++o)
                if (o == owner) base = reinterpret_cast<__nv_bfloat16*>(p.dst[o]);
              drow = base + (static_cast<long long>(p.my_rank) * p.rows_per_owner + row_local) * p.dst_ld;
            } else {
              drow = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(group) * p.c_group_stride +
                     static_cast<long long>(grow) * p.ldc;
            }
            const uint8_t* src = stage + static_cast<size_t>(rr) * kPitch + ch * 16;
            if (out_vec && gcol + 8 <= n_total && ((p.epi == kEpiSlabBf16 ? p.dst_ld : p.ldc) & 7) == 0) {
              *reinterpret_cast<uint4*>(drow + gcol) = *reinterpret_cast<const uint4*>(src);
            } else {
              const __nv_bfloat16* sv = reinterpret_cast<const __nv_bfloat16*>(src);
              for (int t = 0; t < 8 && gcol + t < n_total; ++t) drow[gcol + t] = sv[t];
            }
          }
        }
      }
    }
    tc_fence_before_sync();
    // When the whole grid has landed its contributions, tell every owner once.
    if (p.done_ticket != nullptr) {
      __threadfence_system();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (warp == 2 && lane == 0) {
        const uint32_t total = gridDim.x * gridDim.y * gridDim.z;
        const uint32_t old = atomicAdd(p.done_ticket, 1u);
        if (old == total - 1) {
          for (int i = 0; i < p.n_reset; ++i) p.reset_on_done[i] = 0;
          *p.done_ticket = 0;
          __threadfence_system();
#pragma unroll
          for (int o = 0; o < kMaxRanks; ++o)
            if (o < p.n_owners && p.arrive[o] != nullptr) red_release_sys_add(p.arrive[o], 1u);
        }
      }
    }
  }

  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int BN, int STAGES>
void launch_impl(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int m_tiles,
                 int splits, cudaStream_t stream) {
  using L = SmemLayout<BN, STAGES>;
  static bool configured = false;
  auto kern = gemm_bf16_kernel<BN, STAGES>;
  if (!configured) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal);
    configured = true;
  }
  dim3 grid((p.N + BN - 1) / BN, m_tiles, splits);
  kern<<<grid, kThreads, L::kTotal, stream>>>(tmA, tmB, p);
}

}  // namespace

void launch_gemm_bf16(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int bn,
                      int m_tiles, int splits, cudaStream_t stream) {
  switch (bn) {
    case 64:
      launch_impl<64, 8>(tmA, tmB, p, m_tiles, splits, stream);
      break;
    case 256:
      launch_impl<256, 4>(tmA, tmB, p, m_tiles, splits, stream);
      break;
    default:
      launch_impl<128, 6>(tmA, tmB, p, m_tiles, splits, stream);
      break;
  }
}

}  // namespace oxb
