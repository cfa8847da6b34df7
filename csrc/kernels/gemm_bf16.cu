// tcgen05 bf16 GEMM for sm_100a:  C[g][M,N] (+)= A[g][M,K] * B[g][N,K]^T, fp32 accumulation in TMEM.
//
// Persistent kernel, one CTA per SM. A work item is one 128 x BN output tile over a slice of K
// (split-K); CTA c takes items c, c + grid, c + 2 grid, ... Warp roles: warp 0 = TMA producer,
// warp 1 = TMEM owner + MMA issuer, warps 2..5 = epilogue (one TMEM lane quarter each). Operands
// are staged by TMA into a ring of 128B-swizzled shared-memory tiles; the accumulator is double
// buffered in TMEM (2 x BN columns), so the epilogue of item i drains one buffer while the MMAs
// of item i+1 fill the other. Completion is tracked by mbarriers and every wait is bounded (a
// spin that runs out writes a status code and unwinds).
//
// Fused collectives, all issued by this kernel over NVLink peer mappings:
//  * kEpiRedF32 routes each output row to the fp32 accumulator of the rank that owns it
//    (`red.global.add.v4.f32` into local or peer memory). With one owner this is split-K; with
//    tp owners it is the reduce-scatter of a row-parallel projection; with a RowMeta table it is
//    the MoE combine (weighted scatter-add of expert outputs back to the token's home rank).
//  * kEpiSlabBf16 stores bf16 partial tiles row-contiguously into the row owner's receive slab
//    (half the NVLink bytes of fp32, full-line packets); the owner's finalize kernel sums them.
//    In both cases the last CTA to finish (ticket) bumps an arrival counter on every owner with
//    one system-scope fence and relaxed signals, so the consumer kernel on each owner needs one bounded wait.
//  * The A operand may be an all-gather / dispatch buffer that peers fill: the producer waits
//    (bounded) on per-source counters before its first A load of a tile; weight tiles are
//    requested before that wait.
//  * Dense weights may be stored tile-major ([N/128][K/64][128][64]) so that each TMA box of the
//    weight stream is one contiguous 16 KB run of HBM instead of 128 row segments 2K bytes apart.
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
constexpr int kStageCols = 64;                    // output columns staged per copy-out round
constexpr int kStagePitch = kStageCols * 2 + 16;  // bytes; 16-byte skew keeps smem stores conflict-free
constexpr int kStageBytes = 128 * kStagePitch;

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Relaxed on purpose: the caller issues ONE system-scope fence and then signals every peer; a
// release on each signal would wait a full NVLink round trip per peer, one after the other.
__device__ __forceinline__ void red_relaxed_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
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

// Waits until the source counters [s_lo, s_hi] reach the expected value; `waiters` is the number
// of such waits the whole grid performs, the last of them re-arms the counters.
__device__ bool wait_sources(const GemmParams& p, int s_lo, int s_hi, uint32_t waiters) {
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
  const uint32_t old = atomicAdd(p.ag_ticket, 1u);
  if (old == waiters - 1) {
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
  static constexpr int kStageOffset = STAGES * (kABytes + kBBytes);
  static constexpr int kBarOffset = kStageOffset + kStageBytes;
  static constexpr int kTotal = kBarOffset + 512 + 1024;  // + barriers/scratch + alignment slack
};

struct WorkItem {
  int group, m0, rows, n0, kb0, nkb;
  bool valid;
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
  uint8_t* sStage = smem + L::kStageOffset;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* empty = full + STAGES;
  uint64_t* tmem_full = empty + STAGES;  // [2]
  uint64_t* tmem_empty = tmem_full + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  int* s_counts = reinterpret_cast<int*>(tmem_slot + 2);  // [0] ok flag, [1..] first m tile per group

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int total_kb = (p.K + BK - 1) / BK;
  const bool grouped = p.group_counts != nullptr;
  const int n_tiles = (p.N + BN - 1) / BN;
  const int m_tiles = p.m_tiles;
  const int n_work = n_tiles * m_tiles * p.splits;

  constexpr uint32_t kAccCols = BN < 32 ? 32 : BN;
  constexpr uint32_t kTmemCols = 2 * kAccCols;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(&tmem_full[0], 1);
    mbar_init(&tmem_full[1], 1);
    mbar_init(&tmem_empty[0], 4);
    mbar_init(&tmem_empty[1], 4);
    fence_mbar_init();
    int ok = 1;
    if (grouped) {
      // The per-group row counts are final only once every source has finished dispatching.
      if (p.ag_flags != nullptr) ok = wait_sources(p, 0, p.ag_n_src - 1, gridDim.x) ? 1 : 0;
      int acc = 0;
      for (int e = 0; e < p.n_groups; ++e) {
        s_counts[1 + e] = acc;  // first m tile of group e
        acc += (static_cast<int>(__ldcg(p.group_counts + e)) + BM - 1) / BM;
      }
      s_counts[1 + p.n_groups] = acc;
    }
    s_counts[0] = ok;
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const bool all_ok = s_counts[0] != 0;

  // work item w -> tile coordinates; consecutive items share the weight tile (m fastest)
  auto decode = [&](int w) -> WorkItem {
    WorkItem it;
    const int mt = w % m_tiles;
    const int rest = w / m_tiles;
    const int nt = rest % n_tiles;
    const int z = rest / n_tiles;
    it.n0 = nt * BN;
    it.kb0 = z * p.kb_per_split;
    it.nkb = total_kb - it.kb0;
    if (it.nkb > p.kb_per_split) it.nkb = p.kb_per_split;
    it.group = 0;
    it.m0 = mt * BM;
    it.rows = p.M;
    it.valid = all_ok && it.nkb > 0;
    if (grouped) {
      it.valid = false;
      for (int e = 0; e < p.n_groups; ++e) {
        if (mt >= s_counts[1 + e] && mt < s_counts[2 + e]) {
          it.group = e;
          it.m0 = (mt - s_counts[1 + e]) * BM;
          it.rows = static_cast<int>(__ldcg(p.group_counts + e));
          it.valid = all_ok && it.nkb > 0;
          break;
        }
      }
    }
    return it;
  };

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      uint32_t iter = 0;  // k-block counter across all items of this CTA
      bool ok = true;
      for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x) {
        const WorkItem it = decode(w);
        bool need_wait = p.ag_flags != nullptr && !grouped;
        if (!it.valid) {
          // keep the waiter count of the grid exact: an empty item still passes the gate
          if (need_wait) wait_sources(p, 0, -1, static_cast<uint32_t>(n_work));
          continue;
        }
        for (int kb = 0; kb < it.nkb && ok; ++kb, ++iter) {
          const int s = iter % STAGES;
          const uint32_t ph = (iter / STAGES) & 1;
          if (iter >= STAGES && !mbar_wait(&empty[s], ph ^ 1)) {
            atomicExch(p.status, kStatusMbarTimeoutProducer);
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&full[s], L::kABytes + L::kBBytes);
          // weights first: they do not depend on any peer
          if (p.b_tiled) {
            // tile-major weights: tile index = (n / 128) * total_kb + kb, box = 128 x 64 (or the
            // 64-row half of a tile for BN = 64)
            constexpr int kRowsPerLoad = BN < 128 ? BN : 128;
#pragma unroll
            for (int j = 0; j < (BN + 127) / 128; ++j)
              tma_load_3d(sB + s * L::kBBytes + j * 16384, &tmB, &full[s], 0, BN < 128 ? (it.n0 & 127) : 0,
                          ((it.n0 >> 7) + j) * total_kb + it.kb0 + kb);
            (void)kRowsPerLoad;
          } else {
            tma_load_3d(sB + s * L::kBBytes, &tmB, &full[s], (it.kb0 + kb) * BK, it.n0, it.group);
          }
          if (need_wait) {
            int s_lo = 0, s_hi = p.ag_n_src - 1;  // rows_per_src <= 0: rows are not grouped by source
            if (p.ag_rows_per_src > 0) {
              const int m_end = it.m0 + BM < it.rows ? it.m0 + BM : it.rows;
              s_lo = it.m0 / p.ag_rows_per_src;
              s_hi = (m_end - 1) / p.ag_rows_per_src;
              if (s_hi >= p.ag_n_src) s_hi = p.ag_n_src - 1;
              if (s_lo > s_hi) s_lo = s_hi;
            }
            ok = wait_sources(p, s_lo, s_hi, static_cast<uint32_t>(n_work));
            need_wait = false;
            if (!ok) break;
          }
          tma_load_3d(sA + s * L::kABytes, &tmA, &full[s], (it.kb0 + kb) * BK, it.m0, it.group);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(kFmtBF16, kFmtBF16, BM, BN);
      uint32_t iter = 0, t = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x) {
        const WorkItem it = decode(w);
        if (!it.valid) continue;
        const uint32_t buf = t & 1;
        // the epilogue must have drained this accumulator buffer (two items ago)
        if (t >= 2 && !mbar_wait(&tmem_empty[buf], ((t >> 1) & 1) ^ 1)) {
          atomicExch(p.status, kStatusMbarTimeoutMma);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * kAccCols;
        for (int kb = 0; kb < it.nkb; ++kb, ++iter) {
          const int s = iter % STAGES;
          const uint32_t ph = (iter / STAGES) & 1;
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
            tc_mma_f16(d_tmem, make_desc_kmajor_sw128(a_addr + k * 32),
                       make_desc_kmajor_sw128(b_addr + k * 32), idesc, (kb | k) != 0 ? 1u : 0u);
          }
          tc_commit(&empty[s]);  // frees this smem stage once the MMAs above have read it
        }
        if (ok) tc_commit(&tmem_full[buf]);
        ++t;
      }
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    if (p.prefetch_bytes > 0 && warp == 5) {
      // this CTA's slice of the range, in 4 KB requests spread over the lanes
      constexpr long long kChunk = 4096;
      const long long n_chunks = (p.prefetch_bytes + kChunk - 1) / kChunk;
      const char* base = static_cast<const char*>(p.prefetch_ptr);
      for (long long c = static_cast<long long>(blockIdx.x) * 32 + lane; c < n_chunks;
           c += static_cast<long long>(gridDim.x) * 32) {
        const long long off = c * kChunk;
        const long long left = p.prefetch_bytes - off;
        const uint32_t sz = static_cast<uint32_t>(left < kChunk ? left : kChunk);
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(base + off), "r"(sz) : "memory");
      }
    }
    uint8_t* stage = sStage + static_cast<size_t>(q) * 32 * kStagePitch;
    uint8_t* my_row = stage + static_cast<size_t>(lane) * kStagePitch;
    const bool vec_ok = (p.N & 7) == 0;
    uint32_t t = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < n_work; w += gridDim.x) {
      const WorkItem it = decode(w);
      if (!it.valid) continue;
      const uint32_t buf = t & 1;
      if (ok && !mbar_wait(&tmem_full[buf], (t >> 1) & 1)) {
        if (lane == 0) atomicExch(p.status, kStatusMbarTimeoutEpilogue);
        ok = false;
      }
      ok = __all_sync(0xffffffffu, ok);  // tcgen05.ld below is warp-collective
      if (!ok) break;
      tc_fence_after_sync();
      const int row = it.m0 + q * 32 + lane;
      const bool row_ok = row < it.rows;
      const int n0 = it.n0;
      const int group = it.group;
      const __nv_bfloat16* bias =
          p.bias != nullptr ? p.bias + static_cast<long long>(group) * p.N : nullptr;
      const uint32_t lane_addr = tmem_base + buf * kAccCols + (static_cast<uint32_t>(q * 32) << 16);

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
        // padded shared-memory tile -> row-contiguous 16-byte stores, 64 output columns per
        // round, so local HBM and NVLink both see full lines. Each warp stages and writes only
        // its own 32 rows; __syncwarp is all it needs.
        const bool swiglu = p.epi == kEpiSwigluBf16;
        const int n_total = swiglu ? (p.N >> 1) : p.N;  // output row length
        const int oc0 = swiglu ? (n0 >> 1) : n0;        // first output column of this tile
        const int out_cols = swiglu ? BN / 2 : BN;
        const bool out_vec =
            (n_total & 7) == 0 && (((p.epi == kEpiSlabBf16) ? p.dst_ld : p.ldc) & 7) == 0;
#pragma unroll 1
        for (int oc = 0; oc < out_cols; oc += kStageCols) {
          const int width = out_cols - oc < kStageCols ? out_cols - oc : kStageCols;  // 32 or 64
#pragma unroll 1
          for (int h = 0; h < width; h += 32) {
            float v[32];
            if (swiglu) {
              uint32_t gt[32], up[32];
              const int c = (oc + h) / 32;  // 32 outputs come from accumulator columns [64c, 64c+64)
              tmem_ld_32x32b_x32(lane_addr + c * 64, gt);
              tmem_ld_32x32b_x32(lane_addr + c * 64 + 32, up);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 32; ++j)
                v[j] = act_fn(__uint_as_float(gt[j]), p.act) * __uint_as_float(up[j]);
            } else {
              uint32_t r[32];
              tmem_ld_32x32b_x32(lane_addr + oc + h, r);
              tmem_ld_wait();
              const int col0 = n0 + oc + h;
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                v[j] = __uint_as_float(r[j]);
                if (bias != nullptr && col0 + j < p.N) v[j] += __bfloat162float(bias[col0 + j]);
              }
            }
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint4 o4;
              o4.x = pack_bf16x2(v[j], v[j + 1]);
              o4.y = pack_bf16x2(v[j + 2], v[j + 3]);
              o4.z = pack_bf16x2(v[j + 4], v[j + 5]);
              o4.w = pack_bf16x2(v[j + 6], v[j + 7]);
              *reinterpret_cast<uint4*>(my_row + (h + j) * 2) = o4;
            }
          }
          __syncwarp();
          const int chunks = width / 8;  // 16-byte chunks per staged row: 4 or 8
          const int rows_per_it = 32 / chunks;
          for (int r0 = 0; r0 < 32; r0 += rows_per_it) {
            const int rr = r0 + lane / chunks;
            const int ch = lane % chunks;
            const int grow = it.m0 + q * 32 + rr;
            const int gcol = oc0 + oc + ch * 8;
            if (grow >= it.rows || gcol >= n_total) continue;
            __nv_bfloat16* drow;
            if (p.epi == kEpiSlabBf16) {
              int owner = grow / p.rows_per_owner;
              if (owner >= p.n_owners) owner = p.n_owners - 1;
              const int row_local = grow - owner * p.rows_per_owner;
              __nv_bfloat16* base = nullptr;
#pragma unroll
              for (int o = 0; o < kMaxRanks; ++o)
                if (o == owner) base = reinterpret_cast<__nv_bfloat16*>(p.dst[o]);
              drow = base +
                     (static_cast<long long>(p.my_rank) * p.rows_per_owner + row_local) * p.dst_ld;
            } else {
              drow = reinterpret_cast<__nv_bfloat16*>(p.C) +
                     static_cast<long long>(group) * p.c_group_stride +
                     static_cast<long long>(grow) * p.ldc;
            }
            const uint8_t* src = stage + static_cast<size_t>(rr) * kStagePitch + ch * 16;
            if (out_vec && gcol + 8 <= n_total) {
              *reinterpret_cast<uint4*>(drow + gcol) = *reinterpret_cast<const uint4*>(src);
            } else {
              const __nv_bfloat16* sv = reinterpret_cast<const __nv_bfloat16*>(src);
              for (int e = 0; e < 8 && gcol + e < n_total; ++e) drow[gcol + e] = sv[e];
            }
          }
          __syncwarp();
        }
      }
      // hand the accumulator buffer back to the MMA warp
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[buf]);
      ++t;
    }
    tc_fence_before_sync();
    // When the whole grid has landed its contributions, tell every owner once.
    if (p.done_ticket != nullptr) {
      // One system-scope fence per CTA: the barrier orders the other epilogue threads' stores
      // before it (cumulativity), and a fence per thread would serialise 128 of them.
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (warp == 2 && lane == 0) {
        __threadfence_system();
        const uint32_t old = atomicAdd(p.done_ticket, 1u);
        if (old == gridDim.x - 1) {
          for (int i = 0; i < p.n_reset; ++i) p.reset_on_done[i] = 0;
          *p.done_ticket = 0;
          __threadfence_system();
#pragma unroll
          for (int o = 0; o < kMaxRanks; ++o)
            if (o < p.n_owners && p.arrive[o] != nullptr) red_relaxed_sys_add(p.arrive[o], 1u);
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
void launch_impl(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p,
                 cudaStream_t stream) {
  using L = SmemLayout<BN, STAGES>;
  static bool configured = false;
  static int sm_count = 148;
  auto kern = gemm_bf16_kernel<BN, STAGES>;
  if (!configured) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal);
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    configured = true;
  }
  const int n_work = ((p.N + BN - 1) / BN) * p.m_tiles * p.splits;
  const int grid = n_work < sm_count ? n_work : sm_count;
  kern<<<grid, kThreads, L::kTotal, stream>>>(tmA, tmB, p);
}

}  // namespace

void launch_gemm_bf16(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int bn,
                      cudaStream_t stream) {
  switch (bn) {
    case 64:
      launch_impl<64, 8>(tmA, tmB, p, stream);
      break;
    case 256:
      launch_impl<256, 4>(tmA, tmB, p, stream);
      break;
    default:
      launch_impl<128, 6>(tmA, tmB, p, stream);
      break;
  }
}

}  // namespace oxb
