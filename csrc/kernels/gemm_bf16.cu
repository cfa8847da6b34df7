// tcgen05 bf16 GEMM for sm_100a:  C[g][M,N] (+)= A[g][M,K] * B[g][N,K]^T, fp32 accumulation in TMEM.
//
// Persistent kernel, one CTA per SM. A work item is one (128 * MT) x BN output tile over a slice
// of K (split-K); CTA c takes items c, c + grid, c + 2 grid, ... Warp roles: warp 0 = TMA
// producer, warp 1 = TMEM owner + MMA issuer, warps 2..5 = epilogue (one TMEM lane quarter each).
// Operands are staged by TMA into a ring of 128B-swizzled shared-memory tiles. With MT = 1 the
// accumulator is double buffered in TMEM (2 x BN columns), so the epilogue of item i drains one
// buffer while the MMAs of item i+1 fill the other. Completion is tracked by mbarriers and every
// wait is bounded (a spin that runs out writes a status code and unwinds).
//
// Decode shapes (M <= 256 rows against a large weight matrix) are bound by how many *distinct*
// weight bytes every SM keeps in flight, not by FLOPs: a CTA that shares its weight tile with a
// neighbour (two 128-row M tiles) streams the same bytes twice through the machine. MT = 2 keeps
// both row halves with the CTA that loads the weight tile (two accumulators fed from one B stage,
// up to 512 TMEM columns), and split-K spreads the tiles over all SMs. Split partial tiles of the
// store / SwiGLU / slab epilogues are combined inside the kernel: every split stores its partial
// as bf16 into its own slab of a workspace, the splits of a tile meet at a ticket, and each of
// them sums a share of the tile's columns over all slabs and runs the epilogue on that share
// (the launch is cooperative, so the CTAs that wait for each other are co-resident).
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
#include "quant_expand.cuh"

#include "../common/device_info.h"
#include "../common/sm100.cuh"

namespace oxb {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = 128 bytes = one swizzle atom row
constexpr int kThreads = 192;
constexpr int kDequantWarps = 4;  // KIND 2 only: warps 6..9
constexpr int kStageCols = 64;                    // output columns staged per copy-out round
constexpr int kStagePitch = kStageCols * 2 + 16;  // bytes; 16-byte skew keeps smem stores conflict-free
constexpr int kStageBytes = 128 * kStagePitch;

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
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
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void stamp(const GemmParams& p, int slot) {
  if (p.trace != nullptr) p.trace[static_cast<size_t>(blockIdx.x) * 8 + slot] = global_ns();
}
// SiLU / tanh-GELU on the special-function unit (approximate reciprocal and tanh: the result is
// rounded to bf16 anyway); a full-precision divide and tanhf cost tens of instructions per value in
// an epilogue that only one warp per scheduler runs.
__device__ __forceinline__ float act_fn(float x, int act) {
  if (act == 0) return __fdividef(x, 1.f + __expf(-x));
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.7978845608028654f * (x + 0.044715f * x * x * x)));
  return 0.5f * x * (1.f + t);
}

// NG groups of 32 accumulator columns of this thread's TMEM lane: all loads are issued before the
// one wait (a load-wait pair costs a few hundred cycles).
template <int NG>
__device__ __forceinline__ void tmem_load_cols(uint32_t taddr, float (&a)[NG * 32]) {
  uint32_t r[NG][32];
#pragma unroll
  for (int g = 0; g < NG; ++g) tmem_ld_32x32b_x32(taddr + g * 32, r[g]);
  tmem_ld_wait();
#pragma unroll
  for (int g = 0; g < NG; ++g)
#pragma unroll
    for (int j = 0; j < 32; ++j) a[g * 32 + j] = __uint_as_float(r[g][j]);
}
// Waits until the source counters [s_lo, s_hi] reach the expected value; `waiters` is the number
// of such waits the whole grid performs, the last of them re-arms the counters.
__device__ bool wait_sources(const GemmParams& p, int s_lo, int s_hi, uint32_t waiters) {
  bool ok = true;
  const uint32_t limit = spin_budget(p.spin_limit);
  for (int s = s_lo; s <= s_hi && ok; ++s) {
    uint32_t it = 0;
    while (ld_acquire_sys(p.ag_flags + s) < p.ag_expected) {
      if (++it > limit) {
        set_status_peer_timeout(p.status);
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

// Untiled bulk copy global -> shared (both 16-byte aligned, size a multiple of 16), completion on `bar`.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(smem_dst)),
      "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
// 64 columns of this thread's row summed over the partial slabs that were landed in shared memory:
// `src` = this thread's 16 bytes in the first 8-column group of the first split, groups are 2 KB
// apart, splits `split_bytes` apart. Consecutive lanes read consecutive 16-byte words.
__device__ __forceinline__ void smem_sum_cols(const uint8_t* src, int splits, uint32_t split_bytes,
                                              float (&a)[64]) {
#pragma unroll
  for (int j = 0; j < 64; ++j) a[j] = 0.f;
#pragma unroll 1
  for (int s = 0; s < splits; ++s, src += split_bytes) {
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      const uint4 x = *reinterpret_cast<const uint4*>(src + g * 2048);
      const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&x);
#pragma unroll
      for (int j = 0; j < 8; ++j) a[g * 8 + j] += __bfloat162float(e[j]);
    }
  }
}

// One 128-row x 64-value weight tile of block type T -> the bf16, 128-byte-swizzled operand stage at
// `stage` (what a TMA box of bf16 weights would have written): four rows per lane, two groups of 32
// weights per row; chunk c (16 bytes) of row r sits at chunk c ^ (r % 8) of that row. The type is a
// template parameter so that the packed-block loads of all eight groups can be issued together.
template <int T>
__device__ __forceinline__ void unpack_kblock(const GemmParams& p, int n0, int kblock, uint8_t* stage, int lane) {
  const int r7 = lane & 7;
  uint32_t wq[4][2][8];
  float dl0[4][2], dl1[4][2], ml[4][2];
#pragma unroll
  for (int rr = 0; rr < 4; ++rr) {
    const int n = n0 + rr * 32 + lane;
    const uint8_t* wrow = p.qw + static_cast<long long>(n < p.N ? n : p.N - 1) * p.q_row_bytes;
    expand_q8_pair<T>(wrow, kblock, wq[rr], dl0[rr], dl1[rr], ml[rr]);
  }
#pragma unroll
  for (int rr = 0; rr < 4; ++rr) {
    const int r = rr * 32 + lane;
    const bool in = n0 + r < p.N;  // rows past N are written as zeros
    uint8_t* dst = stage + r * 128;
#pragma unroll
    for (int g = 0; g < 2; ++g) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float dl = in ? (c < 2 ? dl0[rr][g] : dl1[rr][g]) : 0.f;
        const float m = in ? ml[rr][g] : 0.f;
        // signed byte b of a word -> float: (b ^ 0x80) in the mantissa of 2^23, minus (2^23 + 128)
        const uint32_t w0 = wq[rr][g][2 * c] ^ 0x80808080u, w1 = wq[rr][g][2 * c + 1] ^ 0x80808080u;
        float f[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          f[j] = __uint_as_float(__byte_perm(w0, 0x4B000000u, 0x7650 + j)) - 8388736.f;
          f[4 + j] = __uint_as_float(__byte_perm(w1, 0x4B000000u, 0x7650 + j)) - 8388736.f;
        }
        uint4 o;
        __nv_bfloat162 h;
        h = __floats2bfloat162_rn(fmaf(dl, f[0], m), fmaf(dl, f[1], m));
        o.x = *reinterpret_cast<uint32_t*>(&h);
        h = __floats2bfloat162_rn(fmaf(dl, f[2], m), fmaf(dl, f[3], m));
        o.y = *reinterpret_cast<uint32_t*>(&h);
        h = __floats2bfloat162_rn(fmaf(dl, f[4], m), fmaf(dl, f[5], m));
        o.z = *reinterpret_cast<uint32_t*>(&h);
        h = __floats2bfloat162_rn(fmaf(dl, f[6], m), fmaf(dl, f[7], m));
        o.w = *reinterpret_cast<uint32_t*>(&h);
        *reinterpret_cast<uint4*>(dst + (((g * 4 + c) ^ r7) << 4)) = o;
      }
    }
  }
}

template <int BN, int STAGES, int MT, int KIND = 0>
struct SmemLayout {
  static constexpr int kABytes = MT * BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kRingBytes = STAGES * (kABytes + kBBytes);
  // NVFP4: the scale atoms of one k block (4 x 512 bytes per 128 rows) ride along with each stage
  static constexpr int kSFABytes = KIND == 1 ? MT * 2048 : 0;
  static constexpr int kSFBBytes = KIND == 1 ? ((BN + 127) / 128) * 2048 : 0;
  static constexpr int kSFOffset = kRingBytes;
  static constexpr int kStageOffset = kRingBytes + STAGES * (kSFABytes + kSFBBytes);
  static constexpr int kBarOffset = kStageOffset + kStageBytes;
  static constexpr int kTotal = kBarOffset + 512 + 1024;  // + barriers/scratch + alignment slack
};

struct WorkItem {
  int group, m0, rows, n0, kb0, nkb, tile, z;
  bool valid;
};

// KIND: 0 = bf16 x bf16, 1 = NVFP4 x NVFP4 (block scales in TMEM), 2 = bf16 x GGUF-packed weights
// (four more warps, kDequantWarps, rebuild the weight stage in shared memory).
template <int BN, int STAGES, int MT, int KIND = 0>
__global__ void __launch_bounds__(KIND == 2 ? kThreads + 32 * kDequantWarps : kThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const GemmParams p) {
  using L = SmemLayout<BN, STAGES, MT, KIND>;
  static_assert(KIND != 1 || (MT == 1 && BN == 128), "fp4 tiles are 128 x 128");
  static_assert(KIND != 2 || BN == 128, "packed weights are unpacked in 128-row tiles");
  constexpr bool FP4 = KIND == 1;
  constexpr bool PACKED = KIND == 2;
  constexpr int kXStep = FP4 ? 128 : BK;  // TMA x coordinate of one k block (bytes for the packed fp4 maps)
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem =
      reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * L::kABytes;
  uint8_t* sSF = smem + L::kSFOffset;  // [stage][SFA | SFB]
  uint8_t* sStage = smem + L::kStageOffset;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* empty = full + STAGES;
  uint64_t* tmem_full = empty + STAGES;  // [2]
  uint64_t* tmem_empty = tmem_full + 2;  // [2]
  uint64_t* fix_bar = tmem_empty + 2;    // landing of the partial slabs in the split-K fix-up
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(fix_bar + 1);
  int* s_misc = reinterpret_cast<int*>(tmem_slot + 2);  // [0] start-up ok, [1] tile barrier ok
  int* s_counts = s_misc + 2;                           // first m tile per group, grouped mode

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int total_kb = FP4 ? p.kb_total : (p.K + BK - 1) / BK;
  const bool grouped = p.group_counts != nullptr;
  const int n_tiles = (p.N + BN - 1) / BN;
  const int m_tiles = p.m_tiles;
  const int n_work = n_tiles * m_tiles * p.splits;
  const uint32_t spin = spin_budget(p.spin_limit);

  constexpr uint32_t kAccCols = BN < 32 ? 32 : BN;   // TMEM columns of one 128-row accumulator
  constexpr uint32_t kItemCols = MT * kAccCols;      // ... of one work item
  constexpr uint32_t kBufs = 2 * kItemCols <= 512 ? 2 : 1;
  constexpr uint32_t kSFCols = FP4 ? 64 : 0;   // two sets of (16 columns of A scales, 16 of B scales)
  constexpr uint32_t kSFCol0 = kBufs * kItemCols;
  constexpr uint32_t kTmemCols = FP4 ? 512 : kBufs * kItemCols;
  static_assert(kBufs * kItemCols + kSFCols <= 512, "TMEM budget");
  static_assert(kTmemCols <= 512 && (kTmemCols & (kTmemCols - 1)) == 0, "TMEM allocation");

  // Programmatic dependent launch: nothing below that depends on an earlier kernel runs before
  // pdl_wait(); the next kernel of the stream may become resident once every CTA has issued its last
  // MMA (pdl_launch_dependents in the MMA warp). Both are no-ops for a launch without the attribute.
  if (threadIdx.x == 0) {
    stamp(p, 0);
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], PACKED ? 2 : 1);  // the TMA producer (+ the warp that unpacks this stage's weights)
      mbar_init(&empty[s], 1);
    }
    mbar_init(&tmem_full[0], 1);
    mbar_init(&tmem_full[1], 1);
    mbar_init(&tmem_empty[0], 4);
    mbar_init(&tmem_empty[1], 4);
    mbar_init(fix_bar, 1);
    fence_mbar_init();
    int ok = 1;
    if (grouped) {
      pdl_wait();
      // The per-group row counts are final only once every source has finished dispatching.
      if (p.ag_flags != nullptr) ok = wait_sources(p, 0, p.ag_n_src - 1, gridDim.x) ? 1 : 0;
      int acc = 0;
      for (int e = 0; e < p.n_groups; ++e) {
        s_counts[e] = acc;  // first m tile of group e
        acc += (static_cast<int>(__ldcg(p.group_counts + e)) + BM - 1) / BM;
      }
      s_counts[p.n_groups] = acc;
    }
    s_misc[0] = ok;
    s_misc[1] = 1;
  }
  __syncthreads();  // barriers, start-up state
  // The producer warp goes ahead (its first weight tiles depend on no earlier kernel). The other
  // warps wait for the prerequisite grid first, and TMEM is allocated only after that wait: a CTA
  // that held TMEM while it waited could starve a CTA of the prerequisite grid on the same SM.
  uint32_t tmem_base = 0;
  if (warp >= 1 && warp < 6) {
    pdl_wait();
    if (warp == 1) {
      tmem_alloc(tmem_slot, kTmemCols);
      tmem_relinquish();
    }
    tc_fence_before_sync();
    asm volatile("bar.sync 2, 160;" ::: "memory");
    tc_fence_after_sync();
    tmem_base = *tmem_slot;
  }
  const bool all_ok = s_misc[0] != 0;

  // work item w -> tile coordinates; consecutive items share the weight tile (m fastest)
  auto decode = [&](int w) -> WorkItem {
    WorkItem it;
    const int mt = w % m_tiles;
    const int rest = w / m_tiles;
    const int nt = rest % n_tiles;
    it.z = rest / n_tiles;
    it.tile = nt * m_tiles + mt;
    it.n0 = nt * BN;
    it.kb0 = it.z * p.kb_per_split;
    it.nkb = total_kb - it.kb0;
    if (it.nkb > p.kb_per_split) it.nkb = p.kb_per_split;
    it.group = 0;
    it.m0 = mt * BM * MT;
    it.rows = p.M;
    it.valid = all_ok && it.nkb > 0;
    if (grouped) {
      it.valid = false;
      for (int e = 0; e < p.n_groups; ++e) {
        if (mt >= s_counts[e] && mt < s_counts[e + 1]) {
          it.group = e;
          it.m0 = (mt - s_counts[e]) * BM;
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
    // The whole warp runs this loop. TMA copies issued by one thread complete about one per memory
    // round trip (measured: the rate of a single issuing thread does not grow with the number of
    // stages in flight, it grows with the number of issuing threads), so every copy of a stage
    // has its own lane, and consecutive stages use different lanes: lane = stage * 4 + copy.
    constexpr int kBOps = (BN + 127) / 128;  // tile-major weights: one box per 128 weight rows
    uint32_t iter = 0;  // k-block counter across all items of this CTA
    bool ok = true;
    bool pdl_pending = true;  // this warp has not yet waited for the prerequisite grid
    if (grouped) {            // grouped tiles depend on the dispatch from the start
      pdl_wait();
      pdl_pending = false;
    }
    // copies of a k block that depend on earlier kernels or on peers: activations (and their scales)
    auto issue_a = [&](const WorkItem& it, int kb, uint32_t iter_kb) __attribute__((always_inline)) {
      const int s = iter_kb % STAGES;
      const int op = lane - (s & 7) * 4;
      if (FP4 && op == 3)
        bulk_load(sSF + s * (L::kSFABytes + L::kSFBBytes),
                  p.sfa + ((static_cast<long long>(it.group) * p.sfa_group_tiles + (it.m0 >> 7)) * total_kb +
                           it.kb0 + kb) * 2048,
                  L::kSFABytes, &full[s]);
      // rows past M read as zeros (the box is filled in full either way)
      if (p.wide_boxes && MT == 2) {
        if (op == 2) tma_load_3d(sA + s * L::kABytes, &tmA, &full[s], (it.kb0 + kb) * kXStep, it.m0, it.group);
      } else if (op >= 2 && op < 2 + MT)
        tma_load_3d(sA + s * L::kABytes + (op - 2) * (BM * BK * 2), &tmA, &full[s], (it.kb0 + kb) * kXStep,
                    it.m0 + (op - 2) * BM, it.group);
    };
    for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x) {
      const WorkItem it = decode(w);
      bool need_wait = p.ag_flags != nullptr && !grouped;
      if (!it.valid) {
        if (pdl_pending) {
          pdl_wait();
          pdl_pending = false;
        }
        // keep the waiter count of the grid exact: an empty item still passes the gate
        if (need_wait && lane == 0) wait_sources(p, 0, -1, static_cast<uint32_t>(n_work));
        continue;
      }
      // On the first item the weight copies of the whole ring are requested before this warp waits
      // for the prerequisite grid and for the peers; the activation copies of those k blocks follow
      // right after the wait. Later items pass the gate at their first k block.
      const int hold = pdl_pending ? (it.nkb < STAGES ? it.nkb : STAGES) - 1 : 0;
      for (int kb = 0; kb < it.nkb && ok; ++kb, ++iter) {
        const int s = iter % STAGES;
        const uint32_t ph = (iter / STAGES) & 1;
        if (iter >= STAGES && !mbar_wait(&empty[s], ph ^ 1, spin)) ok = false;
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) set_status_once(p.status, kStatusMbarTimeoutProducer);
          break;
        }
        if (lane == 0)
          mbar_arrive_expect_tx(&full[s], L::kABytes + (PACKED ? 0 : L::kBBytes) + L::kSFABytes + L::kSFBBytes);
        __syncwarp();
        const int op = lane - (s & 7) * 4;  // which copy of this stage this lane issues (0..3), if any
        // weights (and their scales) first: they depend on nothing that runs before this kernel
        if (FP4 && op == 1)
          // the scale atoms of this k block: 2 KB per 128 rows, contiguous in [row tile][k block]
          bulk_load(sSF + s * (L::kSFABytes + L::kSFBBytes) + L::kSFABytes,
                    p.sfb + ((static_cast<long long>(it.group) * ((p.N + 127) / 128) + (it.n0 >> 7)) * total_kb +
                             it.kb0 + kb) * 2048,
                    L::kSFBBytes, &full[s]);
        if (PACKED) {
          // the weight stage is written by the unpacking warps
        } else if (p.b_tiled && p.wide_boxes && BN == 256) {
          // both 128-row weight tiles of this k block in one 32 KB copy: [64][128][k block][n tile]
          if (op == 0) tma_load_4d(sB + s * L::kBBytes, &tmB, &full[s], 0, 0, it.kb0 + kb, it.n0 >> 7);
        } else if (p.b_tiled) {
          // tile-major weights: tile index = (n / 128) * total_kb + kb, box = 128 x 64 (or the
          // 64-row half of a tile for BN = 64)
          if (op >= 0 && op < kBOps)
            tma_load_3d(sB + s * L::kBBytes + op * 16384, &tmB, &full[s], 0, BN < 128 ? (it.n0 & 127) : 0,
                        ((it.n0 >> 7) + op) * total_kb + it.kb0 + kb);
        } else if (op == 0) {
          tma_load_3d(sB + s * L::kBBytes, &tmB, &full[s], (it.kb0 + kb) * kXStep, it.n0, it.group);
        }
        if (kb < hold) continue;  // activation copies of this k block are issued at k block `hold`
        if (kb == hold) {
          if (pdl_pending) {
            pdl_wait();
            pdl_pending = false;
          }
          if (need_wait) {
            int src_ok = 1;
            if (lane == 0) {
              int s_lo = 0, s_hi = p.ag_n_src - 1;  // rows_per_src <= 0: rows are not grouped by source
              if (p.ag_rows_per_src > 0) {
                const int m_end = it.m0 + BM * MT < it.rows ? it.m0 + BM * MT : it.rows;
                s_lo = it.m0 / p.ag_rows_per_src;
                s_hi = (m_end - 1) / p.ag_rows_per_src;
                if (s_hi >= p.ag_n_src) s_hi = p.ag_n_src - 1;
                if (s_lo > s_hi) s_lo = s_hi;
              }
              src_ok = wait_sources(p, s_lo, s_hi, static_cast<uint32_t>(n_work)) ? 1 : 0;
            }
            ok = __shfl_sync(0xffffffffu, src_ok, 0) != 0;
            need_wait = false;
            if (!ok) break;
          }
          for (int kk = 0; kk < hold; ++kk) issue_a(it, kk, iter - static_cast<uint32_t>(hold - kk));
        }
        issue_a(it, kb, iter);
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
        const uint32_t buf = t % kBufs;
        const uint32_t use = t / kBufs;
        // the epilogue must have drained this accumulator buffer (kBufs items ago)
        if (use >= 1 && !mbar_wait(&tmem_empty[buf], (use & 1) ^ 1, spin)) {
          set_status_once(p.status, kStatusMbarTimeoutMma);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * kItemCols;
        for (int kb = 0; kb < it.nkb; ++kb, ++iter) {
          const int s = iter % STAGES;
          const uint32_t ph = (iter / STAGES) & 1;
          if (!mbar_wait(&full[s], ph, spin)) {
            set_status_once(p.status, kStatusMbarTimeoutMma);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(sA + s * L::kABytes);
          const uint32_t b_addr = smem_u32(sB + s * L::kBBytes);
          if (FP4) {
            // scales of this k block -> TMEM (alternating column sets), then 4 MMAs of 64 values of K
            constexpr uint32_t idesc4 = make_idesc_nvfp4(BM, BN);
            const uint32_t sfa_t = tmem_base + kSFCol0 + (iter & 1) * 32;
            const uint32_t sfb_t = sfa_t + 16;
            const uint32_t sf_s = smem_u32(sSF + s * (L::kSFABytes + L::kSFBBytes));
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              tc_cp_scales(sfa_t + 4 * j, make_desc_scales(sf_s + j * 512));
              tc_cp_scales(sfb_t + 4 * j, make_desc_scales(sf_s + L::kSFABytes + j * 512));
            }
#pragma unroll
            for (int k = 0; k < 4; ++k)
              tc_mma_nvfp4(d_tmem, make_desc_kmajor_sw128(a_addr + k * 32), make_desc_kmajor_sw128(b_addr + k * 32),
                           idesc4, (kb | k) != 0 ? 1u : 0u, sfa_t + 4 * k, sfb_t + 4 * k);
            tc_commit(&empty[s]);
            continue;
          }
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t db = make_desc_kmajor_sw128(b_addr + k * 32);
#pragma unroll
            for (int h = 0; h < MT; ++h)
              tc_mma_f16(d_tmem + h * kAccCols, make_desc_kmajor_sw128(a_addr + h * (BM * BK * 2) + k * 32),
                         db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          tc_commit(&empty[s]);  // frees this smem stage once the MMAs above have read it
        }
        if (ok) tc_commit(&tmem_full[buf]);
        ++t;
      }
      pdl_launch_dependents();  // only epilogues are left in this CTA
    }
  } else if (PACKED && warp >= 6) {
    // ------------------------------ weight unpacking (KIND 2) -----------------
    // Warp dq takes the k blocks dq, dq + 4, ... of the CTA's sequence and unpacks the whole 128-row
    // tile of each (four rows per lane), so four stages are being filled at once and every lane has
    // the loads of four rows in flight: the unpacking is bound by the latency of the packed-block
    // loads, not by arithmetic. A k block is two groups of 32 weights per row: each is expanded to
    // int8 codes + scales (quant_expand.cuh), converted to bf16 and stored as four 16-byte chunks at
    // the position the 128-byte swizzle of the operand descriptors expects: chunk c of row r sits at
    // chunk c ^ (r % 8) of that row.
    if constexpr (PACKED) {
      const int dq = warp - 6;
      uint32_t iter = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x) {
        const WorkItem it = decode(w);
        if (!it.valid) continue;
        for (int kb = 0; kb < it.nkb && ok; ++kb, ++iter) {
          if ((iter & (kDequantWarps - 1)) != static_cast<uint32_t>(dq)) continue;
          const int s = iter % STAGES;
          const uint32_t ph = (iter / STAGES) & 1;
          if (iter >= STAGES && !mbar_wait(&empty[s], ph ^ 1, spin)) ok = false;
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) {
            if (lane == 0) set_status_once(p.status, kStatusMbarTimeoutProducer);
            break;
          }
          switch (p.q_type) {
            case kQ_Q4_0: unpack_kblock<kQ_Q4_0>(p, it.n0, it.kb0 + kb, sB + s * L::kBBytes, lane); break;
            case kQ_Q4_1: unpack_kblock<kQ_Q4_1>(p, it.n0, it.kb0 + kb, sB + s * L::kBBytes, lane); break;
            case kQ_Q5_0: unpack_kblock<kQ_Q5_0>(p, it.n0, it.kb0 + kb, sB + s * L::kBBytes, lane); break;
            case kQ_Q5_1: unpack_kblock<kQ_Q5_1>(p, it.n0, it.kb0 + kb, sB + s * L::kBBytes, lane); break;
            case kQ_Q8_0: unpack_kblock<kQ_Q8_0>(p, it.n0, it.kb0 + kb, sB + s * L::kBBytes, lane); break;
            case kQ_Q4_K: unpack_kblock<kQ_Q4_K>(p, it.n0, it.kb0 + kb, sB + s * L::kBBytes, lane); break;
            case kQ_Q5_K: unpack_kblock<kQ_Q5_K>(p, it.n0, it.kb0 + kb, sB + s * L::kBBytes, lane); break;
            default: unpack_kblock<kQ_Q6_K>(p, it.n0, it.kb0 + kb, sB + s * L::kBBytes, lane); break;
          }
          // generic-proxy stores -> visible to the tensor core's reads (async proxy), then this warp's arrival
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(&full[s]);
        }
      }
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    uint8_t* stage = sStage + static_cast<size_t>(q) * 32 * kStagePitch;
    uint8_t* my_row = stage + static_cast<size_t>(lane) * kStagePitch;
    const bool vec_ok = (p.N & 7) == 0;
    const bool fix = p.ws != nullptr && p.splits > 1;  // split-K combined in this kernel
    const bool swiglu = p.epi == kEpiSwigluBf16;
    const int n_total = swiglu ? (p.N >> 1) : p.N;  // output row length
    const int out_cols = swiglu ? BN / 2 : BN;      // output columns of one tile
    const int units_per_half = (out_cols + kStageCols - 1) / kStageCols;
    const int n_units = MT * units_per_half;        // 64-output-column x 128-row pieces of a tile
    const size_t ws_half = static_cast<size_t>(BN) * 128;  // bf16 elements of one row half of a slab
    uint32_t t = 0, fix_phase = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < n_work; w += gridDim.x) {
      const WorkItem it = decode(w);
      if (!it.valid) continue;
      const uint32_t buf = t % kBufs;
      const uint32_t use = t / kBufs;
      if (ok && !mbar_wait(&tmem_full[buf], use & 1, spin)) {
        if (lane == 0) set_status_once(p.status, kStatusMbarTimeoutEpilogue);
        ok = false;
      }
      ok = __all_sync(0xffffffffu, ok);  // tcgen05.ld below is warp-collective
      if (!ok) break;
      tc_fence_after_sync();
      if (t == 0 && warp == 2 && lane == 0) stamp(p, 1);
      const int n0 = it.n0;
      const int group = it.group;
      const __nv_bfloat16* bias =
          p.bias != nullptr ? p.bias + static_cast<long long>(group) * p.N : nullptr;
      const uint32_t lane_addr = tmem_base + buf * kItemCols + (static_cast<uint32_t>(q * 32) << 16);
      // this thread's row inside a slab of the split-K workspace: [half][col / 8][128 rows][8]
      const __nv_bfloat16* ws_tile =
          fix ? p.ws + static_cast<size_t>(it.tile) * p.splits * MT * ws_half + (q * 32 + lane) * 8 : nullptr;

      if (fix) {
        // ---- phase A: this split's partial tile -> its slab (bf16; a warp's 32 rows of one
        // 8-column group are 512 contiguous bytes), then meet the other splits of the tile ----
        __nv_bfloat16* slab = const_cast<__nv_bfloat16*>(ws_tile) + static_cast<size_t>(it.z) * MT * ws_half;
        // software pipelined: the TMEM load of chunk i + 1 is in flight while chunk i is packed
        // and stored (64 columns per chunk, two register sets)
        constexpr int kChunks = MT * (BN / 64);
        auto issue = [&](int i, uint32_t (&r)[2][32]) __attribute__((always_inline)) {
          const uint32_t addr = lane_addr + (i / (BN / 64)) * kAccCols + (i % (BN / 64)) * 64;
          tmem_ld_32x32b_x32(addr, r[0]);
          tmem_ld_32x32b_x32(addr + 32, r[1]);
        };
        auto store = [&](int i, const uint32_t (&r)[2][32]) __attribute__((always_inline)) {
          __nv_bfloat16* dst = slab + (i / (BN / 64)) * ws_half + static_cast<size_t>((i % (BN / 64)) * 8) * 1024;
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            const uint32_t* v = &r[g >> 2][(g & 3) * 8];
            uint4 o4;
            o4.x = pack_bf16x2(__uint_as_float(v[0]), __uint_as_float(v[1]));
            o4.y = pack_bf16x2(__uint_as_float(v[2]), __uint_as_float(v[3]));
            o4.z = pack_bf16x2(__uint_as_float(v[4]), __uint_as_float(v[5]));
            o4.w = pack_bf16x2(__uint_as_float(v[6]), __uint_as_float(v[7]));
            __stcg(reinterpret_cast<uint4*>(dst + static_cast<size_t>(g) * 1024), o4);
          }
        };
        uint32_t ra[2][32], rb[2][32];
        issue(0, ra);
#pragma unroll 1
        for (int i = 0; i < kChunks; i += 2) {
          tmem_ld_wait();
          if (i + 1 < kChunks) issue(i + 1, rb);
          store(i, ra);
          if (i + 1 < kChunks) {
            tmem_ld_wait();
            if (i + 2 < kChunks) issue(i + 2, ra);
            store(i + 1, rb);
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[buf]);
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (warp == 2 && lane == 0) {
          stamp(p, 2);
          uint32_t* arrived = p.ws_tickets + 2 * it.tile;
          atomicAdd(arrived, 1u);
          int met = 1;
          uint32_t n = 0;
          while (ld_acquire_gpu(arrived) < static_cast<uint32_t>(p.splits)) {
            if (++n > spin) {
              set_status_peer_timeout(p.status);
              met = 0;
              break;
            }
          }
          s_misc[1] = met;
          stamp(p, 3);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (s_misc[1] == 0) {
          ok = false;
          break;
        }
      }

      // 64 accumulator columns [col, col + 64) of row half h for this thread's row: straight from
      // TMEM, or summed over the slabs of every split (landed in shared memory, see below)
      int unit_acc0 = 0;          // first accumulator column of the unit whose slabs are in shared memory
      uint32_t unit_bytes = 0;    // bytes of one split's share of that unit
      float acc_scale = 1.f;      // NVFP4: second-level scales of this thread's row and of the weights
      auto load_acc = [&](int h, int col, float (&a)[64]) __attribute__((always_inline)) {
        if (!fix) {
          tmem_load_cols<2>(lane_addr + h * kAccCols + col, a);
          if (FP4) {
#pragma unroll
            for (int j = 0; j < 64; ++j) a[j] *= acc_scale;
          }
        } else
          smem_sum_cols(smem + ((col - unit_acc0) >> 3) * 2048 + (q * 32 + lane) * 16, p.splits, unit_bytes, a);
      };

      // with the fix-up the 64-column units of the tile are dealt out over its splits
#pragma unroll 1
      for (int u = fix ? it.z : 0; u < n_units; u += fix ? p.splits : 1) {
        const int h = u / units_per_half;
        const int oc = (u - h * units_per_half) * kStageCols;  // first output column inside the tile
        const int width = out_cols - oc < kStageCols ? out_cols - oc : kStageCols;  // 32 or 64
        if (fix) {
          // Land every split's share of this unit in the operand ring (idle now: the one work item
          // of this CTA has been multiplied) with one bulk copy per split, each issued by its own
          // lane, instead of chains of dependent global loads. A unit of n accumulator columns is
          // n / 8 column groups of 2 KB, contiguous inside a slab.
          unit_acc0 = swiglu ? 2 * oc : oc;
          unit_bytes = static_cast<uint32_t>(swiglu ? 2 * width : width) * 256u;
          asm volatile("bar.sync 1, 128;" ::: "memory");  // the previous unit has been read out of the ring
          if (warp == 2) {
            if (lane == 0) {
              asm volatile("fence.proxy.async;" ::: "memory");  // slabs and ring were touched by plain stores / loads
              mbar_arrive_expect_tx(fix_bar, static_cast<uint32_t>(p.splits) * unit_bytes);
            }
            __syncwarp();
            if (lane < p.splits)
              bulk_load(smem + static_cast<size_t>(lane) * unit_bytes,
                        p.ws + (static_cast<size_t>(it.tile) * p.splits + lane) * MT * ws_half + h * ws_half +
                            static_cast<size_t>(unit_acc0 >> 3) * 1024,
                        unit_bytes, fix_bar);
          }
          if (!mbar_wait(fix_bar, fix_phase, spin)) {
            set_status_once(p.status, kStatusMbarTimeoutEpilogue);
            s_misc[1] = 0;
          }
          fix_phase ^= 1;
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (s_misc[1] == 0) {
            ok = false;
            break;
          }
        }
        const int row = it.m0 + h * BM + q * 32 + lane;
        const bool row_ok = row < it.rows;
        if (FP4) {
          acc_scale = p.w_gscale != nullptr ? p.w_gscale[group] : 1.f;
          if (p.a_gscale != nullptr && row_ok) acc_scale *= p.a_gscale[static_cast<long long>(group) * p.a_gs_stride + row];
        }

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
          float a[64];
          load_acc(h, oc, a);
          const int col0 = n0 + oc;
          if (row_ok && col0 < p.N && red_base != nullptr) {
            float* d = red_base + static_cast<long long>(row_local) * p.dst_ld + col0;
#pragma unroll
            for (int j = 0; j < 64; j += 4) {
              if (vec_ok && col0 + j + 4 <= p.N) {
                red_add_v4_f32(d + j, wgt * a[j], wgt * a[j + 1], wgt * a[j + 2], wgt * a[j + 3]);
              } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                  if (col0 + j + e < p.N) atomicAdd(d + j + e, wgt * a[j + e]);
              }
            }
          }
        } else if (p.epi == kEpiStoreF32) {
          float a[64];
          load_acc(h, oc, a);
          const int col0 = n0 + oc;
          if (row_ok && col0 < p.N) {
            float* d = reinterpret_cast<float*>(p.C) + static_cast<long long>(group) * p.c_group_stride +
                       static_cast<long long>(row) * p.ldc + col0;
            const bool vec = (p.ldc & 3) == 0 && vec_ok;
#pragma unroll
            for (int j = 0; j < 64; j += 4) {
              float o[4] = {a[j], a[j + 1], a[j + 2], a[j + 3]};
              if (bias != nullptr) {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                  if (col0 + j + e < p.N) o[e] += __bfloat162float(bias[col0 + j + e]);
              }
              if (vec && col0 + j + 4 <= p.N) {
                *reinterpret_cast<float4*>(d + j) = make_float4(o[0], o[1], o[2], o[3]);
              } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                  if (col0 + j + e < p.N) d[j + e] = o[e];
              }
            }
          }
        } else {
          // ---- bf16 outputs (plain store, SwiGLU, routed slab store): accumulators -> registers
          // -> a padded shared-memory tile -> row-contiguous 16-byte stores, 64 output columns per
          // round, so local HBM and NVLink both see full lines. Each warp stages and writes only
          // its own 32 rows; __syncwarp is all it needs.
          const int oc0 = (swiglu ? (n0 >> 1) : n0) + oc;  // first output column of this unit
          const bool out_vec =
              (n_total & 7) == 0 && (((p.epi == kEpiSlabBf16) ? p.dst_ld : p.ldc) & 7) == 0;
          if (swiglu) {
            // 32 outputs come from 64 accumulator columns: 32 gate | 32 up
#pragma unroll 1
            for (int c = 0; c < width; c += 32) {
              float a[64];
              load_acc(h, 2 * (oc + c), a);
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                float v[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] = act_fn(a[j + e], p.act) * a[32 + j + e];
                uint4 o4;
                o4.x = pack_bf16x2(v[0], v[1]);
                o4.y = pack_bf16x2(v[2], v[3]);
                o4.z = pack_bf16x2(v[4], v[5]);
                o4.w = pack_bf16x2(v[6], v[7]);
                *reinterpret_cast<uint4*>(my_row + (c + j) * 2) = o4;
              }
            }
          } else {
            float a[64];
            load_acc(h, oc, a);
            const int col0 = n0 + oc;
            if (bias != nullptr) {
#pragma unroll
              for (int j = 0; j < 64; ++j)
                if (col0 + j < p.N) a[j] += __bfloat162float(bias[col0 + j]);
            }
#pragma unroll
            for (int j = 0; j < 64; j += 8) {
              uint4 o4;
              o4.x = pack_bf16x2(a[j], a[j + 1]);
              o4.y = pack_bf16x2(a[j + 2], a[j + 3]);
              o4.z = pack_bf16x2(a[j + 4], a[j + 5]);
              o4.w = pack_bf16x2(a[j + 6], a[j + 7]);
              *reinterpret_cast<uint4*>(my_row + j * 2) = o4;
            }
          }
          __syncwarp();
          const int chunks = width / 8;  // 16-byte chunks per staged row: 4 or 8
          const int rows_per_it = 32 / chunks;
          for (int r0 = 0; r0 < 32; r0 += rows_per_it) {
            const int rr = r0 + lane / chunks;
            const int ch = lane % chunks;
            const int grow = it.m0 + h * BM + q * 32 + rr;
            const int gcol = oc0 + ch * 8;
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

      if (fix) {
        // the last split to leave the tile re-arms its two counters for the next launch
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (warp == 2 && lane == 0) {
          uint32_t* tk = p.ws_tickets + 2 * it.tile;
          const uint32_t old = atomicAdd(tk + 1, 1u);
          if (old == static_cast<uint32_t>(p.splits) - 1) {
            tk[0] = 0;
            tk[1] = 0;
          }
        }
      } else {
        // hand the accumulator buffer back to the MMA warp
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[buf]);
      }
      ++t;
    }
    if (warp == 2 && lane == 0) stamp(p, 4);
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
  if (threadIdx.x == 0) stamp(p, 5);
}

template <int BN, int STAGES, int MT, int KIND = 0>
void launch_impl(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p,
                 cudaStream_t stream) {
  using L = SmemLayout<BN, STAGES, MT, KIND>;
  auto kern = gemm_bf16_kernel<BN, STAGES, MT, KIND>;
  ensure_dynamic_smem(kern, L::kTotal);
  const int sms = sm_count();
  const int n_work = ((p.N + BN - 1) / BN) * p.m_tiles * p.splits;
  const int grid = n_work < sms ? n_work : sms;
  // the splits of a tile wait for each other: ask for a launch that is resident as a whole
  const bool cooperative = p.ws != nullptr && p.splits > 1;
  launch_kernel(kern, dim3(grid), dim3(KIND == 2 ? kThreads + 32 * kDequantWarps : kThreads), L::kTotal, stream,
                /*pdl=*/true, cooperative, tmA, tmB, p);
}

int tiles_of(int M, int N, int bn, int mt) {
  return ((N + bn - 1) / bn) * ((M + 128 * mt - 1) / (128 * mt));
}

}  // namespace

int gemm_max_fixup_splits(int bn, int mt, bool swiglu) {
  // every split's share of one 64-output-column unit is landed in the operand ring at once
  const int stages = mt == 2 ? (bn == 64 ? 5 : (bn == 256 ? 3 : 4)) : (bn == 64 ? 8 : (bn == 256 ? 4 : 6));
  const int ring = stages * (mt * BM * BK * 2 + bn * BK * 2);
  const int acc_cols = swiglu ? (bn >= 128 ? 128 : bn) : 64;
  const int s = ring / (acc_cols * 256);
  return s > 32 ? 32 : s;
}

size_t gemm_ws_bytes(int M, int N, int bn, int mt, int splits) {
  return static_cast<size_t>(tiles_of(M, N, bn, mt)) * splits * mt * bn * 128 * sizeof(__nv_bfloat16);
}
int gemm_ws_tickets(int M, int N, int bn, int mt) { return 2 * tiles_of(M, N, bn, mt); }

void launch_gemm_bf16(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int bn,
                      int mt, cudaStream_t stream) {
  if (p.kind == 1) {
    launch_impl<128, 5, 1, 1>(tmA, tmB, p, stream);
    return;
  }
  if (p.kind == 2) {  // GGUF-packed weights, 128-column tiles
    if (mt == 2)
      launch_impl<128, 4, 2, 2>(tmA, tmB, p, stream);
    else
      launch_impl<128, 6, 1, 2>(tmA, tmB, p, stream);
    return;
  }
  if (mt == 2) {
    switch (bn) {
      case 64:
        launch_impl<64, 5, 2>(tmA, tmB, p, stream);
        break;
      case 256:
        launch_impl<256, 3, 2>(tmA, tmB, p, stream);
        break;
      default:
        launch_impl<128, 4, 2>(tmA, tmB, p, stream);
        break;
    }
    return;
  }
  switch (bn) {
    case 64:
      launch_impl<64, 8, 1>(tmA, tmB, p, stream);
      break;
    case 256:
      launch_impl<256, 4, 1>(tmA, tmB, p, stream);
      break;
    default:
      launch_impl<128, 6, 1>(tmA, tmB, p, stream);
      break;
  }
}

}  // namespace oxb
