// Paged split-KV flash-decode for grouped-query attention on sm_100a.
//
// One CTA = (sequence, KV head, KV split); each of its 4 warps walks 16-token pages
// of that split through the block table and keeps its own online-softmax state for
// all query heads of the group. The products run on tensor cores with the page as
// the M dimension:  S^T[16 tok x 8 heads] = K_page * Q^T,  O^T[dims x 8 heads] +=
// V_page^T * P^T  (mma.sync m16n8k16 -- 8 query heads against one page cannot fill
// a 128-row tcgen05 tile, and this kernel is bound by the KV stream from HBM, which
// every query head of the group shares). Every warp keeps a ring of kRing pages in
// flight with cp.async (16-byte chunks, XOR-swizzled so that the fragment reads are
// bank-conflict free): the bytes a warp has outstanding are what sets the rate of a
// latency-bound stream, and registers cannot hold more than one page. The MMA
// fragments are read from the ring with 16-byte loads in the pattern of the page
// itself: the head-dim permutation that makes this possible is applied identically
// to Q, and V is transposed in registers with byte permutes; P is transposed with
// movmatrix.
//
// A second kernel merges the per-split (max, sum, O) partials.
//
// Replaces split_k_flash_decode_continuous_batch_kernel + reduce
// (oxide-backend-cuda/src/kernels/megakernel_ops.cu:463-682) and the single-sequence
// flash_decode_* kernels (flash_attn.cu:110-528), which are scalar warp-per-head loops.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/device_info.h"
#include "attn.cuh"

namespace oxb {

namespace {

constexpr int kPage = 16;
constexpr int kWarps = 4;
constexpr int kRing = 3;   // pages per warp in the shared-memory ring (2 in flight while 1 is consumed)

// see sm100.cuh (this file is also built into the plain C library, without the tensor-core header)
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void cp_async_16(uint32_t smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_dst), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
// 16-byte chunk c of token row r sits at chunk c ^ swz(r) of that row: the K fragment reads (rows
// 2k, 2k+1 x 4 chunks per quarter warp) and the V fragment reads (4 rows of equal parity x 2 chunks)
// then touch 8 different 16-byte bank groups.
__device__ __forceinline__ int swz(int row) { return (((row >> 1) & 3) << 1) ^ ((row & 1) << 2); }

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
      "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// D = head dim (64 or 128); NT = number of 8-head column tiles (group size <= 8*NT).
// MASS: also record the per-page softmax statistics of every head (see DecodeAttnParams::page_ml).
template <int D, int NT, bool MASS>
__global__ void __launch_bounds__(kWarps * 32)
paged_decode_kernel(const DecodeAttnParams p) {
  constexpr int KS = D / 16;   // k-steps of QK^T
  constexpr int CPL = D / 32;  // 16-byte K chunks per lane per row
  constexpr int VCH = D / 64;  // 16-byte V chunks per lane per token
  constexpr int MT = D / 16;   // m-tiles of O^T

  pdl_wait();  // q and the newest K/V rows come from the kernel before this one
  const int seq = blockIdx.x;
  const int kvh = blockIdx.y;
  const int split = blockIdx.z;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2;
  const int t = lane & 3;
  const int G = p.Hq / p.Hkv;

  const int seq_len = p.seq_lens[seq];
  const int win_start = (p.window > 0 && seq_len > p.window) ? seq_len - p.window : 0;
  int n_pages = (seq_len + kPage - 1) / kPage;
  if (n_pages > p.max_blocks) {
    // a length beyond the block-table row: recorded, and the walk stops at the end of the row
    if (p.status != nullptr && threadIdx.x == 0) atomicCAS(p.status, 0, 5 /* kStatusBadIndex */);
    n_pages = p.max_blocks;
  }
  const int pps = *p.pages_per_split;
  const int first_page = win_start / kPage;
  const int pg_lo = first_page + split * pps;
  int pg_hi = pg_lo + pps;
  if (pg_hi > n_pages) pg_hi = n_pages;

  const long long part_idx0 = (static_cast<long long>(seq) * p.Hq + kvh * G) * p.max_splits;
  if (pg_lo >= pg_hi || seq_len <= 0) {
    // nothing in this split: mark every head's partial as empty
    for (int h = threadIdx.x; h < G; h += blockDim.x) {
      float* ml = p.part_ml + ((part_idx0 + static_cast<long long>(h) * p.max_splits + split) << 1);
      ml[0] = -INFINITY;
      ml[1] = 0.f;
    }
    return;
  }

  // ---- Q fragments (B operand of S^T = K * Q^T), with the shared dim permutation ----
  uint32_t qf[NT][KS][2];
  {
    const __nv_bfloat16* qbase = p.q + static_cast<long long>(seq) * p.q_stride;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int h = nt * 8 + g;
      const bool valid = h < G;
      const __nv_bfloat16* qh = qbase + static_cast<long long>(kvh * G + (valid ? h : 0)) * D;
#pragma unroll
      for (int ci = 0; ci < CPL; ++ci) {
        uint4 v = *reinterpret_cast<const uint4*>(qh + (t + 4 * ci) * 8);
        if (!valid) v = make_uint4(0, 0, 0, 0);
        qf[nt][2 * ci][0] = v.x;
        qf[nt][2 * ci][1] = v.y;
        qf[nt][2 * ci + 1][0] = v.z;
        qf[nt][2 * ci + 1][1] = v.w;
      }
    }
  }

  float m_run[NT][2], l_run[NT][2];
  float o_acc[NT][MT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    m_run[nt][0] = m_run[nt][1] = -INFINITY;
    l_run[nt][0] = l_run[nt][1] = 0.f;
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
      for (int x = 0; x < 4; ++x) o_acc[nt][i][x] = 0.f;
  }

  const int* bt = p.block_tables + static_cast<long long>(seq) * p.max_blocks;
  const long long page_stride = static_cast<long long>(p.Hkv) * kPage * D;  // elements per block
  const long long head_off = static_cast<long long>(kvh) * kPage * D;

  // a block id outside the pool is recorded and replaced by block 0 (never dereferenced)
  auto checked = [&](int b) -> int {
    if (p.num_blocks > 0 && static_cast<unsigned>(b) >= static_cast<unsigned>(p.num_blocks)) {
      if (p.status != nullptr && lane == 0) atomicCAS(p.status, 0, 5 /* kStatusBadIndex */);
      return 0;
    }
    return b;
  };
  // ---- per-warp ring of pages in shared memory ----
  extern __shared__ __align__(128) uint8_t ring_raw[];
  constexpr int kRowBytes = D * 2;
  constexpr int kPageBytes = kPage * kRowBytes;             // K or V of one page
  constexpr int kChunksPerRow = kRowBytes / 16;
  constexpr int kChunksPerLane = kPage * kChunksPerRow / 32;  // 16-byte chunks each lane copies per tensor
  const uint32_t ring = static_cast<uint32_t>(__cvta_generic_to_shared(ring_raw)) +
                        static_cast<uint32_t>(warp) * kRing * 2 * kPageBytes;
  auto issue = [&](int slot, int b) {
    const __nv_bfloat16* kp = p.k_cache + static_cast<long long>(b) * page_stride + head_off;
    const __nv_bfloat16* vp = p.v_cache + static_cast<long long>(b) * page_stride + head_off;
    const uint32_t dk = ring + static_cast<uint32_t>(slot) * 2 * kPageBytes;
    const uint32_t dv = dk + kPageBytes;
#pragma unroll
    for (int j = 0; j < kChunksPerLane; ++j) {
      const int c = lane + 32 * j;
      const int row = c / kChunksPerRow, ch = c % kChunksPerRow;
      const uint32_t off = static_cast<uint32_t>(row * kRowBytes + ((ch ^ swz(row)) << 4));
      cp_async_16(dk + off, kp + row * D + ch * 8);
      cp_async_16(dv + off, vp + row * D + ch * 8);
    }
  };
  // block ids run one page ahead of the copies, the copies kRing - 1 pages ahead of the math
  int page = pg_lo + warp;
  int issue_page = page;
  int blk_next = issue_page < pg_hi ? checked(bt[issue_page]) : 0;
#pragma unroll
  for (int i = 0; i < kRing - 1; ++i) {
    if (issue_page < pg_hi) {
      const int b = blk_next;
      const int np = issue_page + kWarps;
      blk_next = np < pg_hi ? checked(bt[np]) : 0;
      issue(i, b);
    }
    cp_async_commit();
    issue_page += kWarps;
  }
  int slot = 0;
  for (; page < pg_hi; page += kWarps) {
    // top up the ring, then wait until the oldest page has landed
    {
      int s_new = slot + kRing - 1;
      if (s_new >= kRing) s_new -= kRing;
      if (issue_page < pg_hi) {
        const int b = blk_next;
        const int np = issue_page + kWarps;
        blk_next = np < pg_hi ? checked(bt[np]) : 0;
        issue(s_new, b);
      }
      cp_async_commit();
      issue_page += kWarps;
    }
    cp_async_wait<kRing - 1>();
    __syncwarp();
    const uint32_t sk = ring + static_cast<uint32_t>(slot) * 2 * kPageBytes;
    const uint32_t sv = sk + kPageBytes;

    // ---- fragments of the page ----
    uint4 kr[2][CPL];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = g + 8 * r;
#pragma unroll
      for (int ci = 0; ci < CPL; ++ci)
        kr[r][ci] = lds128(sk + row * kRowBytes + (((t + 4 * ci) ^ swz(row)) << 4));
    }
    uint4 vr[4][VCH];
#pragma unroll
    for (int tk = 0; tk < 4; ++tk) {
      const int tok = 2 * t + (tk & 1) + 8 * (tk >> 1);
#pragma unroll
      for (int c = 0; c < VCH; ++c)
        vr[tk][c] = lds128(sv + tok * kRowBytes + (((g + 8 * c) ^ swz(tok)) << 4));
    }

    // ---- S^T = K * Q^T ----
    float s[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
      for (int ci = 0; ci < CPL; ++ci) {
        mma_bf16_16816(s[nt], kr[0][ci].x, kr[1][ci].x, kr[0][ci].y, kr[1][ci].y, qf[nt][2 * ci][0],
                       qf[nt][2 * ci][1]);
        mma_bf16_16816(s[nt], kr[0][ci].z, kr[1][ci].z, kr[0][ci].w, kr[1][ci].w,
                       qf[nt][2 * ci + 1][0], qf[nt][2 * ci + 1][1]);
      }
    }

    // ---- online softmax over the page's 16 tokens (rows of S^T) ----
    const int tok0 = page * kPage + g;
    const bool v0 = tok0 < seq_len && tok0 >= win_start;
    const bool v1 = tok0 + 8 < seq_len && tok0 + 8 >= win_start;
    uint32_t pb[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      float x00 = v0 ? s[nt][0] * p.scale_log2 : -INFINITY;  // tok g,   head 2t
      float x01 = v0 ? s[nt][1] * p.scale_log2 : -INFINITY;  // tok g,   head 2t+1
      float x10 = v1 ? s[nt][2] * p.scale_log2 : -INFINITY;  // tok g+8, head 2t
      float x11 = v1 ? s[nt][3] * p.scale_log2 : -INFINITY;  // tok g+8, head 2t+1
      float mx0 = fmaxf(x00, x10), mx1 = fmaxf(x01, x11);
#pragma unroll
      for (int o = 4; o < 32; o <<= 1) {
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
      }
      const float mn0 = fmaxf(m_run[nt][0], mx0), mn1 = fmaxf(m_run[nt][1], mx1);
      const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;
      const float a0 = ex2(m_run[nt][0] - ms0), a1 = ex2(m_run[nt][1] - ms1);
      m_run[nt][0] = mn0;
      m_run[nt][1] = mn1;
      const float p00 = ex2(x00 - ms0), p01 = ex2(x01 - ms1);
      const float p10 = ex2(x10 - ms0), p11 = ex2(x11 - ms1);
      l_run[nt][0] = l_run[nt][0] * a0 + p00 + p10;
      l_run[nt][1] = l_run[nt][1] * a1 + p01 + p11;
      if constexpr (MASS) {
        float ps0 = p00 + p10, ps1 = p01 + p11;
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
          ps0 += __shfl_xor_sync(0xffffffffu, ps0, o);
          ps1 += __shfl_xor_sync(0xffffffffu, ps1, o);
        }
        const int h0 = nt * 8 + 2 * t;
        if (g == 0 && h0 < G) {
          float2* dst = reinterpret_cast<float2*>(p.page_ml) +
                        (static_cast<long long>(seq) * p.max_blocks + page) * p.Hq + kvh * G + h0;
          dst[0] = make_float2(ms0, ps0);
          if (h0 + 1 < G) dst[1] = make_float2(ms1, ps1);
        }
      }
#pragma unroll
      for (int i = 0; i < MT; ++i) {
        o_acc[nt][i][0] *= a0;
        o_acc[nt][i][1] *= a1;
        o_acc[nt][i][2] *= a0;
        o_acc[nt][i][3] *= a1;
      }
      // P^T fragments: (tok 2t,2t+1 | head g) and (tok 2t+8,2t+9 | head g)
      pb[nt][0] = movmatrix_trans(pack2(p00, p01));
      pb[nt][1] = movmatrix_trans(pack2(p10, p11));
    }

    // ---- O^T += V^T * P^T ----
#pragma unroll
    for (int c = 0; c < VCH; ++c) {
      const uint32_t va[4] = {vr[0][c].x, vr[0][c].y, vr[0][c].z, vr[0][c].w};
      const uint32_t vb[4] = {vr[1][c].x, vr[1][c].y, vr[1][c].z, vr[1][c].w};
      const uint32_t vc[4] = {vr[2][c].x, vr[2][c].y, vr[2][c].z, vr[2][c].w};
      const uint32_t vd[4] = {vr[3][c].x, vr[3][c].y, vr[3][c].z, vr[3][c].w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const uint32_t a0 = __byte_perm(va[e], vb[e], 0x5410);  // dim 2e   | tok 2t, 2t+1
        const uint32_t a1 = __byte_perm(va[e], vb[e], 0x7632);  // dim 2e+1 | tok 2t, 2t+1
        const uint32_t a2 = __byte_perm(vc[e], vd[e], 0x5410);  // dim 2e   | tok 2t+8, 2t+9
        const uint32_t a3 = __byte_perm(vc[e], vd[e], 0x7632);  // dim 2e+1 | tok 2t+8, 2t+9
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
          mma_bf16_16816(o_acc[nt][4 * c + e], a0, a1, a2, a3, pb[nt][0], pb[nt][1]);
      }
    }
    __syncwarp();  // every lane is done with this slot before it is refilled
    if (++slot == kRing) slot = 0;
  }
  cp_async_wait<0>();
  pdl_launch_dependents();  // the KV stream of this CTA is done: the next kernel may become resident

  // ---- merge the 4 warps through shared memory (the ring is free now) ----
  __syncthreads();
  float(*s_o)[8 * NT][D] = reinterpret_cast<float(*)[8 * NT][D]>(ring_raw);
  float(*s_m)[8 * NT] = reinterpret_cast<float(*)[8 * NT]>(ring_raw + sizeof(float) * kWarps * 8 * NT * D);
  float(*s_l)[8 * NT] = s_m + kWarps;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    float l0 = l_run[nt][0], l1 = l_run[nt][1];
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
      l0 += __shfl_xor_sync(0xffffffffu, l0, o);
      l1 += __shfl_xor_sync(0xffffffffu, l1, o);
    }
    if (g == 0) {
      s_m[warp][nt * 8 + 2 * t] = m_run[nt][0];
      s_m[warp][nt * 8 + 2 * t + 1] = m_run[nt][1];
      s_l[warp][nt * 8 + 2 * t] = l0;
      s_l[warp][nt * 8 + 2 * t + 1] = l1;
    }
#pragma unroll
    for (int i = 0; i < MT; ++i) {
      const int c = i >> 2, e = i & 3;
      const int d0 = 8 * g + 64 * c + 2 * e;  // dim of fragment row g; row g+8 is d0 + 1
      s_o[warp][nt * 8 + 2 * t][d0] = o_acc[nt][i][0];
      s_o[warp][nt * 8 + 2 * t + 1][d0] = o_acc[nt][i][1];
      s_o[warp][nt * 8 + 2 * t][d0 + 1] = o_acc[nt][i][2];
      s_o[warp][nt * 8 + 2 * t + 1][d0 + 1] = o_acc[nt][i][3];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int h = idx / D, d = idx - h * D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) M = fmaxf(M, s_m[w][h]);
    float acc = 0.f, L = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float mw = s_m[w][h];
      const float f = mw == -INFINITY ? 0.f : ex2(mw - M);
      acc += f * s_o[w][h][d];
      L += f * s_l[w][h];
    }
    const long long pi = part_idx0 + static_cast<long long>(h) * p.max_splits + split;
    p.part_o[pi * D + d] = acc;
    if (d == 0) {
      p.part_ml[pi * 2] = M;
      p.part_ml[pi * 2 + 1] = L;
    }
  }
}

// out[seq, head, :] = sum_s w_s O_s / sum_s w_s l_s  with  w_s = 2^(m_s - max m)
template <int D>
__global__ void __launch_bounds__(D) decode_merge_kernel(const DecodeAttnParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int seq = blockIdx.x;
  const int head = blockIdx.y;
  const int d = threadIdx.x;
  const long long base = (static_cast<long long>(seq) * p.Hq + head) * p.max_splits;
  float M = -INFINITY;
  for (int s = 0; s < p.max_splits; ++s) M = fmaxf(M, p.part_ml[(base + s) * 2]);
  float acc = 0.f, L = 0.f;
  for (int s = 0; s < p.max_splits; ++s) {
    const float ms = p.part_ml[(base + s) * 2];
    if (ms == -INFINITY) continue;
    const float f = ex2(ms - M);
    acc += f * p.part_o[(base + s) * D + d];
    L += f * p.part_ml[(base + s) * 2 + 1];
  }
  const float r = L > 0.f ? acc / L : 0.f;
  const __nv_bfloat16 rb = __float2bfloat16(r);
  p.out[static_cast<long long>(seq) * p.out_stride + head * D + d] = rb;
  if (p.q8 != nullptr) {
    // a warp holds one block of 32 values: scale = amax / 127, codes, scale * sum
    const float v = __bfloat162float(rb);
    float amax = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float dq = amax / 127.f;
    const float inv = amax > 0.f ? 127.f / amax : 0.f;
    const int q = __float2int_rn(v * inv);
    int sum = q;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const long long e = (static_cast<long long>(seq) * p.Hq + head) * D + d;
    p.q8[e] = static_cast<signed char>(q);
    if ((d & 31) == 0) {
      p.q8_d[e >> 5] = dq;
      p.q8_s[e >> 5] = dq * static_cast<float>(sum);
    }
  }
}

// block_mass[seq, page] = sum_h page_sum[h] * 2^(page_max[h] - M_h) / L_h, with (M_h, L_h) the merged
// statistics of head h over all splits: the softmax probability mass the step's query put on the page.
__global__ void __launch_bounds__(128) block_mass_kernel(const DecodeAttnParams p) {
  __shared__ float s_M[128], s_rL[128];
  const int seq = blockIdx.x;
  const int seq_len = p.seq_lens[seq];
  int n_pages = (seq_len + kPage - 1) / kPage;
  if (n_pages > p.max_blocks) n_pages = p.max_blocks;
  const int win_start = (p.window > 0 && seq_len > p.window) ? seq_len - p.window : 0;
  const int first_page = win_start / kPage;
  int last_page = first_page + *p.pages_per_split * p.max_splits;  // pages past the last split were not walked
  if (last_page > n_pages) last_page = n_pages;
  for (int h = threadIdx.x; h < p.Hq; h += blockDim.x) {
    const long long base = (static_cast<long long>(seq) * p.Hq + h) * p.max_splits;
    float M = -INFINITY;
    for (int s = 0; s < p.max_splits; ++s) M = fmaxf(M, p.part_ml[(base + s) * 2]);
    float L = 0.f;
    for (int s = 0; s < p.max_splits; ++s) {
      const float ms = p.part_ml[(base + s) * 2];
      if (ms != -INFINITY) L += ex2(ms - M) * p.part_ml[(base + s) * 2 + 1];
    }
    s_M[h] = M;
    s_rL[h] = L > 0.f ? 1.f / L : 0.f;
  }
  __syncthreads();
  for (int page = threadIdx.x; page < p.max_blocks; page += blockDim.x) {
    float mass = 0.f;
    if (page >= first_page && page < last_page && seq_len > 0) {
      const float2* ml =
          reinterpret_cast<const float2*>(p.page_ml) + (static_cast<long long>(seq) * p.max_blocks + page) * p.Hq;
      for (int h = 0; h < p.Hq; ++h) {
        const float2 v = ml[h];
        if (v.y > 0.f) mass += v.y * ex2(v.x - s_M[h]) * s_rL[h];
      }
    }
    p.block_mass[static_cast<long long>(seq) * p.max_blocks + page] = mass;
  }
}

}  // namespace

template <int D, int NT>
void launch_split(const DecodeAttnParams& p, dim3 grid, cudaStream_t stream) {
  // the ring (kWarps x kRing pages of K and V) is also the scratch of the warp merge at the end
  constexpr size_t ring = static_cast<size_t>(kWarps) * kRing * 2 * kPage * D * 2;
  constexpr size_t merge = sizeof(float) * kWarps * 8 * NT * (D + 2);
  constexpr size_t smem = ring > merge ? ring : merge;
  if (p.page_ml != nullptr) {
    auto kern = paged_decode_kernel<D, NT, true>;
    ensure_dynamic_smem(kern, smem);
    launch_kernel(kern, grid, dim3(kWarps * 32), smem, stream, /*pdl=*/true, false, p);
  } else {
    auto kern = paged_decode_kernel<D, NT, false>;
    ensure_dynamic_smem(kern, smem);
    launch_kernel(kern, grid, dim3(kWarps * 32), smem, stream, /*pdl=*/true, false, p);
  }
}

cudaError_t launch_paged_decode(const DecodeAttnParams& p, int batch, int head_dim, cudaStream_t stream) {
  const int G = p.Hq / p.Hkv;
  dim3 grid(batch, p.Hkv, p.max_splits);
  dim3 mgrid(batch, p.Hq);
  if (head_dim == 128) {
    if (G <= 8)
      launch_split<128, 1>(p, grid, stream);
    else
      launch_split<128, 2>(p, grid, stream);
  } else {
    if (G <= 8)
      launch_split<64, 1>(p, grid, stream);
    else
      launch_split<64, 2>(p, grid, stream);
  }
  // a failed first launch leaves the partials stale: do not merge them into `out`
  const cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) return e;
  if (head_dim == 128)
    launch_kernel(decode_merge_kernel<128>, mgrid, dim3(128), 0, stream, /*pdl=*/true, false, p);
  else
    launch_kernel(decode_merge_kernel<64>, mgrid, dim3(64), 0, stream, /*pdl=*/true, false, p);
  if (p.page_ml != nullptr && p.block_mass != nullptr) block_mass_kernel<<<batch, 128, 0, stream>>>(p);
  return cudaPeekAtLastError();
}

}  // namespace oxb
