// Paged causal flash-attention for prefill chunks (ragged batch) on sm_100a.
//
// One CTA = one 64-row query tile of one (sequence, query head); each warp owns 16
// query rows and streams the 16-token KV pages of the sequence through the block
// table, up to its causal limit. The chunk's own K/V have already been appended to
// the paged cache, so prior context (earlier chunks, radix-cache hits) and the
// current chunk are read the same way. Online softmax in registers; mma.sync
// m16n8k16 bf16 with 16-byte global loads feeding fragments directly (same head-dim
// permutation trick as the decode kernel).
//
// Replaces flash_causal_batched_prefill_kernel
// (oxide-backend-cuda/src/kernels/flash_attn.cu:536-781), an O(S^2) scalar kernel
// over a contiguous slot cache.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "attn.cuh"

namespace oxb {

namespace {

constexpr int kPage = 16;
constexpr int kWarps = 4;
constexpr int kTileQ = 64;

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
      "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pk(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int D>
__global__ void __launch_bounds__(kWarps * 32) paged_prefill_kernel(const PrefillAttnParams p) {
  constexpr int KS = D / 16;
  constexpr int CPL = D / 32;
  constexpr int VCH = D / 64;
  constexpr int NTO = D / 8;  // n-tiles of O

  __shared__ __align__(16) __nv_bfloat16 s_out[kTileQ][D];

  const int tile = blockIdx.x;
  const int head = blockIdx.y;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2;
  const int t = lane & 3;
  const int G = p.Hq / p.Hkv;
  const int kvh = head / G;

  const int seq = p.tile_seq[tile];
  const int q0 = p.tile_q0[tile] + warp * 16;
  const int q_len = p.q_lens[seq];
  const int ctx = p.ctx_lens[seq];
  const int row_base = p.q_start[seq];
  const int pos_off = ctx - q_len;  // position of query 0 of this chunk

  const int r0 = q0 + g, r1 = q0 + g + 8;
  const bool rv0 = r0 < q_len, rv1 = r1 < q_len;
  const int pos0 = pos_off + r0, pos1 = pos_off + r1;

  // ---- Q fragments ----
  uint32_t qa[KS][4];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = r == 0 ? r0 : r1;
    const bool rv = r == 0 ? rv0 : rv1;
    const __nv_bfloat16* qp =
        p.q + static_cast<long long>(row_base + (rv ? row : 0)) * p.q_stride + head * D;
#pragma unroll
    for (int ci = 0; ci < CPL; ++ci) {
      uint4 v = *reinterpret_cast<const uint4*>(qp + (t + 4 * ci) * 8);
      if (!rv) v = make_uint4(0, 0, 0, 0);
      qa[2 * ci][r] = v.x;
      qa[2 * ci][r + 2] = v.y;
      qa[2 * ci + 1][r] = v.z;
      qa[2 * ci + 1][r + 2] = v.w;
    }
  }

  float o_acc[NTO][4];
#pragma unroll
  for (int i = 0; i < NTO; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  // causal limit of this warp's 16 rows
  int last_row = q0 + 15;
  if (last_row > q_len - 1) last_row = q_len - 1;
  const int max_pos = pos_off + last_row;  // < 0 when the warp has no valid row
  const int n_pages = q0 < q_len ? max_pos / kPage + 1 : 0;
  int first_page = 0;
  if (p.window > 0) {
    const int lo = pos_off + q0 - p.window + 1;
    if (lo > 0) first_page = lo / kPage;
  }

  const int* bt = p.block_tables + static_cast<long long>(seq) * p.max_blocks;
  const long long page_stride = static_cast<long long>(p.Hkv) * kPage * D;
  const long long head_off = static_cast<long long>(kvh) * kPage * D;

  auto checked = [&](int b) -> int {
    if (p.num_blocks > 0 && static_cast<unsigned>(b) >= static_cast<unsigned>(p.num_blocks)) {
      if (p.status != nullptr && (threadIdx.x & 31) == 0) atomicExch(p.status, 5 /* kStatusBadIndex */);
      return 0;
    }
    return b;
  };
  int blk = first_page < n_pages ? checked(bt[first_page]) : 0;
  for (int page = first_page; page < n_pages; ++page) {
    const int next_blk = page + 1 < n_pages ? bt[page + 1] : 0;  // checked when it is consumed
    const __nv_bfloat16* kp = p.k_cache + static_cast<long long>(blk) * page_stride + head_off;
    const __nv_bfloat16* vp = p.v_cache + static_cast<long long>(blk) * page_stride + head_off;

    uint4 kr[2][CPL];
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
      for (int ci = 0; ci < CPL; ++ci)
        kr[r][ci] = __ldg(reinterpret_cast<const uint4*>(kp + (g + 8 * r) * D + (t + 4 * ci) * 8));
    uint4 vr[4][VCH];
#pragma unroll
    for (int tk = 0; tk < 4; ++tk) {
      const int tok = 2 * t + (tk & 1) + 8 * (tk >> 1);
#pragma unroll
      for (int c = 0; c < VCH; ++c)
        vr[tk][c] = __ldg(reinterpret_cast<const uint4*>(vp + tok * D + (g + 8 * c) * 8));
    }

    // ---- S = Q K^T, two 8-token column tiles ----
    float s[2][4];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      s[r][0] = s[r][1] = s[r][2] = s[r][3] = 0.f;
#pragma unroll
      for (int ci = 0; ci < CPL; ++ci) {
        mma16816(s[r], qa[2 * ci], kr[r][ci].x, kr[r][ci].y);
        mma16816(s[r], qa[2 * ci + 1], kr[r][ci].z, kr[r][ci].w);
      }
    }

    // ---- mask + online softmax ----
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
#pragma unroll
      for (int x = 0; x < 2; ++x) {
        const int tk = page * kPage + 8 * r + 2 * t + x;
        const bool a0 = rv0 && tk <= pos0 && (p.window <= 0 || tk > pos0 - p.window);
        const bool a1 = rv1 && tk <= pos1 && (p.window <= 0 || tk > pos1 - p.window);
        s[r][x] = a0 ? s[r][x] * p.scale_log2 : -INFINITY;
        s[r][2 + x] = a1 ? s[r][2 + x] * p.scale_log2 : -INFINITY;
        mx0 = fmaxf(mx0, s[r][x]);
        mx1 = fmaxf(mx1, s[r][2 + x]);
      }
    }
#pragma unroll
    for (int o = 1; o < 4; o <<= 1) {
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
    }
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;
    const float al0 = ex2f(m0 - ms0), al1 = ex2f(m1 - ms1);
    m0 = mn0;
    m1 = mn1;
    float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
#pragma unroll
      for (int x = 0; x < 2; ++x) {
        s[r][x] = ex2f(s[r][x] - ms0);
        s[r][2 + x] = ex2f(s[r][2 + x] - ms1);
        ps0 += s[r][x];
        ps1 += s[r][2 + x];
      }
    }
    l0 = l0 * al0 + ps0;
    l1 = l1 * al1 + ps1;
#pragma unroll
    for (int i = 0; i < NTO; ++i) {
      o_acc[i][0] *= al0;
      o_acc[i][1] *= al0;
      o_acc[i][2] *= al1;
      o_acc[i][3] *= al1;
    }
    const uint32_t pa[4] = {pk(s[0][0], s[0][1]), pk(s[0][2], s[0][3]), pk(s[1][0], s[1][1]),
                            pk(s[1][2], s[1][3])};

    // ---- O += P V ----
#pragma unroll
    for (int c = 0; c < VCH; ++c) {
      const uint32_t va[4] = {vr[0][c].x, vr[0][c].y, vr[0][c].z, vr[0][c].w};
      const uint32_t vb[4] = {vr[1][c].x, vr[1][c].y, vr[1][c].z, vr[1][c].w};
      const uint32_t vc[4] = {vr[2][c].x, vr[2][c].y, vr[2][c].z, vr[2][c].w};
      const uint32_t vd[4] = {vr[3][c].x, vr[3][c].y, vr[3][c].z, vr[3][c].w};
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const uint32_t sel = (e & 1) ? 0x7632u : 0x5410u;
        const uint32_t b0 = __byte_perm(va[e >> 1], vb[e >> 1], sel);
        const uint32_t b1 = __byte_perm(vc[e >> 1], vd[e >> 1], sel);
        mma16816(o_acc[8 * c + e], pa, b0, b1);
      }
    }
    blk = checked(next_blk);
  }

  // ---- finalize: divide by the row sums, stage in smem, write coalesced ----
#pragma unroll
  for (int o = 1; o < 4; o <<= 1) {
    l0 += __shfl_xor_sync(0xffffffffu, l0, o);
    l1 += __shfl_xor_sync(0xffffffffu, l1, o);
  }
  const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f;
  const float inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
  const int sr = warp * 16;
#pragma unroll
  for (int i = 0; i < NTO; ++i) {
    const int c = i >> 3, e = i & 7;
    const int d0 = 8 * (2 * t + 8 * c) + e;  // column 2t; column 2t+1 is 8 dims further
    s_out[sr + g][d0] = __float2bfloat16(o_acc[i][0] * inv0);
    s_out[sr + g][d0 + 8] = __float2bfloat16(o_acc[i][1] * inv0);
    s_out[sr + g + 8][d0] = __float2bfloat16(o_acc[i][2] * inv1);
    s_out[sr + g + 8][d0 + 8] = __float2bfloat16(o_acc[i][3] * inv1);
  }
  __syncwarp();
  constexpr int CH = D / 8;  // 16-byte chunks per row
  for (int idx = lane; idx < 16 * CH; idx += 32) {
    const int rr = idx / CH, ch = idx - rr * CH;
    const int row = q0 + rr;
    if (row < q_len) {
      const uint4 v = *reinterpret_cast<const uint4*>(&s_out[sr + rr][ch * 8]);
      *reinterpret_cast<uint4*>(p.out + static_cast<long long>(row_base + row) * p.out_stride +
                                head * D + ch * 8) = v;
    }
  }
}

}  // namespace

void launch_paged_prefill(const PrefillAttnParams& p, int n_tiles, int head_dim,
                          cudaStream_t stream) {
  if (n_tiles <= 0) return;
  dim3 grid(n_tiles, p.Hq);
  if (head_dim == 128)
    paged_prefill_kernel<128><<<grid, kWarps * 32, 0, stream>>>(p);
  else
    paged_prefill_kernel<64><<<grid, kWarps * 32, 0, stream>>>(p);
}

}  // namespace oxb
