// Fused elementwise / normalisation kernels between the GEMMs (sm_100a).
//
//  finalize_norm : tail of the fused GEMM->reduce-scatter. Waits (bounded) until every
//                  contribution has arrived in this rank's fp32 accumulator, then per
//                  row: h = acc + bias + residual; residual_out = h; y = RMSNorm(h) * w;
//                  y is stored into the all-gather buffer of EVERY rank (peer stores over
//                  NVLink) and a per-source counter on each destination is bumped with a
//                  system-scope release. The accumulator is zeroed for its next use.
//                  With one rank and no counters it is residual-add + RMSNorm.
//                  (reference: fused_residual_rmsnorm_q8_1_cuda_kernel, norms_rope.cu:190-280;
//                   rms_norm_f32_kernel, norms_rope.cu:37-89)
//  qkv_rope_append: bias + optional per-head QK RMSNorm + half-split RoPE + write of K and V
//                  into the paged cache through a slot mapping, Q to a dense buffer.
//                  (reference: rope_continuous_batch_kernel megakernel_ops.cu:359-427,
//                   fused_qknorm_rope_batch_kernel norms_batch.cu:56-131,
//                   write_v_cache_continuous_batch_kernel megakernel_ops.cu:429-461,
//                   fused_paged_kv_write_fp16_kernel vec_ops_activations.cu:181-201)
//  swiglu        : SiLU(gate) * up or tanh-GELU(gate) * up (vec_ops_activations.cu:118-163).
//  embed_gather, fwht128 (fwht.cu:10-38), kv_block_copy, softcap.
#include "fused_ops.cuh"

#include "../common/device_info.h"
#include "../common/sm100.cuh"

namespace oxb {

namespace {

__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Relaxed: callers fence once at system scope, then signal all peers back to back.
__device__ __forceinline__ void red_relaxed_sys_add_u32(uint32_t* p, uint32_t v) {
  asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ float block_sum(float v, float* scratch) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float r = lane < nw ? scratch[lane] : 0.f;
  r = warp_sum(r);
  __syncthreads();
  return r;
}

constexpr int kNormMaxThreads = 1024;
constexpr int kNormMaxChunks = 4;  // 8-element chunks per thread: N <= 1024 * 8 * 4

// One CTA per row (looping when there are more rows than resident CTAs); every thread owns up to
// kNormMaxChunks 8-element chunks, kept in registers.
// int8 quantisation of V consecutive bf16-rounded values of this thread as part of a block of 32 that
// 32 / V neighbouring lanes hold together (the numbers of quant_q8_1_kernel): scale = amax / 127.
template <int V>
__device__ __forceinline__ void q8_block_store(const float (&y)[V], int8_t* q8, float* d_out, float* s_out,
                                               bool leader) {
  const unsigned m = __activemask();
  float v[V], amax = 0.f;
#pragma unroll
  for (int j = 0; j < V; ++j) {
    v[j] = __bfloat162float(__float2bfloat16(y[j]));
    amax = fmaxf(amax, fabsf(v[j]));
  }
#pragma unroll
  for (int o = 1; o < 32 / V; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(m, amax, o));
  const float d = amax / 127.f;
  const float inv = amax > 0.f ? 127.f / amax : 0.f;  // one division per block, not one per value
  int sum = 0;
  int8_t q[V];
#pragma unroll
  for (int j = 0; j < V; ++j) {
    const int qi = __float2int_rn(v[j] * inv);
    q[j] = static_cast<int8_t>(qi);
    sum += qi;
  }
#pragma unroll
  for (int o = 1; o < 32 / V; o <<= 1) sum += __shfl_xor_sync(m, sum, o);
  if constexpr (V == 8) {
    *reinterpret_cast<uint2*>(q8) = *reinterpret_cast<const uint2*>(q);
  } else {
    *reinterpret_cast<uint32_t*>(q8) = *reinterpret_cast<const uint32_t*>(q);
  }
  if (leader) {
    *d_out = d;
    *s_out = d * static_cast<float>(sum);
  }
}

// All global loads of a row are issued before the first dependent instruction, so a row costs
// about one memory round trip however few rows (CTAs) there are.
// Q8: also write the int8 view of the output rows (a separate instantiation: the extra values in
// flight would push the register-resident rows of the plain kernel into local memory).
// CH: 8-element chunks per thread (1 covers rows of up to 8192 values with 1024 threads: eight fp32
// values per thread instead of 32 leave the kernel free of spills).
template <bool Q8, int CH>
__global__ void __launch_bounds__(kNormMaxThreads) finalize_norm_kernel(const FinalizeNormParams p) {
  extern __shared__ float s_h[];  // N floats, used only by the MoE router path
  __shared__ float s_red[32];
  __shared__ int s_ok;
  pdl_launch_dependents();
  pdl_wait();  // the accumulators / slabs, the residual and the hand-off counters belong to earlier kernels
  const int N = p.N;
  const int nthr = blockDim.x;

  if (p.arrive != nullptr) {
    if (threadIdx.x == 0) {
      int ok = 1;
      uint32_t it = 0;
      const uint32_t limit = spin_budget(p.spin_limit);
      while (ld_acquire_sys_u32(p.arrive) < p.expected) {
        if (++it > limit) {
          set_status_peer_timeout(p.status);
          ok = 0;
          break;
        }
      }
      s_ok = ok;
    }
    __syncthreads();
    if (!s_ok) return;
  }

  // A CTA walks rows blockIdx.x, blockIdx.x + gridDim.x, ...: with many rows (prefill) the wait
  // above, the system fence and the signals below are paid once per CTA, not once per row.
  uint32_t rows_done = 0;
  for (int row = blockIdx.x; row < p.rows; row += gridDim.x, ++rows_done) {
  const long long roff = static_cast<long long>(row) * N;
  float h[CH][8];
  uint4 res[CH], bia[CH];
  // ---- phase 1: issue every load ----
#pragma unroll
  for (int ci = 0; ci < CH; ++ci) {
    const int c = (ci * nthr + threadIdx.x) * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) h[ci][j] = 0.f;
    res[ci] = make_uint4(0, 0, 0, 0);
    bia[ci] = make_uint4(0, 0, 0, 0);
    if (c >= N) continue;
    if (p.acc != nullptr) {
      const float4* a = reinterpret_cast<const float4*>(p.acc + roff + c);
      const float4 x0 = __ldcg(a), x1 = __ldcg(a + 1);
      h[ci][0] = x0.x; h[ci][1] = x0.y; h[ci][2] = x0.z; h[ci][3] = x0.w;
      h[ci][4] = x1.x; h[ci][5] = x1.y; h[ci][6] = x1.z; h[ci][7] = x1.w;
    }
    if (p.residual_in != nullptr) res[ci] = *reinterpret_cast<const uint4*>(p.residual_in + roff + c);
    if (p.bias != nullptr) bia[ci] = *reinterpret_cast<const uint4*>(p.bias + c);
  }
  if (p.rs_slab != nullptr) {
    // bf16 partial tiles from every source rank (written by peers): L2-coherent loads
    for (int sidx = 0; sidx < p.n_slabs; ++sidx) {
      uint4 v[CH];
#pragma unroll
      for (int ci = 0; ci < CH; ++ci) {
        const int c = (ci * nthr + threadIdx.x) * 8;
        v[ci] = make_uint4(0, 0, 0, 0);
        if (c < N)
          v[ci] = __ldcg(reinterpret_cast<const uint4*>(p.rs_slab + sidx * p.slab_stride + roff + c));
      }
#pragma unroll
      for (int ci = 0; ci < CH; ++ci) {
        const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&v[ci]);
#pragma unroll
        for (int j = 0; j < 8; ++j) h[ci][j] += __bfloat162float(e[j]);
      }
    }
  }
  // ---- phase 2: combine, re-arm the accumulator, residual out, sum of squares ----
  float ss = 0.f;
#pragma unroll
  for (int ci = 0; ci < CH; ++ci) {
    const int c = (ci * nthr + threadIdx.x) * 8;
    if (c >= N) continue;
    if (p.acc != nullptr) {
      float4* a = reinterpret_cast<float4*>(p.acc + roff + c);
      const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
      __stcg(a, z);
      __stcg(a + 1, z);
    }
    const __nv_bfloat16* rr = reinterpret_cast<const __nv_bfloat16*>(&res[ci]);
    const __nv_bfloat16* bb = reinterpret_cast<const __nv_bfloat16*>(&bia[ci]);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      h[ci][j] += __bfloat162float(rr[j]) + __bfloat162float(bb[j]);
      ss += h[ci][j] * h[ci][j];
    }
    if (p.residual_out != nullptr) {
      uint4 o;
      o.x = pack_bf16x2(h[ci][0], h[ci][1]);
      o.y = pack_bf16x2(h[ci][2], h[ci][3]);
      o.z = pack_bf16x2(h[ci][4], h[ci][5]);
      o.w = pack_bf16x2(h[ci][6], h[ci][7]);
      *reinterpret_cast<uint4*>(p.residual_out + roff + c) = o;
    }
  }
  float inv = 1.f;
  if (p.norm_w != nullptr) {
    const float tot = block_sum(ss, s_red);
    inv = rsqrtf(tot / static_cast<float>(N) + p.eps);
  }
  long long orow = p.out_row_off + row;
  if (p.out_row_map != nullptr) orow = p.out_row_map[row];
  const bool store_out = orow >= 0;
  const long long ooff = orow * static_cast<long long>(N);
#pragma unroll
  for (int ci = 0; ci < CH; ++ci) {
    const int c = (ci * nthr + threadIdx.x) * 8;
    if (c >= N) continue;
    float y[8];
    if (p.norm_w != nullptr) {
      const uint4 w = *reinterpret_cast<const uint4*>(p.norm_w + c);
      const __nv_bfloat16* ww = reinterpret_cast<const __nv_bfloat16*>(&w);
#pragma unroll
      for (int j = 0; j < 8; ++j) y[j] = h[ci][j] * inv * (__bfloat162float(ww[j]) + p.w_offset);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) y[j] = h[ci][j];
    }
    if (p.router_w != nullptr) {
#pragma unroll
      for (int j = 0; j < 8; ++j) s_h[c + j] = y[j];  // kept for the router and the dispatch
      continue;
    }
    uint4 o;
    o.x = pack_bf16x2(y[0], y[1]);
    o.y = pack_bf16x2(y[2], y[3]);
    o.z = pack_bf16x2(y[4], y[5]);
    o.w = pack_bf16x2(y[6], y[7]);
#pragma unroll
    for (int d = 0; d < kMaxPeers; ++d)
      if (d < p.n_dst && store_out) *reinterpret_cast<uint4*>(p.out[d] + ooff + c) = o;
    if constexpr (Q8) {
      if (store_out) {
        const long long blk = orow * static_cast<long long>(N >> 5) + (c >> 5);
        q8_block_store<8>(y, p.q8 + ooff + c, p.q8_d + blk, p.q8_s + blk, (c & 31) == 0);
      }
    }
  }

  if (p.router_w != nullptr) {
    // ---- router: logits over all experts, top-k, softmax over the selected logits ----
    __shared__ float s_logit[64];
    __shared__ int s_sel[8];
    __shared__ float s_wgt[8];
    __shared__ int s_slot[8];
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    for (int e = warp; e < p.n_experts; e += nw) {
      const __nv_bfloat16* wr = p.router_w + static_cast<long long>(e) * N;
      float s = 0.f;
      for (int c = lane * 8; c < N; c += 32 * 8) {
        const uint4 w = *reinterpret_cast<const uint4*>(wr + c);
        const __nv_bfloat16* ww = reinterpret_cast<const __nv_bfloat16*>(&w);
#pragma unroll
        for (int j = 0; j < 8; ++j) s += s_h[c + j] * __bfloat162float(ww[j]);
      }
      s = warp_sum(s);
      if (lane == 0) s_logit[e] = s;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float mx = -INFINITY;
      for (int k = 0; k < p.top_k; ++k) {
        int best = 0;
        float bv = -INFINITY;
        for (int e = 0; e < p.n_experts; ++e) {
          bool taken = false;
          for (int t = 0; t < k; ++t) taken |= s_sel[t] == e;
          if (!taken && s_logit[e] > bv) {
            bv = s_logit[e];
            best = e;
          }
        }
        s_sel[k] = best;
        s_wgt[k] = bv;
        mx = fmaxf(mx, bv);
      }
      float sum = 0.f;
      for (int k = 0; k < p.top_k; ++k) {
        s_wgt[k] = __expf(s_wgt[k] - mx);
        sum += s_wgt[k];
      }
      for (int k = 0; k < p.top_k; ++k) s_wgt[k] = s_wgt[k] / sum * p.routed_scale;
    }
    __syncthreads();
    // ---- claim a slab row on each selected expert's owner (remote atomic) and record the way home
    if (threadIdx.x < p.top_k) {
      const int k = threadIdx.x;
      const int e = s_sel[k];
      const int o = e / p.experts_per_rank, el = e - o * p.experts_per_rank;
      uint32_t* cnt = nullptr;
      MoeRowMeta* meta = nullptr;
#pragma unroll
      for (int d = 0; d < kMaxPeers; ++d)
        if (d == o) {
          cnt = p.slab_cnt[d];
          meta = p.meta[d];
        }
      int slot = static_cast<int>(atomicAdd(cnt + el, 1u));
      if (slot >= p.cap) {
        set_status_once(p.status, kStatusBadIndex);
        slot = -1;
      } else {
        MoeRowMeta m;
        m.rank = p.my_rank;
        m.row = row;
        m.weight = s_wgt[k];
        m.pad = 0;
        meta[static_cast<long long>(el) * p.cap + slot] = m;
      }
      s_slot[k] = slot;
    }
    __syncthreads();
    for (int k = 0; k < p.top_k; ++k) {
      const int slot = s_slot[k];
      if (slot < 0) continue;
      const int e = s_sel[k];
      const int o = e / p.experts_per_rank, el = e - o * p.experts_per_rank;
      __nv_bfloat16* base = nullptr;
#pragma unroll
      for (int d = 0; d < kMaxPeers; ++d)
        if (d == o) base = p.slab[d];
      __nv_bfloat16* drow = base + (static_cast<long long>(el) * p.cap + slot) * N;
      for (int c = threadIdx.x * 8; c < N; c += blockDim.x * 8) {
        uint4 o4;
        o4.x = pack_bf16x2(s_h[c], s_h[c + 1]);
        o4.y = pack_bf16x2(s_h[c + 2], s_h[c + 3]);
        o4.z = pack_bf16x2(s_h[c + 4], s_h[c + 5]);
        o4.w = pack_bf16x2(s_h[c + 6], s_h[c + 7]);
        *reinterpret_cast<uint4*>(drow + c) = o4;
      }
    }
  }

  __syncthreads();  // shared scratch (s_red, router state) is reused by the next row
  }                 // row loop

  const bool signal = p.out_flag[0] != nullptr;
  if (signal || p.arrive != nullptr) {
    __syncthreads();
    if (threadIdx.x == 0) {
      if (signal) {
        // one system-scope fence per CTA, after the barrier that orders every thread's stores;
        // the flags count rows, so this CTA adds the number of rows it pushed
        __threadfence_system();
#pragma unroll
        for (int d = 0; d < kMaxPeers; ++d)
          if (d < p.n_dst) red_relaxed_sys_add_u32(p.out_flag[d], rows_done);
      }
      if (p.arrive != nullptr) {
        // every CTA has passed its wait once the ticket is full: re-arm the arrival counter
        const uint32_t old = atomicAdd(p.ticket, 1u);
        if (old == gridDim.x - 1) {
          *const_cast<uint32_t*>(p.arrive) = 0;
          __threadfence();
          *p.ticket = 0;
        }
      }
    }
  }
}

// One CTA per token. Thread i handles rotation pair (d, d + D/2) of some head.
__global__ void __launch_bounds__(256) qkv_rope_append_kernel(const QkvRopeParams p) {
  extern __shared__ float s_row[];  // this CTA's heads: heads_per_cta * D floats
  __shared__ float s_ssq[160];      // per-head reciprocal RMS (indexed by the head's position in this CTA)
  __shared__ float s_sin[128], s_cos[128];  // the token's rotation, shared by every head (D <= 256)
  pdl_launch_dependents();
  pdl_wait();  // the QKV rows come from the kernel before this one
  const int tok = blockIdx.x;
  const int D = p.D, half = D >> 1;
  const int n_heads = p.Hq + 2 * p.Hkv;  // Q heads, then K heads, then V heads
  const int W = n_heads * D;
  // blockIdx.y selects a contiguous range of heads, so that few tokens still fill the SMs
  const int hpc = (n_heads + gridDim.y - 1) / gridDim.y;
  const int h_lo = blockIdx.y * hpc;
  const int h_hi = h_lo + hpc < n_heads ? h_lo + hpc : n_heads;
  if (h_lo >= h_hi) return;
  const int c_lo = h_lo * D, c_hi = h_hi * D;
  const long long roff = static_cast<long long>(tok) * W;
  const int pos = p.positions[tok];
  const int n_rot_heads = p.Hq + p.Hkv;
  if (h_lo < n_rot_heads) {
    // one precise sincos per frequency and token instead of one per (head, frequency)
    for (int d = threadIdx.x; d < half; d += blockDim.x) {
      float sn, cs;
      sincosf(static_cast<float>(pos) * p.inv_freq[d], &sn, &cs);
      s_sin[d] = sn * p.rope_mscale;
      s_cos[d] = cs * p.rope_mscale;
    }
  }

  for (int c = c_lo + threadIdx.x * 4; c < c_hi; c += blockDim.x * 4) {
    float v[4];
    if (p.acc_f32 != nullptr) {
      float4* a = reinterpret_cast<float4*>(const_cast<float*>(p.acc_f32) + roff + c);
      const float4 x = __ldcg(a);
      v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
      __stcg(a, make_float4(0.f, 0.f, 0.f, 0.f));
    } else {
      const uint2 x = *reinterpret_cast<const uint2*>(p.qkv_bf16 + roff + c);
      const __nv_bfloat16* xx = reinterpret_cast<const __nv_bfloat16*>(&x);
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = __bfloat162float(xx[j]);
    }
    if (p.bias != nullptr) {
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] += __bfloat162float(p.bias[c + j]);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) s_row[c - c_lo + j] = v[j];
  }
  __syncthreads();

  const int r_hi = h_hi < n_rot_heads ? h_hi : n_rot_heads;  // rotated heads of this CTA: [h_lo, r_hi)
  const bool qk_norm = p.q_norm_w != nullptr;
  if (qk_norm) {
    // one warp per head computes the head's mean square
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    for (int h = h_lo + warp; h < r_hi; h += nw) {
      float ss = 0.f;
      for (int d = lane; d < D; d += 32) {
        const float x = s_row[(h - h_lo) * D + d];
        ss += x * x;
      }
      ss = warp_sum(ss);
      if (lane == 0) s_ssq[h - h_lo] = rsqrtf(ss / static_cast<float>(D) + p.norm_eps);
    }
    __syncthreads();
  }

  const long long slot = p.slot_mapping[tok];
  const bool store_kv = slot >= 0 && slot < p.num_slots;
  if (slot >= p.num_slots && threadIdx.x == 0 && blockIdx.y == 0) set_status_once(p.status, kStatusBadIndex);
  const long long blk = slot >> 4;
  const int off = static_cast<int>(slot & 15);

  // rotate Q and K heads
  for (int i = threadIdx.x; i < (r_hi - h_lo) * half; i += blockDim.x) {
    const int lh = i / half, d = i - lh * half;
    const int h = h_lo + lh;
    float x0 = s_row[lh * D + d], x1 = s_row[lh * D + d + half];
    if (qk_norm) {
      const __nv_bfloat16* w = h < p.Hq ? p.q_norm_w : p.k_norm_w;
      const float r = s_ssq[lh];
      x0 = x0 * r * (__bfloat162float(w[d]) + p.norm_w_offset);
      x1 = x1 * r * (__bfloat162float(w[d + half]) + p.norm_w_offset);
    }
    const float sn = s_sin[d], cs = s_cos[d];
    const float y0 = x0 * cs - x1 * sn;
    const float y1 = x1 * cs + x0 * sn;
    if (h < p.Hq) {
      __nv_bfloat16* q = p.q_out + static_cast<long long>(tok) * p.Hq * D + h * D;
      q[d] = __float2bfloat16(y0);
      q[d + half] = __float2bfloat16(y1);
    } else if (store_kv) {
      const int kh = h - p.Hq;
      __nv_bfloat16* k = p.k_cache + ((blk * p.Hkv + kh) * 16 + off) * D;
      k[d] = __float2bfloat16(y0);
      k[d + half] = __float2bfloat16(y1);
    }
  }
  if (store_kv && h_hi > n_rot_heads) {
    // V heads of this CTA: [max(h_lo, n_rot_heads), h_hi)
    const int v_lo = h_lo > n_rot_heads ? h_lo : n_rot_heads;
    for (int i = threadIdx.x; i < (h_hi - v_lo) * D; i += blockDim.x) {
      const int lv = i / D, d = i - lv * D;
      const int kh = v_lo + lv - n_rot_heads;
      p.v_cache[((blk * p.Hkv + kh) * 16 + off) * D + d] = __float2bfloat16(s_row[(v_lo + lv - h_lo) * D + d]);
    }
  }
}

__global__ void swiglu_kernel(const SwigluParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const long long total = static_cast<long long>(p.M) * p.I / 4;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long e = i * 4;
    const long long m = e / p.I;
    const int c = static_cast<int>(e - m * p.I);
    float gt[4], up[4];
    if (p.acc_f32 != nullptr) {
      float4* ga = reinterpret_cast<float4*>(const_cast<float*>(p.acc_f32) + m * 2 * p.I + c);
      float4* ua = reinterpret_cast<float4*>(const_cast<float*>(p.acc_f32) + m * 2 * p.I + p.I + c);
      const float4 gv = __ldcg(ga), uv = __ldcg(ua);
      gt[0] = gv.x; gt[1] = gv.y; gt[2] = gv.z; gt[3] = gv.w;
      up[0] = uv.x; up[1] = uv.y; up[2] = uv.z; up[3] = uv.w;
      const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
      __stcg(ga, z);
      __stcg(ua, z);
    } else {
      const uint2 gv = *reinterpret_cast<const uint2*>(p.gu_bf16 + m * 2 * p.I + c);
      const uint2 uv = *reinterpret_cast<const uint2*>(p.gu_bf16 + m * 2 * p.I + p.I + c);
      const __nv_bfloat16* gg = reinterpret_cast<const __nv_bfloat16*>(&gv);
      const __nv_bfloat16* uu = reinterpret_cast<const __nv_bfloat16*>(&uv);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        gt[j] = __bfloat162float(gg[j]);
        up[j] = __bfloat162float(uu[j]);
      }
    }
    float y[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float a;
      if (p.act == 0) {
        a = gt[j] / (1.f + __expf(-gt[j]));
      } else {
        const float x = gt[j];
        a = 0.5f * x * (1.f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
      }
      y[j] = a * up[j];
    }
    uint2 o;
    o.x = pack_bf16x2(y[0], y[1]);
    o.y = pack_bf16x2(y[2], y[3]);
    *reinterpret_cast<uint2*>(p.out + m * p.I + c) = o;
    if (p.q8 != nullptr) {
      const long long blk = m * (p.I >> 5) + (c >> 5);
      q8_block_store<4>(y, p.q8 + m * p.I + c, p.q8_d + blk, p.q8_s + blk, (c & 31) == 0);
    }
  }
}

__global__ void embed_gather_kernel(const int* tokens, const __nv_bfloat16* table,
                                    __nv_bfloat16* out, int N, int vocab, float scale,
                                    int vocab_start) {
  const int row = blockIdx.x;
  const int tok = tokens[row] - vocab_start;
  const bool valid = tok >= 0 && tok < vocab;  // vocab-parallel: rows of other shards give zeros
  const __nv_bfloat16* src = table + static_cast<long long>(valid ? tok : 0) * N;
  __nv_bfloat16* dst = out + static_cast<long long>(row) * N;
  for (int c = threadIdx.x * 8; c < N; c += blockDim.x * 8) {
    uint4 v = valid ? *reinterpret_cast<const uint4*>(src + c) : make_uint4(0, 0, 0, 0);
    if (scale != 1.f && valid) {
      __nv_bfloat16* e = reinterpret_cast<__nv_bfloat16*>(&v);
#pragma unroll
      for (int j = 0; j < 8; ++j) e[j] = __float2bfloat16(__bfloat162float(e[j]) * scale);
    }
    *reinterpret_cast<uint4*>(dst + c) = v;
  }
}

__global__ void cast_acc_bf16_kernel(float* acc, const __nv_bfloat16* bias, __nv_bfloat16* out,
                                     int M, int N, long long ldo) {
  const long long total = static_cast<long long>(M) * N / 4;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long e = i * 4;
    const long long m = e / N;
    const int c = static_cast<int>(e - m * N);
    float4* a = reinterpret_cast<float4*>(acc + e);
    float4 v = __ldcg(a);
    __stcg(a, make_float4(0.f, 0.f, 0.f, 0.f));
    if (bias != nullptr) {
      v.x += __bfloat162float(bias[c]);
      v.y += __bfloat162float(bias[c + 1]);
      v.z += __bfloat162float(bias[c + 2]);
      v.w += __bfloat162float(bias[c + 3]);
    }
    uint2 o;
    o.x = pack_bf16x2(v.x, v.y);
    o.y = pack_bf16x2(v.z, v.w);
    *reinterpret_cast<uint2*>(out + m * ldo + c) = o;
  }
}

// 128-point Walsh-Hadamard transform per block of 128 floats, scaled by 1/sqrt(128).
__global__ void __launch_bounds__(128) fwht128_kernel(float* x, long long n_blocks) {
  __shared__ float s[128];
  for (long long b = blockIdx.x; b < n_blocks; b += gridDim.x) {
    s[threadIdx.x] = x[b * 128 + threadIdx.x];
    __syncthreads();
#pragma unroll
    for (int h = 1; h < 128; h <<= 1) {
      const int i = threadIdx.x;
      const float a = s[i & ~h], c = s[i | h];
      __syncthreads();
      s[i] = (i & h) ? a - c : a + c;
      __syncthreads();
    }
    x[b * 128 + threadIdx.x] = s[threadIdx.x] * 0.08838834764831845f;
    __syncthreads();
  }
}

// Copies whole KV blocks (copy-on-write of a shared partial block, context-shift compaction).
__global__ void kv_block_copy_kernel(__nv_bfloat16* k_cache, __nv_bfloat16* v_cache,
                                     const int* src_blocks, const int* dst_blocks,
                                     long long block_elems) {
  const int pair = blockIdx.x;
  const long long s = static_cast<long long>(src_blocks[pair]) * block_elems;
  const long long d = static_cast<long long>(dst_blocks[pair]) * block_elems;
  __nv_bfloat16* base = blockIdx.y == 0 ? k_cache : v_cache;
  for (long long i = threadIdx.x * 8; i < block_elems; i += blockDim.x * 8)
    *reinterpret_cast<uint4*>(base + d + i) = *reinterpret_cast<const uint4*>(base + s + i);
}

__global__ void softcap_kernel(float* x, long long n, float cap) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    x[i] = cap * tanhf(x[i] / cap);
}

// Reference counterpart: advance_decode_step_kernel (oxide-backend-cuda/src/kernels/megakernel_ops.cu:331-357)
// and the pinned step counter the host spins on (oxide-backend-cuda/src/lib.rs:4150-4247).
__global__ void advance_decode_step_kernel(const AdvanceStepParams p) {
  __shared__ unsigned int s_step;
  if (threadIdx.x == 0) s_step = *p.step_counter + 1;
  __syncthreads();
  const unsigned int step = s_step;
  for (int r = threadIdx.x; r < p.rows; r += blockDim.x) {
    const int tok = p.sampled[r];
    if (p.seq_lens[r] > 0) {  // padding rows of the batch bucket stay as they are
      const int pos = p.positions[r] + 1;
      const int blk = pos >> 4;
      if (blk >= p.max_blocks) {
        if (p.status != nullptr) atomicCAS(p.status, 0, kStatusBadIndex);
      } else {
        p.token_ids[r] = tok;
        p.positions[r] = pos;
        p.seq_lens[r] += 1;
        p.slot_mapping[r] = static_cast<long long>(p.block_tables[static_cast<long long>(r) * p.max_blocks + blk]) * 16 + (pos & 15);
      }
    }
    p.mailbox[static_cast<size_t>((step - 1) % p.ring) * p.rows + r] =
        (static_cast<unsigned long long>(step) << 32) | static_cast<unsigned int>(tok);
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) *p.step_counter = step;
}

}  // namespace

void launch_advance_decode_step(const AdvanceStepParams& p, cudaStream_t stream) {
  if (p.rows <= 0) return;
  advance_decode_step_kernel<<<1, 256, 0, stream>>>(p);
}

void launch_finalize_norm(const FinalizeNormParams& p, cudaStream_t stream) {
  if (p.rows <= 0) return;
  // threads: one 8-element chunk per thread up to 1024 threads, then several chunks per thread
  int threads = (p.N / 8 + 31) / 32 * 32;
  if (threads > kNormMaxThreads) threads = kNormMaxThreads;
  if (threads < 32) threads = 32;
  const size_t smem = p.router_w != nullptr ? static_cast<size_t>(p.N) * sizeof(float) : 0;
  const bool one = static_cast<long long>(threads) * 8 >= p.N;  // one chunk per thread covers the row
  ensure_dynamic_smem(finalize_norm_kernel<false, 1>, smem);
  ensure_dynamic_smem(finalize_norm_kernel<true, 1>, smem);
  ensure_dynamic_smem(finalize_norm_kernel<false, kNormMaxChunks>, smem);
  ensure_dynamic_smem(finalize_norm_kernel<true, kNormMaxChunks>, smem);
  // a CTA loops over rows, so any grid is correct; two CTAs per SM keep a second row's loads in
  // flight where registers allow two resident CTAs, and cost nothing where they do not
  const int max_ctas = 2 * sm_count();
  const int grid = p.rows < max_ctas ? p.rows : max_ctas;
  if (p.q8 != nullptr && one)
    launch_kernel(finalize_norm_kernel<true, 1>, dim3(grid), dim3(threads), smem, stream, /*pdl=*/true, false, p);
  else if (p.q8 != nullptr)
    launch_kernel(finalize_norm_kernel<true, kNormMaxChunks>, dim3(grid), dim3(threads), smem, stream, true, false, p);
  else if (one)
    launch_kernel(finalize_norm_kernel<false, 1>, dim3(grid), dim3(threads), smem, stream, /*pdl=*/true, false, p);
  else
    launch_kernel(finalize_norm_kernel<false, kNormMaxChunks>, dim3(grid), dim3(threads), smem, stream, true, false, p);
}

void launch_qkv_rope_append(const QkvRopeParams& p, cudaStream_t stream) {
  if (p.M <= 0) return;
  // heads are split over blockIdx.y until about two CTAs per SM exist (a step of 64 tokens would
  // otherwise leave more than half of the SMs idle); a CTA keeps at least 4 heads
  const int n_heads = p.Hq + 2 * p.Hkv;
  int chunks = (2 * sm_count() + p.M - 1) / p.M;
  if (chunks > n_heads / 4) chunks = n_heads / 4;
  if (chunks < 1) chunks = 1;
  const int hpc = (n_heads + chunks - 1) / chunks;
  chunks = (n_heads + hpc - 1) / hpc;
  const size_t smem = static_cast<size_t>(hpc) * p.D * sizeof(float);
  ensure_dynamic_smem(qkv_rope_append_kernel, smem);
  launch_kernel(qkv_rope_append_kernel, dim3(p.M, chunks), dim3(256), smem, stream, /*pdl=*/true, false, p);
}

void launch_swiglu(const SwigluParams& p, cudaStream_t stream) {
  const long long total = static_cast<long long>(p.M) * p.I / 4;
  if (total <= 0) return;
  int blocks = static_cast<int>((total + 255) / 256);
  if (blocks > sm_count() * 16) blocks = sm_count() * 16;
  launch_kernel(swiglu_kernel, dim3(blocks), dim3(256), 0, stream, /*pdl=*/true, false, p);
}

void launch_embed_gather(const int* tokens, const __nv_bfloat16* table, __nv_bfloat16* out, int M,
                         int N, int vocab, float scale, int vocab_start, cudaStream_t stream) {
  if (M <= 0) return;
  embed_gather_kernel<<<M, 256, 0, stream>>>(tokens, table, out, N, vocab, scale, vocab_start);
}

void launch_cast_acc_bf16(float* acc, const __nv_bfloat16* bias, __nv_bfloat16* out, int M, int N,
                          long long ldo, cudaStream_t stream) {
  const long long total = static_cast<long long>(M) * N / 4;
  if (total <= 0) return;
  int blocks = static_cast<int>((total + 255) / 256);
  if (blocks > sm_count() * 16) blocks = sm_count() * 16;
  cast_acc_bf16_kernel<<<blocks, 256, 0, stream>>>(acc, bias, out, M, N, ldo);
}

void launch_fwht128(float* x, long long n_blocks, cudaStream_t stream) {
  if (n_blocks <= 0) return;
  int blocks = n_blocks > sm_count() * 8 ? sm_count() * 8 : static_cast<int>(n_blocks);
  fwht128_kernel<<<blocks, 128, 0, stream>>>(x, n_blocks);
}

void launch_kv_block_copy(__nv_bfloat16* k_cache, __nv_bfloat16* v_cache, const int* src_blocks,
                          const int* dst_blocks, int n_pairs, long long block_elems,
                          cudaStream_t stream) {
  if (n_pairs <= 0) return;
  kv_block_copy_kernel<<<dim3(n_pairs, 2), 256, 0, stream>>>(k_cache, v_cache, src_blocks,
                                                            dst_blocks, block_elems);
}

void launch_softcap(float* logits, long long n, float cap, cudaStream_t stream) {
  if (n <= 0) return;
  int blocks = static_cast<int>((n + 255) / 256);
  if (blocks > sm_count() * 16) blocks = sm_count() * 16;
  softcap_kernel<<<blocks, 256, 0, stream>>>(logits, n, cap);
}

}  // namespace oxb
