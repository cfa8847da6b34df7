// Device sampler (sm_100a): per-row greedy argmax, and temperature / top-k / min-p / top-p
// sampling with an optional allow-bitmask (grammar, banned tokens).
//
// One CTA per row. Sampling path: 4-pass radix select of the C = max(top_k, 256) largest
// logits (C <= 1024) -> gather -> bitonic sort in shared memory -> softmax over the candidates
// -> min-p -> top-k -> top-p -> renormalise -> inverse-CDF draw from a counter-based RNG.
// The order of the filters is the reference's (oxide-core/src/sampler.rs:173-390, which
// also truncates to max(k,256) candidates before the softmax, sampler.rs:274-280).
// Replaces argmax_f32_kernel / argmax_stage1/2 (sampling_dfa.cu:2-159) and the Gumbel-max
// sample_stage1 kernel (sampling_dfa.cu:180-274), whose top_p argument is ignored.
#include "sampler.cuh"

#include <math.h>

#include "../common/sm100.cuh"

namespace oxb {

namespace {

constexpr int kThreads = 1024;
constexpr int kMaxCand = 1024;

__device__ __forceinline__ uint32_t f2key(float f) {
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ bool allowed(const uint32_t* mask, int i) {
  return mask == nullptr || ((mask[i >> 5] >> (i & 31)) & 1u);
}
__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

__device__ void block_argmax(const float* row, const uint32_t* mask, int V, int* out_idx,
                             float* out_val) {
  __shared__ float s_v[32];
  __shared__ int s_i[32];
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = allowed(mask, i) ? row[i] : -INFINITY;
    if (v > best || (v == best && i < bi)) {
      best = v;
      bi = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    s_v[warp] = best;
    s_i[warp] = bi;
  }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    best = lane < nw ? s_v[lane] : -INFINITY;
    bi = lane < nw ? s_i[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) {
        best = ov;
        bi = oi;
      }
    }
    if (lane == 0) {
      *out_idx = bi == 0x7fffffff ? 0 : bi;
      *out_val = best;
    }
  }
  __syncthreads();
}

__global__ void __launch_bounds__(kThreads) sample_kernel(const SampleParams p) {
  __shared__ int s_hist[256];
  __shared__ float s_val[kMaxCand];
  __shared__ int s_idx[kMaxCand];
  __shared__ int s_count, s_tok;
  __shared__ uint32_t s_prefix;
  __shared__ int s_remaining;
  __shared__ float s_best;

  const int row = blockIdx.x;
  const float* logits = p.logits + static_cast<long long>(row) * p.ld;
  const uint32_t* mask =
      p.allow_mask != nullptr ? p.allow_mask + static_cast<long long>(row) * p.mask_words : nullptr;
  const int V = p.V;
  const float temp = p.temperature != nullptr ? p.temperature[row] : 0.f;
  int top_k = p.top_k != nullptr ? p.top_k[row] : 0;
  const float top_p = p.top_p != nullptr ? p.top_p[row] : 1.f;
  const float min_p = p.min_p != nullptr ? p.min_p[row] : 0.f;

  if (temp <= 0.f || top_k == 1) {
    block_argmax(logits, mask, V, &s_tok, &s_best);
    if (threadIdx.x == 0) {
      p.out_tokens[row] = s_tok;
      if (p.out_logit != nullptr) p.out_logit[row] = s_best;
    }
    return;
  }
  if (top_k <= 0 || top_k > V) top_k = V;
  int C = top_k > 256 ? top_k : 256;
  if (C > kMaxCand) C = kMaxCand;
  if (C > V) C = V;

  // ---- radix select: key of the C-th largest allowed logit ----
  if (threadIdx.x == 0) {
    s_prefix = 0;
    s_remaining = C;
  }
  __syncthreads();
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    for (int i = threadIdx.x; i < 256; i += blockDim.x) s_hist[i] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix;
    const uint32_t pmask = pass == 0 ? 0u : (0xFFFFFFFFu << (32 - 8 * pass));
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      if (!allowed(mask, i)) continue;
      const uint32_t k = f2key(logits[i]);
      if ((k & pmask) == prefix) atomicAdd(&s_hist[(k >> shift) & 0xFF], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int rem = s_remaining;
      int b = 255;
      for (; b > 0; --b) {
        if (s_hist[b] >= rem) break;
        rem -= s_hist[b];
      }
      s_prefix = prefix | (static_cast<uint32_t>(b) << shift);
      s_remaining = rem;
    }
    __syncthreads();
  }
  const uint32_t kth = s_prefix;

  // ---- gather candidates: everything above the threshold, ties until C is reached ----
  if (threadIdx.x == 0) s_count = 0;
  for (int i = threadIdx.x; i < kMaxCand; i += blockDim.x) {
    s_val[i] = -INFINITY;
    s_idx[i] = 0x7fffffff;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    if (!allowed(mask, i)) continue;
    const float v = logits[i];
    if (f2key(v) > kth) {
      const int s = atomicAdd(&s_count, 1);
      if (s < kMaxCand) {
        s_val[s] = v;
        s_idx[s] = i;
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    if (!allowed(mask, i)) continue;
    const float v = logits[i];
    if (f2key(v) == kth) {
      const int s = atomicAdd(&s_count, 1);
      if (s < C) {
        s_val[s] = v;
        s_idx[s] = i;
      }
    }
  }
  __syncthreads();
  int n = s_count < C ? s_count : C;

  // ---- bitonic sort, descending by value then ascending by index (deterministic) ----
  for (int k = 2; k <= kMaxCand; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      const int i = threadIdx.x;
      const int ixj = i ^ j;
      if (ixj > i) {
        const float a = s_val[i], b = s_val[ixj];
        const int ia = s_idx[i], ib = s_idx[ixj];
        const bool a_first = a > b || (a == b && ia < ib);  // a sorts before b
        const bool up = (i & k) == 0;
        if (up ? !a_first : a_first) {
          s_val[i] = b;
          s_val[ixj] = a;
          s_idx[i] = ib;
          s_idx[ixj] = ia;
        }
      }
      __syncthreads();
    }
  }

  // ---- with top-k off the candidates are only the 1024 largest logits: the softmax denominator
  // (what top-p and the reported log-probability are measured against) is taken over every allowed
  // logit, so the thresholds are those of the full distribution ----
  const bool full_mass = top_k >= V && V > C;
  if (full_mass && n > 0) {
    const float inv_t = 1.f / temp;
    const float mx = s_val[0] * inv_t;
    float part = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x)
      if (allowed(mask, i)) part += __expf(logits[i] * inv_t - mx);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    float* s_part = reinterpret_cast<float*>(s_hist);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = part;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int w = 0; w < (blockDim.x >> 5); ++w) t += s_part[w];
      s_best = t;
    }
    __syncthreads();
  }

  // ---- filters and draw (serial over <= 1024 sorted candidates) ----
  if (threadIdx.x == 0) {
    if (n <= 0) {
      p.out_tokens[row] = 0;
      return;
    }
    const float inv_t = 1.f / temp;
    const float mx = s_val[0] * inv_t;
    float sum = 0.f;
    for (int i = 0; i < n; ++i) {
      const float e = __expf(s_val[i] * inv_t - mx);
      s_val[i] = e;
      sum += e;
    }
    if (full_mass) sum = fmaxf(sum, s_best);
    // min-p: keep probabilities >= min_p * p_max (p_max is candidate 0)
    int keep = n;
    if (min_p > 0.f) {
      const float thr = min_p * s_val[0];
      int c = 0;
      while (c < n && s_val[c] >= thr) ++c;
      keep = c > 0 ? c : 1;
    }
    if (top_k < keep) keep = top_k;
    // top-p: cumulative mass of the candidate softmax (not renormalised after min-p / top-k,
    // as in the reference pipeline)
    if (top_p < 1.f) {
      float cum = 0.f;
      int c = 0;
      while (c < keep) {
        cum += s_val[c] / sum;
        ++c;
        if (cum >= top_p) break;
      }
      keep = c > 0 ? c : 1;
    }
    float tot = 0.f;
    for (int i = 0; i < keep; ++i) tot += s_val[i];
    const uint64_t seed = p.seeds != nullptr ? p.seeds[row] : 0ull;
    const uint64_t ctr = p.counters != nullptr ? p.counters[row] : 0ull;
    const uint64_t r = splitmix64(seed ^ splitmix64(ctr + 0x51ED2701ull));
    const float u = static_cast<float>(r >> 40) * (1.0f / 16777216.0f);
    const float target = u * tot;
    float cum = 0.f;
    int pick = keep - 1;
    for (int i = 0; i < keep; ++i) {
      cum += s_val[i];
      if (cum > target) {
        pick = i;
        break;
      }
    }
    p.out_tokens[row] = s_idx[pick];
    if (p.out_logit != nullptr) p.out_logit[row] = logf(s_val[pick] / sum);
  }
}

__global__ void __launch_bounds__(kThreads) argmax_kernel(const float* logits, long long ld, int V,
                                                          int* out, float* out_val) {
  __shared__ int s_tok;
  __shared__ float s_best;
  block_argmax(logits + static_cast<long long>(blockIdx.x) * ld, nullptr, V, &s_tok, &s_best);
  if (threadIdx.x == 0) {
    out[blockIdx.x] = s_tok;
    if (out_val != nullptr) out_val[blockIdx.x] = s_best;
  }
}

// Vocab-parallel argmax: combine per-rank (value, index) pairs gathered as [ranks, B].
__global__ void argmax_combine_kernel(const float* vals, const int* idxs, int ranks, int B,
                                      int* out) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  float best = -INFINITY;
  int bi = 0;
  for (int r = 0; r < ranks; ++r) {
    const float v = vals[r * B + b];
    const int i = idxs[r * B + b];
    if (v > best || (v == best && i < bi)) {
      best = v;
      bi = i;
    }
  }
  out[b] = bi;
}

__global__ void __launch_bounds__(kThreads) argmax_push_kernel(const ArgmaxExchangeParams p) {
  __shared__ int s_tok;
  __shared__ float s_best;
  const int row = blockIdx.x;
  block_argmax(p.logits + static_cast<long long>(row) * p.ld, nullptr, p.V_local, &s_tok, &s_best);
  if (threadIdx.x == 0) {
    const unsigned long long word = (static_cast<unsigned long long>(f2key(s_best)) << 32) |
                                    (0xFFFFFFFFu - static_cast<uint32_t>(s_tok + p.vocab_start));
    const size_t off = (static_cast<size_t>(p.slot) * p.ranks + p.my_rank) * p.max_rows + row;
#pragma unroll
    for (int o = 0; o < 8; ++o)
      if (o < p.ranks)
        asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p.tab[o] + off), "l"(word) : "memory");
  }
}

__global__ void argmax_collect_kernel(const ArgmaxExchangeParams p) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= p.rows) return;
  unsigned long long* mine = p.tab[p.my_rank] + static_cast<size_t>(p.slot) * p.ranks * p.max_rows + row;
  const uint32_t limit = p.spin_limit != 0 ? p.spin_limit : (1u << 22);
  unsigned long long best = 0;
  for (int r = 0; r < p.ranks; ++r) {
    unsigned long long* w = mine + static_cast<size_t>(r) * p.max_rows;
    unsigned long long v = 0;
    uint32_t it = 0;
    while (true) {
      asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(w) : "memory");
      if (v != 0) break;
      if (++it > limit) {
        if (p.status != nullptr) atomicCAS(p.status, 0, 4 /* kStatusPeerFlagTimeout */);
        break;
      }
    }
    if (v > best) best = v;
    *w = 0;  // empty again for the slot's next use (two steps from now)
  }
  p.out_tokens[row] = best != 0 ? static_cast<int>(0xFFFFFFFFu - static_cast<uint32_t>(best & 0xFFFFFFFFull)) : 0;
}

}  // namespace

void launch_argmax_exchange(const ArgmaxExchangeParams& p, cudaStream_t stream) {
  if (p.rows <= 0) return;
  argmax_push_kernel<<<p.rows, kThreads, 0, stream>>>(p);
  argmax_collect_kernel<<<(p.rows + 127) / 128, 128, 0, stream>>>(p);
}

void launch_sample(const SampleParams& p, int rows, cudaStream_t stream) {
  if (rows <= 0) return;
  sample_kernel<<<rows, kThreads, 0, stream>>>(p);
}
void launch_argmax(const float* logits, long long ld, int V, int rows, int* out, float* out_val,
                   cudaStream_t stream) {
  if (rows <= 0) return;
  argmax_kernel<<<rows, kThreads, 0, stream>>>(logits, ld, V, out, out_val);
}
void launch_argmax_combine(const float* vals, const int* idxs, int ranks, int B, int* out,
                           cudaStream_t stream) {
  if (B <= 0) return;
  argmax_combine_kernel<<<(B + 127) / 128, 128, 0, stream>>>(vals, idxs, ranks, B, out);
}

}  // namespace oxb
