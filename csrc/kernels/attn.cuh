// Parameter blocks of the paged attention kernels.
// KV cache layout (per layer): [num_blocks, Hkv, 16 tokens, head_dim] bf16 for K and for V.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace oxb {

struct DecodeAttnParams {
  const __nv_bfloat16* q;  // [B, Hq, D], row stride q_stride (elements)
  long long q_stride;
  const __nv_bfloat16* k_cache;
  const __nv_bfloat16* v_cache;
  const int* block_tables;     // [B, max_blocks]
  const int* seq_lens;         // [B] context length including the current token
  const int* pages_per_split;  // device scalar, >= 1
  float* part_o;               // [B, Hq, max_splits, D]
  float* part_ml;              // [B, Hq, max_splits, 2]  (running max in log2 units, sum)
  __nv_bfloat16* out;          // [B, Hq*D], row stride out_stride
  long long out_stride;
  int max_blocks, Hq, Hkv, max_splits, window;
  float scale_log2;  // softmax scale * log2(e)
  // Bounds check of block-table entries: an id outside [0, num_blocks) is recorded in *status
  // (kStatusBadIndex) and page 0 is read instead. num_blocks <= 0 or status == nullptr: no check.
  int num_blocks;
  int* status;
  // Heavy-hitter statistics (optional, both or neither): the split kernel records for every attended
  // page and query head the pair (reference max in log2 units, sum of 2^(x - max) over the page's 16
  // tokens) in page_ml [B, max_blocks, Hq, 2]; after the merge a third kernel turns them into
  // block_mass [B, max_blocks] = sum over heads of the softmax probability that fell into the page
  // (0 for pages outside the attended range).
  float* page_ml;
  float* block_mass;
  // Optional int8 view of `out` for an integer GEMV that consumes it (blocks of 32 values with an
  // fp32 scale = amax / 127 and scale * sum): q8 [B, Hq*D] int8, q8_d / q8_s [B, Hq*D / 32], written
  // by the merge kernel.
  signed char* q8;
  float* q8_d;
  float* q8_s;
};

// Launches the split kernel and then the merge; the merge is skipped when the first launch failed.
// Coverage rule: pages_per_split * max_splits pages must cover the longest attended window, a
// split beyond max_splits does not exist and its tokens would be left out.
cudaError_t launch_paged_decode(const DecodeAttnParams& p, int batch, int head_dim, cudaStream_t stream);

struct PrefillAttnParams {
  const __nv_bfloat16* q;  // [T, Hq, D] ragged over sequences, row stride q_stride
  long long q_stride;
  const __nv_bfloat16* k_cache;
  const __nv_bfloat16* v_cache;
  const int* block_tables;  // [n_seqs, max_blocks]
  const int* tile_seq;      // [n_tiles] sequence of each 64-row query tile
  const int* tile_q0;       // [n_tiles] first query index of the tile inside its sequence
  const int* q_start;       // [n_seqs] first row of the sequence in q
  const int* q_lens;        // [n_seqs] query tokens of this chunk
  const int* ctx_lens;      // [n_seqs] context length after this chunk (KV tokens in the cache)
  __nv_bfloat16* out;       // [T, Hq*D], row stride out_stride
  long long out_stride;
  int max_blocks, Hq, Hkv, window;
  float scale_log2;
  int num_blocks;  // bound for block-table entries (<= 0: unchecked), violations go to *status
  int* status;
};

void launch_paged_prefill_tc(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV,
                             const PrefillAttnParams& p, int n_tiles, int head_dim, int* status,
                             cudaStream_t stream);

}  // namespace oxb
