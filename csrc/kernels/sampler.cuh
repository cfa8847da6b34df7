#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace oxb {

struct SampleParams {
  const float* logits;  // [rows, V], row stride ld
  long long ld;
  int V;
  const float* temperature;    // [rows]; <= 0 selects greedy
  const int* top_k;            // [rows]; <= 0 disables
  const float* top_p;          // [rows]
  const float* min_p;          // [rows]
  const uint64_t* seeds;       // [rows]
  const uint64_t* counters;    // [rows] draw index of the sequence (for reproducible streams)
  const uint32_t* allow_mask;  // [rows, mask_words] bit = 1 allowed; nullptr = everything
  int mask_words;
  int* out_tokens;   // [rows]
  float* out_logit;  // [rows] nullable: max logit (greedy) or log-prob of the pick
};

void launch_sample(const SampleParams& p, int rows, cudaStream_t stream);
void launch_argmax(const float* logits, long long ld, int V, int rows, int* out, float* out_val,
                   cudaStream_t stream);
void launch_argmax_combine(const float* vals, const int* idxs, int ranks, int B, int* out,
                           cudaStream_t stream);

}  // namespace oxb
