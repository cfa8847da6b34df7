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

// Vocab-parallel greedy sampling over peer memory, no library collective: every rank takes the argmax
// of its vocabulary shard and stores ONE 64-bit word per row, (ordered value << 32) | ~index, into the
// table of every rank (`tab[o]` = rank o's table, [2 slots][ranks][max_rows] words, zero = empty). A word
// is its own flag, so no fence and no separate signal are needed; the combine kernel waits (bounded,
// kStatusPeerFlagTimeout in *status on expiry) until the words of all ranks of the row are there, picks
// the largest value (lowest index on ties), writes the token and clears the words for the slot's next use.
struct ArgmaxExchangeParams {
  const float* logits;   // [rows, V_local], row stride ld
  long long ld;
  int V_local, vocab_start, rows, max_rows, ranks, my_rank, slot;
  unsigned long long* tab[8];
  int* out_tokens;       // [rows]
  int* status;
  uint32_t spin_limit;
};
void launch_argmax_exchange(const ArgmaxExchangeParams& p, cudaStream_t stream);

}  // namespace oxb
