#include "block_manager.h"

#include <algorithm>
#include <numeric>

namespace oxb {

std::vector<int> SequenceBlockTable::prune_heavy_hitters(const std::vector<float>& scores,
                                                         int sink_blocks, int rolling_blocks,
                                                         int budget_blocks) {
  const int n = static_cast<int>(blocks_.size());
  std::vector<int> keep;
  if (n <= budget_blocks) {
    keep.resize(n);
    std::iota(keep.begin(), keep.end(), 0);
    return keep;
  }
  sink_blocks = std::min(sink_blocks, n);
  rolling_blocks = std::min(rolling_blocks, n - sink_blocks);
  std::vector<char> kept(n, 0);
  for (int i = 0; i < sink_blocks; ++i) kept[i] = 1;
  for (int i = n - rolling_blocks; i < n; ++i) kept[i] = 1;
  int remaining = budget_blocks - sink_blocks - rolling_blocks;
  if (remaining > 0) {
    std::vector<int> middle;
    for (int i = sink_blocks; i < n - rolling_blocks; ++i) middle.push_back(i);
    std::stable_sort(middle.begin(), middle.end(), [&](int a, int b) {
      const float sa = a < static_cast<int>(scores.size()) ? scores[a] : 0.f;
      const float sb = b < static_cast<int>(scores.size()) ? scores[b] : 0.f;
      return sa > sb;
    });
    for (int i = 0; i < remaining && i < static_cast<int>(middle.size()); ++i) kept[middle[i]] = 1;
  }
  std::vector<int> new_blocks;
  const int tail_tokens = num_tokens_ - (n - 1) * kTokensPerBlock;  // tokens in the last block
  for (int i = 0; i < n; ++i) {
    if (kept[i]) {
      keep.push_back(i);
      new_blocks.push_back(blocks_[i]);
    } else {
      pool_->release(blocks_[i]);
    }
  }
  blocks_.swap(new_blocks);
  num_tokens_ = (static_cast<int>(blocks_.size()) - 1) * kTokensPerBlock + tail_tokens;
  if (committed_ > num_tokens_) committed_ = num_tokens_;
  return keep;
}

}  // namespace oxb
