// Block-granular radix prefix cache over the paged KV pool.
//
// A compressed trie whose edges are runs of whole 16-token blocks. Every cached block carries one
// pool reference held by the cache, so a hit simply appends the block ids to the new sequence's
// block table (zero copy) and eviction can only take blocks nobody else references.
// Eviction is LRU over leaves (logical clock) or by utility count / (1 + 0.1 * age).
//
// Capability parity with RadixPrefixCache (oxide-alloc/src/radix_cache.rs:35-283: longest-prefix
// match, insert with node split, LRU leaf eviction, utility eviction). The reference's GPU mode
// shares a prefix by copying a whole slot (continuous_batching.rs:406-414); here it is by reference.
#pragma once
#include <cstdint>
#include <memory>
#include <unordered_map>
#include <vector>

#include "block_manager.h"

namespace oxb {

class RadixCache {
 public:
  explicit RadixCache(BlockPool* pool) : pool_(pool), root_(new Node()) {}
  ~RadixCache() { clear(); }

  struct Match {
    std::vector<int> blocks;
    int tokens = 0;
  };
  // Longest cached prefix of `tokens` in whole blocks. Never matches the entire prompt when
  // `leave_one` is set (the last token must still be computed to produce logits).
  Match match(const int32_t* tokens, int n, bool leave_one);
  // Cache the first `n_blocks` full blocks of `tokens` (block ids in `blocks`). Blocks already
  // cached keep their existing ids; returns how many new blocks the cache took a reference on.
  int insert(const int32_t* tokens, const int* blocks, int n_blocks);
  // Free at least `want` blocks if possible; returns the number of blocks released to the pool.
  int evict(int want, bool by_utility = false);
  void clear();

  // Demotion hook: when recording, every leaf that evict() removes is logged with its whole token
  // prefix (root to the end of the leaf), so the owner of the device pool can copy the blocks'
  // contents to a slower tier before anything overwrites them.
  struct Evicted {
    std::vector<int32_t> tokens;  // the prefix the blocks complete, a multiple of 16 tokens
    int first_block = 0;          // index (in blocks of that prefix) of blocks[0]
    std::vector<int> blocks;
  };
  void record_evictions(bool on) { record_evictions_ = on; }
  std::vector<Evicted> take_evicted() {
    std::vector<Evicted> out;
    out.swap(evicted_);
    return out;
  }

  int cached_blocks() const { return cached_blocks_; }
  uint64_t lookups() const { return lookups_; }
  uint64_t hit_tokens() const { return hit_tokens_; }
  uint64_t lookup_tokens() const { return lookup_tokens_; }
  int num_nodes() const { return num_nodes_; }

 private:
  struct Node {
    std::vector<int32_t> tokens;  // multiple of 16
    std::vector<int> blocks;
    std::unordered_map<uint64_t, std::unique_ptr<Node>> children;  // key: hash of first block
    Node* parent = nullptr;
    uint64_t last_access = 0;
    uint64_t access_count = 0;
  };
  static uint64_t chunk_key(const int32_t* t);
  void collect_leaves(Node* n, std::vector<Node*>* out);
  void remove_leaf(Node* leaf);

  BlockPool* pool_;
  std::unique_ptr<Node> root_;
  uint64_t clock_ = 0;
  int cached_blocks_ = 0;
  int num_nodes_ = 0;
  uint64_t lookups_ = 0, hit_tokens_ = 0, lookup_tokens_ = 0;
  bool record_evictions_ = false;
  std::vector<Evicted> evicted_;
};

}  // namespace oxb
