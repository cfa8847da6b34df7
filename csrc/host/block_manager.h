// Paged-KV block pool and per-sequence block tables (host side of the device KV pool).
//
// The device pool is [num_blocks, Hkv, 16, D] per layer; this class only hands out block ids.
// Blocks are reference counted so that the radix prefix cache and any number of sequences can
// share a block (zero-copy prefix reuse); a partially filled shared block is copied on write.
//
// Capability parity with the reference's PagedKvArena / SequenceBlockTable
// (oxide-alloc/src/paged_kv.rs:51-358), TransactionalBlockTable (transactional.rs:4-175) and
// the refcounted SharedPhysicalBlock of oxide-core/src/dag.rs:9-146 -- redesigned around a
// device-resident pool instead of host Vec<f32> pages.
#pragma once
#include <cstdint>
#include <mutex>
#include <stdexcept>
#include <utility>
#include <vector>

namespace oxb {

constexpr int kTokensPerBlock = 16;

class BlockPool {
 public:
  explicit BlockPool(int num_blocks) : ref_(num_blocks, 0) {
    free_.reserve(num_blocks);
    for (int i = num_blocks - 1; i >= 0; --i) free_.push_back(i);
  }
  int num_blocks() const { return static_cast<int>(ref_.size()); }
  int num_free() const {
    std::lock_guard<std::mutex> g(mu_);
    return static_cast<int>(free_.size());
  }
  // -1 when the pool is exhausted.
  int allocate() {
    std::lock_guard<std::mutex> g(mu_);
    if (free_.empty()) return -1;
    int b = free_.back();
    free_.pop_back();
    ref_[b] = 1;
    return b;
  }
  void retain(int b) {
    std::lock_guard<std::mutex> g(mu_);
    check(b);
    if (ref_[b] <= 0) throw std::runtime_error("BlockPool::retain on a free block");
    ++ref_[b];
  }
  // Returns true when the block went back to the free list.
  bool release(int b) {
    std::lock_guard<std::mutex> g(mu_);
    check(b);
    if (ref_[b] <= 0) throw std::runtime_error("BlockPool::release on a free block");
    if (--ref_[b] == 0) {
      free_.push_back(b);
      return true;
    }
    return false;
  }
  int ref_count(int b) const {
    std::lock_guard<std::mutex> g(mu_);
    check(b);
    return ref_[b];
  }

 private:
  void check(int b) const {
    if (b < 0 || b >= static_cast<int>(ref_.size())) throw std::out_of_range("block id");
  }
  mutable std::mutex mu_;
  std::vector<int> ref_;
  std::vector<int> free_;
};

// Block list of one sequence. `num_tokens` counts tokens whose KV is (or is about to be) stored.
class SequenceBlockTable {
 public:
  explicit SequenceBlockTable(BlockPool* pool) : pool_(pool) {}
  ~SequenceBlockTable() { release_all(); }
  SequenceBlockTable(const SequenceBlockTable&) = delete;
  SequenceBlockTable& operator=(const SequenceBlockTable&) = delete;

  const std::vector<int>& blocks() const { return blocks_; }
  int num_tokens() const { return num_tokens_; }
  int committed_tokens() const { return committed_; }

  // Adopt already-filled shared blocks (a radix-cache hit). The table takes one reference each.
  void adopt_prefix(const std::vector<int>& shared, int tokens) {
    if (!blocks_.empty()) throw std::runtime_error("adopt_prefix on a non-empty table");
    for (int b : shared) {
      pool_->retain(b);
      blocks_.push_back(b);
    }
    num_tokens_ = committed_ = tokens;
  }

  // Makes room for `n` more tokens. Returns false (and changes nothing) if the pool runs dry.
  // `cow` receives (src, dst) pairs when a shared, partially filled tail block had to be forked.
  bool advance(int n, std::vector<std::pair<int, int>>* cow = nullptr) {
    const int need_tokens = num_tokens_ + n;
    const int need_blocks = (need_tokens + kTokensPerBlock - 1) / kTokensPerBlock;
    std::vector<int> fresh;
    int fork_src = -1, fork_dst = -1;
    const bool tail_partial = (num_tokens_ % kTokensPerBlock) != 0;
    if (n > 0 && tail_partial && !blocks_.empty() && pool_->ref_count(blocks_.back()) > 1) {
      fork_dst = pool_->allocate();
      if (fork_dst < 0) return false;
      fork_src = blocks_.back();
    }
    for (int i = static_cast<int>(blocks_.size()); i < need_blocks; ++i) {
      int b = pool_->allocate();
      if (b < 0) {
        for (int f : fresh) pool_->release(f);
        if (fork_dst >= 0) pool_->release(fork_dst);
        return false;
      }
      fresh.push_back(b);
    }
    if (fork_dst >= 0) {
      pool_->release(fork_src);
      blocks_.back() = fork_dst;
      if (cow != nullptr) cow->emplace_back(fork_src, fork_dst);
    }
    blocks_.insert(blocks_.end(), fresh.begin(), fresh.end());
    num_tokens_ = need_tokens;
    return true;
  }

  // Holds blocks for `n` tokens beyond num_tokens() without changing the length, so that the next
  // advance() calls up to that point allocate nothing (a burst of decode steps whose block table is
  // handed to the device once). All or nothing. rewind_to() gives unused reservations back.
  bool reserve(int n) {
    const int need_blocks = (num_tokens_ + n + kTokensPerBlock - 1) / kTokensPerBlock;
    std::vector<int> fresh;
    for (int i = static_cast<int>(blocks_.size()); i < need_blocks; ++i) {
      int b = pool_->allocate();
      if (b < 0) {
        for (int f : fresh) pool_->release(f);
        return false;
      }
      fresh.push_back(b);
    }
    blocks_.insert(blocks_.end(), fresh.begin(), fresh.end());
    return true;
  }

  // Speculative decoding: everything up to num_tokens() becomes permanent.
  void commit() { committed_ = num_tokens_; }
  // O(blocks dropped) rollback to `tokens` (>= committed prefix is the caller's contract).
  void rewind_to(int tokens) {
    if (tokens > num_tokens_) throw std::runtime_error("rewind_to beyond the end");
    const int keep = (tokens + kTokensPerBlock - 1) / kTokensPerBlock;
    while (static_cast<int>(blocks_.size()) > keep) {
      pool_->release(blocks_.back());
      blocks_.pop_back();
    }
    num_tokens_ = tokens;
    if (committed_ > tokens) committed_ = tokens;
  }
  void rollback() { rewind_to(committed_); }

  // H2O + StreamingLLM pruning at block granularity: keep `sink_blocks` first blocks, the last
  // `rolling_blocks`, and the highest-scoring middle blocks up to `budget_blocks` in total.
  // Returns the indices (into the old list) that were kept, in order; the caller compacts
  // positions accordingly. Dropped blocks are released.
  std::vector<int> prune_heavy_hitters(const std::vector<float>& scores, int sink_blocks,
                                       int rolling_blocks, int budget_blocks);

  void release_all() {
    for (int b : blocks_) pool_->release(b);
    blocks_.clear();
    num_tokens_ = committed_ = 0;
  }

 private:
  BlockPool* pool_;
  std::vector<int> blocks_;
  int num_tokens_ = 0;
  int committed_ = 0;
};

}  // namespace oxb
