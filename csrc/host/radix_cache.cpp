#include "radix_cache.h"

#include <algorithm>
#include <cstring>

namespace oxb {

uint64_t RadixCache::chunk_key(const int32_t* t) {
  uint64_t h = 1469598103934665603ull;  // FNV-1a over the 16 token ids of a block
  for (int i = 0; i < kTokensPerBlock; ++i) {
    uint32_t v = static_cast<uint32_t>(t[i]);
    for (int b = 0; b < 4; ++b) {
      h ^= (v >> (8 * b)) & 0xFF;
      h *= 1099511628211ull;
    }
  }
  return h;
}

RadixCache::Match RadixCache::match(const int32_t* tokens, int n, bool leave_one) {
  Match m;
  ++lookups_;
  lookup_tokens_ += static_cast<uint64_t>(n);
  int usable = leave_one ? n - 1 : n;
  int max_blocks = usable / kTokensPerBlock;
  Node* node = root_.get();
  int pos = 0;  // in blocks
  ++clock_;
  while (pos < max_blocks) {
    auto it = node->children.find(chunk_key(tokens + pos * kTokensPerBlock));
    if (it == node->children.end()) break;
    Node* child = it->second.get();
    const int child_blocks = static_cast<int>(child->blocks.size());
    int common = 0;
    while (common < child_blocks && pos + common < max_blocks &&
           std::memcmp(child->tokens.data() + common * kTokensPerBlock,
                       tokens + (pos + common) * kTokensPerBlock,
                       sizeof(int32_t) * kTokensPerBlock) == 0)
      ++common;
    if (common == 0) break;  // hash collision
    child->last_access = clock_;
    ++child->access_count;
    for (int i = 0; i < common; ++i) m.blocks.push_back(child->blocks[i]);
    pos += common;
    if (common < child_blocks) break;
    node = child;
  }
  m.tokens = pos * kTokensPerBlock;
  hit_tokens_ += static_cast<uint64_t>(m.tokens);
  return m;
}

int RadixCache::insert(const int32_t* tokens, const int* blocks, int n_blocks) {
  Node* node = root_.get();
  int pos = 0;
  int added = 0;
  ++clock_;
  while (pos < n_blocks) {
    const uint64_t key = chunk_key(tokens + pos * kTokensPerBlock);
    auto it = node->children.find(key);
    if (it == node->children.end()) {
      std::unique_ptr<Node> leaf(new Node());
      leaf->parent = node;
      leaf->tokens.assign(tokens + pos * kTokensPerBlock, tokens + n_blocks * kTokensPerBlock);
      leaf->blocks.assign(blocks + pos, blocks + n_blocks);
      leaf->last_access = clock_;
      leaf->access_count = 1;
      for (int b : leaf->blocks) pool_->retain(b);
      added += n_blocks - pos;
      cached_blocks_ += n_blocks - pos;
      node->children.emplace(key, std::move(leaf));
      ++num_nodes_;
      return added;
    }
    Node* child = it->second.get();
    const int child_blocks = static_cast<int>(child->blocks.size());
    int common = 0;
    while (common < child_blocks && pos + common < n_blocks &&
           std::memcmp(child->tokens.data() + common * kTokensPerBlock,
                       tokens + (pos + common) * kTokensPerBlock,
                       sizeof(int32_t) * kTokensPerBlock) == 0)
      ++common;
    if (common == 0) return added;  // hash collision: leave the existing entry alone
    child->last_access = clock_;
    if (common < child_blocks) {
      // split: child keeps the common head, a new node takes its tail
      std::unique_ptr<Node> tail(new Node());
      tail->tokens.assign(child->tokens.begin() + common * kTokensPerBlock, child->tokens.end());
      tail->blocks.assign(child->blocks.begin() + common, child->blocks.end());
      tail->children = std::move(child->children);
      for (auto& kv : tail->children) kv.second->parent = tail.get();
      tail->parent = child;
      tail->last_access = child->last_access;
      tail->access_count = child->access_count;
      child->children.clear();
      child->tokens.resize(common * kTokensPerBlock);
      child->blocks.resize(common);
      const uint64_t tkey = chunk_key(tail->tokens.data());
      child->children.emplace(tkey, std::move(tail));
      ++num_nodes_;
    }
    pos += common;
    node = child;
  }
  return added;
}

void RadixCache::collect_leaves(Node* n, std::vector<Node*>* out) {
  if (n != root_.get() && n->children.empty()) {
    out->push_back(n);
    return;
  }
  for (auto& kv : n->children) collect_leaves(kv.second.get(), out);
}

void RadixCache::remove_leaf(Node* leaf) {
  Node* parent = leaf->parent;
  for (int b : leaf->blocks) pool_->release(b);
  cached_blocks_ -= static_cast<int>(leaf->blocks.size());
  const uint64_t key = chunk_key(leaf->tokens.data());
  parent->children.erase(key);
  --num_nodes_;
}

int RadixCache::evict(int want, bool by_utility) {
  int freed = 0;
  while (freed < want) {
    std::vector<Node*> leaves;
    collect_leaves(root_.get(), &leaves);
    // only leaves whose blocks nobody but the cache holds can give memory back
    Node* victim = nullptr;
    double best = 0.0;
    for (Node* l : leaves) {
      bool exclusive = true;
      for (int b : l->blocks)
        if (pool_->ref_count(b) != 1) {
          exclusive = false;
          break;
        }
      if (!exclusive) continue;
      double score;
      if (by_utility) {
        const double age = static_cast<double>(clock_ - l->last_access);
        score = static_cast<double>(l->access_count) / (1.0 + 0.1 * age);
      } else {
        score = static_cast<double>(l->last_access);
      }
      if (victim == nullptr || score < best) {
        victim = l;
        best = score;
      }
    }
    if (victim == nullptr) break;
    freed += static_cast<int>(victim->blocks.size());
    if (record_evictions_) {
      Evicted e;
      std::vector<Node*> path;
      for (Node* n = victim; n != nullptr && n != root_.get(); n = n->parent) path.push_back(n);
      for (auto it = path.rbegin(); it != path.rend(); ++it)
        e.tokens.insert(e.tokens.end(), (*it)->tokens.begin(), (*it)->tokens.end());
      e.first_block = static_cast<int>((e.tokens.size() - victim->tokens.size()) / kTokensPerBlock);
      e.blocks = victim->blocks;
      evicted_.push_back(std::move(e));
    }
    remove_leaf(victim);
  }
  return freed;
}

void RadixCache::clear() {
  std::vector<Node*> stack{root_.get()};
  std::vector<Node*> all;
  while (!stack.empty()) {
    Node* n = stack.back();
    stack.pop_back();
    all.push_back(n);
    for (auto& kv : n->children) stack.push_back(kv.second.get());
  }
  for (Node* n : all)
    for (int b : n->blocks) pool_->release(b);
  root_.reset(new Node());
  cached_blocks_ = 0;
  num_nodes_ = 0;
}

}  // namespace oxb
