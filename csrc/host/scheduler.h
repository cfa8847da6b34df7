// Continuous-batching scheduler core (host, C++).
//
// Each call of schedule() builds one engine step: every running sequence in the decode phase
// contributes one token, and the rest of the token budget goes to prefill chunks (continuing
// chunks first, then newly admitted requests, whose prompts are first matched against the radix
// prefix cache). The chunked-prefill budget follows the reference's SLA formula
//   clamp(min((sla_itl - (base + 350us * B)) / alpha, max_batched - B), chunk_min, chunk_max)
// (oxide-engine/src/continuous_batching.rs:88-112). Speculative drafts ride along as short
// verify chunks. update() consumes the sampled tokens, applies stop rules, accepts drafts,
// rolls the block table back after a partial acceptance, feeds finished blocks to the prefix
// cache and returns token events.
//
// Capability parity: ContinuousBatchingEngine (continuous_batching.rs:205-1395) admission,
// chunking, radix LRU at >90% -> 80%, cancellation, finish reasons; block-table bookkeeping of
// speculative decoding (speculative.rs:232-304, transactional.rs:4-175).
#pragma once
#include <cstdint>
#include <deque>
#include <map>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "block_manager.h"
#include "radix_cache.h"

namespace oxb {

struct SchedulerConfig {
  int num_blocks = 1024;
  int max_num_seqs = 64;
  int max_num_batched_tokens = 2048;
  int max_blocks_per_seq = 512;
  int chunk_min = 32;
  int chunk_max = 512;
  double sla_itl_us = 25000.0;
  double base_us = 2000.0;
  double per_token_us = 25.0;        // alpha
  double decode_us_per_seq = 350.0;
  bool enable_radix = true;
  double radix_high = 0.90;
  double radix_low = 0.80;
  bool sla_budget = true;            // false: budget = max_num_batched_tokens - decodes
  // Context shift (oxide-alloc/src/kv_advanced.rs:299-339): a sequence that fills its window keeps
  // its first `shift_keep_tokens` and drops the oldest max(shift_step_tokens, overflow) after them,
  // instead of ending with "length". Whole 16-token blocks are dropped; positions stay absolute.
  bool context_shift = false;
  int shift_keep_tokens = 4;
  int shift_step_tokens = 256;
};

enum class Phase : int { Waiting = 0, Prefill = 1, Decode = 2, Finished = 3 };

struct Request {
  int64_t id = 0;
  std::vector<int32_t> tokens;  // prompt followed by generated tokens
  int prompt_len = 0;
  int max_new_tokens = 0;
  std::vector<int32_t> stop_ids;
  bool ignore_eos = false;
  int computed = 0;             // tokens whose KV is in the cache
  int dropped = 0;              // of those, tokens removed from the middle by heavy-hitter pruning
  int prefix_hit = 0;           // tokens served by the radix cache at admission
  int cached_blocks = 0;        // full blocks already offered to the radix cache
  Phase phase = Phase::Waiting;
  std::vector<int32_t> drafts;  // speculative tokens to verify in the next step
  uint64_t arrival = 0;
  int preemptions = 0;
  std::unique_ptr<SequenceBlockTable> table;
  int generated() const { return static_cast<int>(tokens.size()) - prompt_len; }
};

struct TokenEvent {
  int64_t req_id;
  int32_t token;
  bool finished;
  std::string reason;  // "", "stop", "length", "cancelled", "prefill_error: ..."
};

struct StepPlan {
  int n_tokens = 0;
  int n_decode = 0;
  int n_prefill = 0;
  int max_blocks = 0;  // columns of the block-table arrays
  std::vector<int32_t> token_ids, positions;
  std::vector<int64_t> slot_mapping;
  std::vector<int64_t> decode_ids;
  std::vector<int32_t> decode_seq_lens, decode_block_tables;
  std::vector<int64_t> prefill_ids;
  std::vector<int32_t> q_start, q_lens, ctx_lens, prefill_block_tables, tile_seq, tile_q0;
  std::vector<int32_t> logit_rows;
  std::vector<int64_t> logit_req;
  std::vector<int32_t> cow_src, cow_dst;
  int prefill_tokens = 0;
};

class Scheduler {
 public:
  explicit Scheduler(const SchedulerConfig& cfg);

  void add_request(int64_t id, const std::vector<int32_t>& prompt, int max_new_tokens,
                   const std::vector<int32_t>& stop_ids, bool ignore_eos);
  bool cancel(int64_t id, std::vector<TokenEvent>* events);
  void set_drafts(int64_t id, const std::vector<int32_t>& drafts);
  // Heavy-hitter (H2O) pruning of a decoding request between steps: keeps the sink blocks, the
  // rolling window and the best-scored middle blocks within `budget_blocks`; the dropped blocks go
  // back to the pool, positions stay absolute. Returns the kept block indices (empty: not pruned).
  std::vector<int> prune_request(int64_t id, const std::vector<float>& block_scores, int sink_blocks,
                                 int rolling_blocks, int budget_blocks);
  // Grammar jump-forward: tokens that the grammar leaves no choice about are appended to a decoding
  // request without sampling; they are computed as one prefill chunk in the next step, whose last
  // row gives the logits of the next free choice (continuous_batching.rs:475,807,1328). Returns one
  // event per appended token (the request may finish on a stop id or its length limit).
  std::vector<TokenEvent> append_forced(int64_t id, const std::vector<int32_t>& forced);
  // Decode burst: holds KV blocks for up to `n` further tokens of a decoding request, so that the
  // next decode plans of that request allocate nothing and the block table of the first plan is
  // valid for all of them. Returns how many tokens are covered (0..n; fewer when the pool, the
  // context limit or the request's token budget is short).
  int reserve_ahead(int64_t id, int n);
  // KV tiers. Number of whole blocks of `tokens` that the device prefix cache holds right now.
  int radix_cached_blocks(const std::vector<int32_t>& tokens);
  // Makes the first `n_blocks` blocks of `tokens` a cached prefix: blocks already cached stay, the
  // rest are taken from the pool and handed to the cache. Returns the ids of the new blocks, in
  // order (the caller fills them before the next launch); empty when the pool is short.
  std::vector<int> radix_adopt(const std::vector<int32_t>& tokens, int n_blocks);
  // Events that schedule() produced (requests it had to end because they can never fit the pool).
  std::vector<TokenEvent> take_events();
  // Fault hook: the next prefill chunk of this request fails (host-side fault injection).
  void inject_prefill_error(int64_t id, const std::string& msg);

  StepPlan schedule();
  // `sampled[i]` is the token drawn from logits row i of the plan that was just executed.
  std::vector<TokenEvent> update(const StepPlan& plan, const std::vector<int32_t>& sampled);

  int prefill_budget(int active_decodes) const;
  int num_waiting() const { return static_cast<int>(waiting_.size()); }
  int num_running() const { return static_cast<int>(running_.size()); }
  int num_free_blocks() const { return pool_.num_free(); }
  bool has_work() const { return !waiting_.empty() || !running_.empty(); }
  const Request* find(int64_t id) const;
  BlockPool& pool() { return pool_; }
  RadixCache& radix() { return radix_; }
  const SchedulerConfig& config() const { return cfg_; }
  uint64_t preemptions() const { return preemptions_; }
  uint64_t context_shifts() const { return context_shifts_; }
  std::vector<int64_t> running_ids() const;

 private:
  bool ensure_blocks(Request* r, int n_tokens, StepPlan* plan);
  void shift_context(Request* r, int incoming);
  void preempt(Request* r);
  void abort(Request* r, const std::string& reason);
  void finish(Request* r);
  void offer_to_radix(Request* r);
  void radix_pressure();

  SchedulerConfig cfg_;
  BlockPool pool_;
  RadixCache radix_;
  std::deque<std::unique_ptr<Request>> waiting_;
  std::vector<std::unique_ptr<Request>> running_;
  std::unordered_map<int64_t, std::string> prefill_faults_;
  std::vector<TokenEvent> deferred_;
  std::vector<int64_t> cow_owner_;  // request id of each copy-on-write pair of the plan being built
  uint64_t arrivals_ = 0;
  uint64_t preemptions_ = 0;
  uint64_t context_shifts_ = 0;
};

}  // namespace oxb
