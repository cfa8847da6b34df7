#include "scheduler.h"

#include <algorithm>
#include <cmath>
#include <stdexcept>

namespace oxb {

namespace {
constexpr int kTileQ = 128;  // query rows per prefill-attention tile (one tcgen05 M tile)
}

Scheduler::Scheduler(const SchedulerConfig& cfg) : cfg_(cfg), pool_(cfg.num_blocks), radix_(&pool_) {}

void Scheduler::add_request(int64_t id, const std::vector<int32_t>& prompt, int max_new_tokens,
                            const std::vector<int32_t>& stop_ids, bool ignore_eos) {
  if (prompt.empty()) throw std::invalid_argument("empty prompt");
  if (static_cast<int>(prompt.size()) + 1 > cfg_.max_blocks_per_seq * kTokensPerBlock)
    throw std::invalid_argument("prompt longer than the per-sequence KV capacity");
  std::unique_ptr<Request> r(new Request());
  r->id = id;
  r->tokens = prompt;
  r->prompt_len = static_cast<int>(prompt.size());
  r->max_new_tokens = max_new_tokens;
  r->stop_ids = stop_ids;
  r->ignore_eos = ignore_eos;
  r->arrival = arrivals_++;
  r->table.reset(new SequenceBlockTable(&pool_));
  waiting_.push_back(std::move(r));
}

const Request* Scheduler::find(int64_t id) const {
  for (auto& r : running_)
    if (r->id == id) return r.get();
  for (auto& r : waiting_)
    if (r->id == id) return r.get();
  return nullptr;
}

std::vector<int64_t> Scheduler::running_ids() const {
  std::vector<int64_t> ids;
  for (auto& r : running_) ids.push_back(r->id);
  return ids;
}

bool Scheduler::cancel(int64_t id, std::vector<TokenEvent>* events) {
  for (auto it = waiting_.begin(); it != waiting_.end(); ++it) {
    if ((*it)->id == id) {
      if (events) events->push_back({id, -1, true, "cancelled"});
      waiting_.erase(it);
      return true;
    }
  }
  for (auto it = running_.begin(); it != running_.end(); ++it) {
    if ((*it)->id == id) {
      if (events) events->push_back({id, -1, true, "cancelled"});
      (*it)->table->release_all();
      running_.erase(it);
      return true;
    }
  }
  return false;
}

void Scheduler::set_drafts(int64_t id, const std::vector<int32_t>& drafts) {
  // a pruned sequence decodes one token at a time (its KV is no longer a contiguous prefix)
  for (auto& r : running_)
    if (r->id == id && r->phase == Phase::Decode && r->dropped == 0) r->drafts = drafts;
}

std::vector<int> Scheduler::prune_request(int64_t id, const std::vector<float>& block_scores,
                                          int sink_blocks, int rolling_blocks, int budget_blocks) {
  for (auto& r : running_) {
    if (r->id != id || r->phase != Phase::Decode) continue;
    const int before = static_cast<int>(r->table->blocks().size());
    if (before <= budget_blocks) return {};
    std::vector<int> keep =
        r->table->prune_heavy_hitters(block_scores, sink_blocks, rolling_blocks, budget_blocks);
    r->dropped += (before - static_cast<int>(keep.size())) * kTokensPerBlock;
    r->drafts.clear();
    return keep;
  }
  return {};
}

void Scheduler::inject_prefill_error(int64_t id, const std::string& msg) { prefill_faults_[id] = msg; }

int Scheduler::prefill_budget(int active_decodes) const {
  const int room = cfg_.max_num_batched_tokens - active_decodes;
  if (room <= 0) return 0;
  if (!cfg_.sla_budget) return room;
  const double decode_est = cfg_.base_us + cfg_.decode_us_per_seq * active_decodes;
  double by_sla = (cfg_.sla_itl_us - decode_est) / cfg_.per_token_us;
  if (by_sla < 0) by_sla = 0;
  int b = static_cast<int>(std::min<double>(by_sla, room));
  b = std::max(b, cfg_.chunk_min);
  b = std::min(b, cfg_.chunk_max);
  return std::min(b, room);
}

void Scheduler::radix_pressure() {
  if (!cfg_.enable_radix) return;
  const int total = pool_.num_blocks();
  const int used = total - pool_.num_free();
  if (used > static_cast<int>(cfg_.radix_high * total)) {
    const int target = static_cast<int>(cfg_.radix_low * total);
    radix_.evict(used - target);
  }
}

bool Scheduler::ensure_blocks(Request* r, int n_tokens, StepPlan* plan) {
  std::vector<std::pair<int, int>> cow;
  auto record = [&]() {
    for (auto& c : cow) {
      plan->cow_src.push_back(c.first);
      plan->cow_dst.push_back(c.second);
      cow_owner_.push_back(r->id);
    }
  };
  if (r->table->advance(n_tokens, &cow)) {
    record();
    return true;
  }
  if (cfg_.enable_radix) {
    const int need = (n_tokens + kTokensPerBlock - 1) / kTokensPerBlock + 1;
    radix_.evict(need);
    cow.clear();
    if (r->table->advance(n_tokens, &cow)) {
      record();
      return true;
    }
  }
  return false;
}

void Scheduler::shift_context(Request* r, int incoming) {
  const int limit = cfg_.max_blocks_per_seq * kTokensPerBlock;
  const int n_blocks = static_cast<int>(r->table->blocks().size());
  const int sink = std::max(1, (cfg_.shift_keep_tokens + kTokensPerBlock - 1) / kTokensPerBlock);
  const int overflow = r->computed - r->dropped + incoming - limit;
  const int drop_tokens = std::max(cfg_.shift_step_tokens, overflow);
  int drop = (drop_tokens + kTokensPerBlock - 1) / kTokensPerBlock;
  drop = std::min(drop, n_blocks - sink - 1);  // the block being written always stays
  if (drop <= 0) return;
  const int rolling = n_blocks - sink - drop;
  r->table->prune_heavy_hitters({}, sink, rolling, sink + rolling);
  r->dropped += drop * kTokensPerBlock;
  r->drafts.clear();
  ++context_shifts_;
}

void Scheduler::preempt(Request* r) {
  // recompute-style preemption: drop the KV, keep the tokens, go back to the head of the queue
  ++preemptions_;
  ++r->preemptions;
  r->table->release_all();
  r->computed = 0;
  r->dropped = 0;
  r->cached_blocks = 0;
  r->drafts.clear();
  r->phase = Phase::Waiting;
  for (auto it = running_.begin(); it != running_.end(); ++it) {
    if (it->get() == r) {
      std::unique_ptr<Request> owned = std::move(*it);
      running_.erase(it);
      waiting_.push_front(std::move(owned));
      return;
    }
  }
}

void Scheduler::abort(Request* r, const std::string& reason) {
  deferred_.push_back({r->id, -1, true, reason});
  r->table->release_all();
  r->phase = Phase::Finished;
  for (auto it = running_.begin(); it != running_.end(); ++it) {
    if (it->get() == r) {
      running_.erase(it);
      return;
    }
  }
}

std::vector<TokenEvent> Scheduler::take_events() {
  std::vector<TokenEvent> out;
  out.swap(deferred_);
  return out;
}

std::vector<TokenEvent> Scheduler::append_forced(int64_t id, const std::vector<int32_t>& forced) {
  std::vector<TokenEvent> events;
  for (auto& up : running_) {
    Request* r = up.get();
    if (r->id != id) continue;
    if (r->phase != Phase::Decode || r->dropped != 0 || forced.empty()) return events;
    r->drafts.clear();
    const int cap = cfg_.max_blocks_per_seq * kTokensPerBlock;
    for (int32_t tok : forced) {
      if (r->generated() >= r->max_new_tokens || static_cast<int>(r->tokens.size()) + 1 >= cap) break;
      r->tokens.push_back(tok);
      bool stop = false;
      if (!r->ignore_eos)
        for (int32_t sid : r->stop_ids) stop |= sid == tok;
      std::string reason;
      if (stop)
        reason = "stop";
      else if (r->generated() >= r->max_new_tokens)
        reason = "length";
      events.push_back({r->id, tok, !reason.empty(), reason});
      if (!reason.empty()) {
        finish(r);
        return events;
      }
    }
    // the tokens after `computed` (the last sampled one and the forced ones) are prefilled as one
    // chunk; its last row yields the logits of the next free choice
    if (static_cast<int>(r->tokens.size()) - r->computed > 1) r->phase = Phase::Prefill;
    return events;
  }
  return events;
}

int Scheduler::reserve_ahead(int64_t id, int n) {
  for (auto& up : running_) {
    Request* r = up.get();
    if (r->id != id) continue;
    // context shift and pruning address blocks by position from the end of the table: no spare blocks there
    if (r->phase != Phase::Decode || r->dropped != 0 || cfg_.context_shift) return 0;
    const int cap = cfg_.max_blocks_per_seq * kTokensPerBlock;
    n = std::min(n, r->max_new_tokens - r->generated());
    n = std::min(n, cap - 1 - static_cast<int>(r->tokens.size()));
    while (n > 0 && !r->table->reserve(n)) n /= 2;
    return std::max(n, 0);
  }
  return 0;
}

int Scheduler::radix_cached_blocks(const std::vector<int32_t>& tokens) {
  if (!cfg_.enable_radix) return 0;
  return radix_.match(tokens.data(), static_cast<int>(tokens.size()), false).tokens / kTokensPerBlock;
}

std::vector<int> Scheduler::radix_adopt(const std::vector<int32_t>& tokens, int n_blocks) {
  std::vector<int> fresh;
  if (!cfg_.enable_radix || n_blocks <= 0 || static_cast<int>(tokens.size()) < n_blocks * kTokensPerBlock)
    return fresh;
  RadixCache::Match m = radix_.match(tokens.data(), n_blocks * kTokensPerBlock, false);
  const int have = m.tokens / kTokensPerBlock;
  if (have >= n_blocks) return fresh;
  for (int i = have; i < n_blocks; ++i) {
    const int b = pool_.allocate();
    if (b < 0) {
      for (int f : fresh) pool_.release(f);
      fresh.clear();
      return fresh;
    }
    fresh.push_back(b);
  }
  std::vector<int> ids(m.blocks.begin(), m.blocks.begin() + have);
  ids.insert(ids.end(), fresh.begin(), fresh.end());
  const int added = radix_.insert(tokens.data(), ids.data(), n_blocks);  // the cache takes its own reference
  for (int b : fresh) pool_.release(b);                                  // ... and is now the only holder
  if (added != static_cast<int>(fresh.size())) fresh.clear();            // nothing was taken (key collision)
  return fresh;
}

void Scheduler::offer_to_radix(Request* r) {
  if (!cfg_.enable_radix || r->dropped > 0) return;  // pruned KV is not a reusable prefix
  const int n_full = std::min<int>(r->computed, static_cast<int>(r->tokens.size())) / kTokensPerBlock;
  if (n_full <= r->cached_blocks) return;
  radix_.insert(r->tokens.data(), r->table->blocks().data(), n_full);
  r->cached_blocks = n_full;
}

void Scheduler::finish(Request* r) {
  offer_to_radix(r);
  r->table->release_all();
  r->phase = Phase::Finished;
  for (auto it = running_.begin(); it != running_.end(); ++it) {
    if (it->get() == r) {
      running_.erase(it);
      return;
    }
  }
}

StepPlan Scheduler::schedule() {
  StepPlan plan;
  cow_owner_.clear();
  radix_pressure();

  std::sort(running_.begin(), running_.end(),
            [](const std::unique_ptr<Request>& a, const std::unique_ptr<Request>& b) {
              return a->arrival < b->arrival;
            });

  struct Item {
    Request* r;
    int len;
    int kind;  // 0 decode, 1 prefill chunk, 2 verify chunk
  };
  std::vector<Item> decodes, chunks;
  // A preempted request may already sit in this step's lists (it was given blocks earlier in the
  // pass): take it out again.
  auto drop_item = [&](Request* v) {
    auto gone = [v](const Item& it) { return it.r == v; };
    decodes.erase(std::remove_if(decodes.begin(), decodes.end(), gone), decodes.end());
    chunks.erase(std::remove_if(chunks.begin(), chunks.end(), gone), chunks.end());
    // its copy-on-write pairs too: the destination blocks are free again and may be handed out
    size_t w = 0;
    for (size_t k = 0; k < cow_owner_.size(); ++k) {
      if (cow_owner_[k] == v->id) continue;
      plan.cow_src[w] = plan.cow_src[k];
      plan.cow_dst[w] = plan.cow_dst[k];
      cow_owner_[w++] = cow_owner_[k];
    }
    plan.cow_src.resize(w);
    plan.cow_dst.resize(w);
    cow_owner_.resize(w);
  };
  // Gets `n` more token slots for `r`, preempting younger requests (recompute style) while the
  // pool is short. Returns false when r itself had to give way: it is then back in the waiting
  // queue, or, when it was the only request left and still does not fit, aborted with `why`.
  auto blocks_or_preempt = [&](Request* r, int n, const char* why) -> bool {
    bool ok = ensure_blocks(r, n, &plan);
    while (!ok) {
      Request* victim = running_.back().get();
      if (victim == r) {
        drop_item(r);
        if (running_.size() == 1)
          abort(r, why);  // it has the whole pool to itself and still cannot grow
        else
          preempt(r);
        return false;
      }
      drop_item(victim);
      preempt(victim);
      ok = ensure_blocks(r, n, &plan);
    }
    return true;
  };

  // ---- 1. decode phase sequences (oldest first; the youngest is preempted when KV runs out) ----
  size_t i = 0;
  while (i < running_.size()) {
    Request* r = running_[i].get();
    if (r->phase != Phase::Decode) {
      ++i;
      continue;
    }
    const int need = 1 + static_cast<int>(r->drafts.size());
    const int limit = cfg_.max_blocks_per_seq * kTokensPerBlock;
    if (r->computed - r->dropped + need > limit) r->drafts.clear();
    if (cfg_.context_shift && r->computed - r->dropped + 1 > limit) shift_context(r, 1);
    const int n = 1 + static_cast<int>(r->drafts.size());
    if (!blocks_or_preempt(r, n, "length")) continue;  // running_[i] is now the next request
    if (n == 1)
      decodes.push_back({r, 1, 0});
    else
      chunks.push_back({r, n, 2});
    ++i;
  }

  int n_dec_tokens = 0;
  for (auto& d : decodes) n_dec_tokens += d.len;
  for (auto& c : chunks) n_dec_tokens += c.len;
  int budget = prefill_budget(n_dec_tokens);

  // ---- 2. continuing prefill chunks ----
  // While requests are waiting for a free slot's worth of budget, long prompts already in
  // flight take at most half of the step so that short newcomers are not stuck behind them.
  // A chunk that finds no free block preempts younger requests like a decode row does:
  // otherwise two half-prefilled prompts that together fill the pool would wait on each other
  // for ever.
  const bool newcomers = !waiting_.empty() && static_cast<int>(running_.size()) < cfg_.max_num_seqs;
  int continuing_budget = budget;
  if (newcomers) continuing_budget = std::max(std::min(cfg_.chunk_min, budget), budget / 2);
  for (size_t k = 0; k < running_.size() && budget > 0 && continuing_budget > 0;) {
    Request* r = running_[k].get();
    if (r->phase != Phase::Prefill) {
      ++k;
      continue;
    }
    const int remaining = static_cast<int>(r->tokens.size()) - r->computed;
    const int c = std::min(remaining, std::min(budget, continuing_budget));
    if (c <= 0) {
      ++k;
      continue;
    }
    if (!blocks_or_preempt(r, c, "prefill_error: prompt does not fit the KV pool")) continue;
    chunks.push_back({r, c, 1});
    budget -= c;
    continuing_budget -= c;
    ++k;
  }

  // ---- 3. admission of waiting requests ----
  while (!waiting_.empty() && budget > 0 &&
         static_cast<int>(running_.size()) < cfg_.max_num_seqs) {
    Request* r = waiting_.front().get();
    if (cfg_.enable_radix && r->computed == 0) {
      RadixCache::Match m = radix_.match(r->tokens.data(), static_cast<int>(r->tokens.size()), true);
      if (m.tokens > 0) {
        r->table->adopt_prefix(m.blocks, m.tokens);
        r->computed = m.tokens;
        r->prefix_hit = m.tokens;
        r->cached_blocks = m.tokens / kTokensPerBlock;
      }
    }
    const int remaining = static_cast<int>(r->tokens.size()) - r->computed;
    const int c = std::min(remaining, budget);
    if (!ensure_blocks(r, c, &plan)) {
      r->table->release_all();
      r->computed = 0;
      r->cached_blocks = 0;
      if (running_.empty()) {
        // the whole pool is free and the first chunk still does not fit
        std::unique_ptr<Request> owned = std::move(waiting_.front());
        waiting_.pop_front();
        deferred_.push_back({owned->id, -1, true, "prefill_error: prompt does not fit the KV pool"});
        continue;
      }
      break;  // no memory: stay queued
    }
    r->phase = Phase::Prefill;
    std::unique_ptr<Request> owned = std::move(waiting_.front());
    waiting_.pop_front();
    running_.push_back(std::move(owned));
    chunks.push_back({r, c, 1});
    budget -= c;
  }

  // ---- build the flat arrays: decode rows first, then chunk rows ----
  int max_blocks = 1;
  for (auto& d : decodes) max_blocks = std::max<int>(max_blocks, d.r->table->blocks().size());
  for (auto& c : chunks) max_blocks = std::max<int>(max_blocks, c.r->table->blocks().size());
  plan.max_blocks = max_blocks;
  plan.n_decode = static_cast<int>(decodes.size());
  plan.n_prefill = static_cast<int>(chunks.size());

  // `pos` is the absolute position; the KV index skips what pruning removed from the middle
  auto slot_of = [](const Request* r, int pos) -> int64_t {
    const auto& b = r->table->blocks();
    const int kv = pos - r->dropped;
    return static_cast<int64_t>(b[kv / kTokensPerBlock]) * kTokensPerBlock + kv % kTokensPerBlock;
  };
  auto push_table = [&](std::vector<int32_t>* dst, const Request* r) {
    const auto& b = r->table->blocks();
    for (int k = 0; k < max_blocks; ++k)
      dst->push_back(k < static_cast<int>(b.size()) ? b[k] : 0);
  };

  for (auto& d : decodes) {
    Request* r = d.r;
    const int pos = r->computed;
    plan.token_ids.push_back(r->tokens.back());
    plan.positions.push_back(pos);
    plan.slot_mapping.push_back(slot_of(r, pos));
    plan.decode_ids.push_back(r->id);
    plan.decode_seq_lens.push_back(pos + 1 - r->dropped);
    push_table(&plan.decode_block_tables, r);
    plan.logit_rows.push_back(static_cast<int32_t>(plan.token_ids.size()) - 1);
    plan.logit_req.push_back(r->id);
  }
  int s = 0;
  for (auto& c : chunks) {
    Request* r = c.r;
    const int start = static_cast<int>(plan.token_ids.size());
    plan.prefill_ids.push_back(r->id);
    plan.q_start.push_back(start);
    plan.q_lens.push_back(c.len);
    plan.ctx_lens.push_back(r->computed - r->dropped + c.len);
    push_table(&plan.prefill_block_tables, r);
    for (int q0 = 0; q0 < c.len; q0 += kTileQ) {
      plan.tile_seq.push_back(s);
      plan.tile_q0.push_back(q0);
    }
    for (int j = 0; j < c.len; ++j) {
      const int pos = r->computed + j;
      int32_t tok;
      if (c.kind == 2)
        tok = j == 0 ? r->tokens.back() : r->drafts[j - 1];
      else
        tok = r->tokens[pos];
      plan.token_ids.push_back(tok);
      plan.positions.push_back(pos);
      plan.slot_mapping.push_back(slot_of(r, pos));
      const bool last = j == c.len - 1;
      const bool wants_logits =
          c.kind == 2 || (last && r->computed + c.len == static_cast<int>(r->tokens.size()));
      if (wants_logits) {
        plan.logit_rows.push_back(static_cast<int32_t>(plan.token_ids.size()) - 1);
        plan.logit_req.push_back(r->id);
      }
    }
    if (c.kind == 1) plan.prefill_tokens += c.len;
    ++s;
  }
  plan.n_tokens = static_cast<int>(plan.token_ids.size());
  return plan;
}

std::vector<TokenEvent> Scheduler::update(const StepPlan& plan, const std::vector<int32_t>& sampled) {
  std::vector<TokenEvent> events;
  if (sampled.size() != plan.logit_rows.size())
    throw std::invalid_argument("update: one sampled token per logits row expected");

  auto find_running = [&](int64_t id) -> Request* {
    for (auto& r : running_)
      if (r->id == id) return r.get();
    return nullptr;
  };
  auto emit = [&](Request* r, int32_t tok) -> bool {
    // returns true when the request finished with this token
    r->tokens.push_back(tok);
    bool stop = false;
    if (!r->ignore_eos)
      for (int32_t sid : r->stop_ids) stop |= sid == tok;
    std::string reason;
    if (stop)
      reason = "stop";
    else if (r->generated() >= r->max_new_tokens)
      reason = "length";
    else if (!cfg_.context_shift &&
             static_cast<int>(r->tokens.size()) - r->dropped >= cfg_.max_blocks_per_seq * kTokensPerBlock)
      reason = "length";
    events.push_back({r->id, tok, !reason.empty(), reason});
    return !reason.empty();
  };

  size_t li = 0;  // cursor into logit rows
  for (int d = 0; d < plan.n_decode; ++d) {
    Request* r = find_running(plan.decode_ids[d]);
    const int32_t tok = sampled[li++];
    if (r == nullptr) continue;  // cancelled meanwhile
    r->computed += 1;
    r->table->commit();
    if (emit(r, tok)) finish(r);
  }
  for (int c = 0; c < plan.n_prefill; ++c) {
    const int64_t id = plan.prefill_ids[c];
    const int len = plan.q_lens[c];
    // logits rows that belong to this chunk
    const int row_lo = plan.q_start[c], row_hi = row_lo + len;
    size_t first = li;
    while (li < plan.logit_rows.size() && plan.logit_rows[li] >= row_lo &&
           plan.logit_rows[li] < row_hi)
      ++li;
    const int n_logits = static_cast<int>(li - first);
    Request* r = find_running(id);
    if (r == nullptr) continue;
    auto fault = prefill_faults_.find(id);
    if (fault != prefill_faults_.end() && r->phase == Phase::Prefill) {
      events.push_back({id, -1, true, "prefill_error: " + fault->second});
      prefill_faults_.erase(fault);
      r->table->release_all();
      for (auto it = running_.begin(); it != running_.end(); ++it)
        if (it->get() == r) {
          running_.erase(it);
          break;
        }
      continue;
    }
    if (r->phase == Phase::Prefill) {
      r->computed += len;
      r->table->commit();
      offer_to_radix(r);
      if (n_logits == 1) {
        r->phase = Phase::Decode;
        if (emit(r, sampled[first])) finish(r);
      }
    } else {
      // speculative verify: rows = [last token, draft_0 .. draft_{k-1}]
      const int k = len - 1;
      int accepted = 0;
      while (accepted < k && accepted < static_cast<int>(r->drafts.size()) &&
             r->drafts[accepted] == sampled[first + accepted])
        ++accepted;
      r->drafts.clear();
      bool done = false;
      int emitted = 0;
      for (int j = 0; j <= accepted && !done; ++j) {
        done = emit(r, sampled[first + j]);
        ++emitted;
      }
      // KV is valid for the input token and for every accepted draft that was emitted
      r->computed += emitted;
      r->table->rewind_to(r->computed - r->dropped);
      r->table->commit();
      if (done) finish(r);
    }
  }
  return events;
}

}  // namespace oxb
