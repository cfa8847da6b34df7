// Python bindings of the C++ host runtime (extension `oxb_host`): block pool, sequence block
// tables, radix prefix cache and the continuous-batching scheduler core.
#include <cstring>
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/functional.h>
#include <pybind11/stl.h>

#include "block_manager.h"
#include "radix_cache.h"
#include "scheduler.h"
#include "worker.h"

namespace py = pybind11;
using namespace oxb;

namespace {

template <typename T>
py::array_t<T> to_array(const std::vector<T>& v) {
  py::array_t<T> a(static_cast<py::ssize_t>(v.size()));
  if (!v.empty()) std::memcpy(a.mutable_data(), v.data(), v.size() * sizeof(T));
  return a;
}

std::vector<int32_t> from_array(const py::array_t<int32_t, py::array::c_style | py::array::forcecast>& a) {
  return std::vector<int32_t>(a.data(), a.data() + a.size());
}

}  // namespace

PYBIND11_MODULE(oxb_host, m) {
  m.doc() = "C++ host runtime of the B200-native Oxide engine";
  m.attr("TOKENS_PER_BLOCK") = kTokensPerBlock;
  // Chained FNV-1a hash of every whole block of a token list: hash_i = fnv1a(bytes of block i, seeded
  // with offset_basis ^ hash_{i-1}); the identity of the prefix that a KV block completes (KV tiers).
  m.def("prefix_hashes", [](py::array_t<int32_t, py::array::c_style | py::array::forcecast> tokens, int block) {
    const int32_t* t = tokens.data();
    const py::ssize_t n = tokens.size();
    py::list out;
    if (block <= 0) return out;
    uint64_t prev = 0;
    for (py::ssize_t i = 0; i + block <= n; i += block) {
      uint64_t h = 0xCBF29CE484222325ull ^ prev;
      for (int j = 0; j < block; ++j) {
        const uint32_t v = static_cast<uint32_t>(t[i + j]);
        for (int b = 0; b < 4; ++b) {
          h ^= (v >> (8 * b)) & 0xFFu;
          h *= 0x100000001B3ull;
        }
      }
      out.append(py::int_(h));
      prev = h;
    }
    return out;
  });

  py::class_<BlockPool>(m, "BlockPool")
      .def(py::init<int>())
      .def("num_blocks", &BlockPool::num_blocks)
      .def("num_free", &BlockPool::num_free)
      .def("allocate", &BlockPool::allocate)
      .def("retain", &BlockPool::retain)
      .def("release", &BlockPool::release)
      .def("ref_count", &BlockPool::ref_count);

  py::class_<SequenceBlockTable>(m, "SequenceBlockTable")
      .def(py::init<BlockPool*>(), py::keep_alive<1, 2>())
      .def("blocks", [](const SequenceBlockTable& t) { return t.blocks(); })
      .def("num_tokens", &SequenceBlockTable::num_tokens)
      .def("committed_tokens", &SequenceBlockTable::committed_tokens)
      .def("adopt_prefix", &SequenceBlockTable::adopt_prefix)
      .def("advance",
           [](SequenceBlockTable& t, int n) {
             std::vector<std::pair<int, int>> cow;
             bool ok = t.advance(n, &cow);
             return py::make_tuple(ok, cow);
           })
      .def("commit", &SequenceBlockTable::commit)
      .def("rewind_to", &SequenceBlockTable::rewind_to)
      .def("rollback", &SequenceBlockTable::rollback)
      .def("prune_heavy_hitters", &SequenceBlockTable::prune_heavy_hitters, py::arg("scores"),
           py::arg("sink_blocks") = 1, py::arg("rolling_blocks") = 16,
           py::arg("budget_blocks") = 128)
      .def("release_all", &SequenceBlockTable::release_all);

  py::class_<RadixCache>(m, "RadixCache")
      .def(py::init<BlockPool*>(), py::keep_alive<1, 2>())
      .def("match",
           [](RadixCache& c, const py::array_t<int32_t, py::array::c_style | py::array::forcecast>& t,
              bool leave_one) {
             RadixCache::Match mm = c.match(t.data(), static_cast<int>(t.size()), leave_one);
             return py::make_tuple(mm.blocks, mm.tokens);
           },
           py::arg("tokens"), py::arg("leave_one") = true)
      .def("insert",
           [](RadixCache& c, const py::array_t<int32_t, py::array::c_style | py::array::forcecast>& t,
              const std::vector<int>& blocks) {
             const int n_blocks = std::min<int>(static_cast<int>(blocks.size()),
                                                static_cast<int>(t.size()) / kTokensPerBlock);
             return c.insert(t.data(), blocks.data(), n_blocks);
           })
      .def("evict", &RadixCache::evict, py::arg("want"), py::arg("by_utility") = false)
      .def("clear", &RadixCache::clear)
      .def("cached_blocks", &RadixCache::cached_blocks)
      .def("lookups", &RadixCache::lookups)
      .def("hit_tokens", &RadixCache::hit_tokens)
      .def("lookup_tokens", &RadixCache::lookup_tokens)
      .def("num_nodes", &RadixCache::num_nodes);

  py::class_<SchedulerConfig>(m, "SchedulerConfig")
      .def(py::init<>())
      .def_readwrite("num_blocks", &SchedulerConfig::num_blocks)
      .def_readwrite("max_num_seqs", &SchedulerConfig::max_num_seqs)
      .def_readwrite("max_num_batched_tokens", &SchedulerConfig::max_num_batched_tokens)
      .def_readwrite("max_blocks_per_seq", &SchedulerConfig::max_blocks_per_seq)
      .def_readwrite("chunk_min", &SchedulerConfig::chunk_min)
      .def_readwrite("chunk_max", &SchedulerConfig::chunk_max)
      .def_readwrite("sla_itl_us", &SchedulerConfig::sla_itl_us)
      .def_readwrite("base_us", &SchedulerConfig::base_us)
      .def_readwrite("per_token_us", &SchedulerConfig::per_token_us)
      .def_readwrite("decode_us_per_seq", &SchedulerConfig::decode_us_per_seq)
      .def_readwrite("enable_radix", &SchedulerConfig::enable_radix)
      .def_readwrite("radix_high", &SchedulerConfig::radix_high)
      .def_readwrite("radix_low", &SchedulerConfig::radix_low)
      .def_readwrite("sla_budget", &SchedulerConfig::sla_budget)
      .def_readwrite("context_shift", &SchedulerConfig::context_shift)
      .def_readwrite("shift_keep_tokens", &SchedulerConfig::shift_keep_tokens)
      .def_readwrite("shift_step_tokens", &SchedulerConfig::shift_step_tokens);

  py::class_<TokenEvent>(m, "TokenEvent")
      .def_readonly("req_id", &TokenEvent::req_id)
      .def_readonly("token", &TokenEvent::token)
      .def_readonly("finished", &TokenEvent::finished)
      .def_readonly("reason", &TokenEvent::reason)
      .def("__repr__", [](const TokenEvent& e) {
        return "TokenEvent(req_id=" + std::to_string(e.req_id) + ", token=" +
               std::to_string(e.token) + ", finished=" + (e.finished ? "True" : "False") +
               ", reason='" + e.reason + "')";
      });

  py::class_<StepPlan>(m, "StepPlan")
      .def_readonly("n_tokens", &StepPlan::n_tokens)
      .def_readonly("n_decode", &StepPlan::n_decode)
      .def_readonly("n_prefill", &StepPlan::n_prefill)
      .def_readonly("max_blocks", &StepPlan::max_blocks)
      .def_readonly("prefill_tokens", &StepPlan::prefill_tokens)
      .def_property_readonly("token_ids", [](const StepPlan& p) { return to_array(p.token_ids); })
      .def_property_readonly("positions", [](const StepPlan& p) { return to_array(p.positions); })
      .def_property_readonly("slot_mapping", [](const StepPlan& p) { return to_array(p.slot_mapping); })
      .def_property_readonly("decode_ids", [](const StepPlan& p) { return to_array(p.decode_ids); })
      .def_property_readonly("decode_seq_lens", [](const StepPlan& p) { return to_array(p.decode_seq_lens); })
      .def_property_readonly("decode_block_tables", [](const StepPlan& p) { return to_array(p.decode_block_tables); })
      .def_property_readonly("prefill_ids", [](const StepPlan& p) { return to_array(p.prefill_ids); })
      .def_property_readonly("q_start", [](const StepPlan& p) { return to_array(p.q_start); })
      .def_property_readonly("q_lens", [](const StepPlan& p) { return to_array(p.q_lens); })
      .def_property_readonly("ctx_lens", [](const StepPlan& p) { return to_array(p.ctx_lens); })
      .def_property_readonly("prefill_block_tables", [](const StepPlan& p) { return to_array(p.prefill_block_tables); })
      .def_property_readonly("tile_seq", [](const StepPlan& p) { return to_array(p.tile_seq); })
      .def_property_readonly("tile_q0", [](const StepPlan& p) { return to_array(p.tile_q0); })
      .def_property_readonly("logit_rows", [](const StepPlan& p) { return to_array(p.logit_rows); })
      .def_property_readonly("logit_req", [](const StepPlan& p) { return to_array(p.logit_req); })
      .def_property_readonly("cow_src", [](const StepPlan& p) { return to_array(p.cow_src); })
      .def_property_readonly("cow_dst", [](const StepPlan& p) { return to_array(p.cow_dst); });

  py::class_<Scheduler>(m, "Scheduler")
      .def(py::init<const SchedulerConfig&>())
      .def("add_request",
           [](Scheduler& s, int64_t id,
              const py::array_t<int32_t, py::array::c_style | py::array::forcecast>& prompt,
              int max_new_tokens, const std::vector<int32_t>& stop_ids, bool ignore_eos) {
             s.add_request(id, from_array(prompt), max_new_tokens, stop_ids, ignore_eos);
           },
           py::arg("id"), py::arg("prompt"), py::arg("max_new_tokens"),
           py::arg("stop_ids") = std::vector<int32_t>{}, py::arg("ignore_eos") = false)
      .def("cancel",
           [](Scheduler& s, int64_t id) {
             std::vector<TokenEvent> ev;
             bool ok = s.cancel(id, &ev);
             return py::make_tuple(ok, ev);
           })
      .def("set_drafts", &Scheduler::set_drafts)
      .def("prune_request", &Scheduler::prune_request, py::arg("id"), py::arg("block_scores"),
           py::arg("sink_blocks") = 1, py::arg("rolling_blocks") = 16, py::arg("budget_blocks") = 128)
      .def("inject_prefill_error", &Scheduler::inject_prefill_error)
      .def("append_forced", &Scheduler::append_forced)
      .def("reserve_ahead", &Scheduler::reserve_ahead)
      .def("radix_cached_blocks", &Scheduler::radix_cached_blocks)
      .def("radix_adopt", &Scheduler::radix_adopt)
      .def("record_evictions", [](Scheduler& s, bool on) { s.radix().record_evictions(on); })
      .def("take_evicted",
           [](Scheduler& s) {
             py::list out;
             for (auto& e : s.radix().take_evicted()) {
               py::array_t<int32_t> toks(static_cast<py::ssize_t>(e.tokens.size()));
               std::memcpy(toks.mutable_data(), e.tokens.data(), e.tokens.size() * sizeof(int32_t));
               out.append(py::make_tuple(toks, e.first_block, e.blocks));
             }
             return out;
           })
      .def("take_events", &Scheduler::take_events)
      .def("schedule", &Scheduler::schedule)
      .def("update",
           [](Scheduler& s, const StepPlan& plan,
              const py::array_t<int32_t, py::array::c_style | py::array::forcecast>& sampled) {
             return s.update(plan, from_array(sampled));
           })
      .def("prefill_budget", &Scheduler::prefill_budget)
      .def("num_waiting", &Scheduler::num_waiting)
      .def("num_running", &Scheduler::num_running)
      .def("num_free_blocks", &Scheduler::num_free_blocks)
      .def("has_work", &Scheduler::has_work)
      .def("preemptions", &Scheduler::preemptions)
      .def("context_shifts", &Scheduler::context_shifts)
      .def("running_ids", &Scheduler::running_ids)
      .def("request_tokens",
           [](const Scheduler& s, int64_t id) -> py::object {
             const Request* r = s.find(id);
             if (r == nullptr) return py::none();
             return to_array(r->tokens);
           })
      .def("request_info",
           [](const Scheduler& s, int64_t id) -> py::object {
             const Request* r = s.find(id);
             if (r == nullptr) return py::none();
             py::dict d;
             d["computed"] = r->computed;
             d["dropped"] = r->dropped;
             d["prompt_len"] = r->prompt_len;
             d["generated"] = r->generated();
             d["prefix_hit"] = r->prefix_hit;
             d["phase"] = static_cast<int>(r->phase);
             d["preemptions"] = r->preemptions;
             d["blocks"] = r->table->blocks();
             return d;
           })
      .def("radix_stats",
           [](Scheduler& s) {
             py::dict d;
             d["lookups"] = s.radix().lookups();
             d["hit_tokens"] = s.radix().hit_tokens();
             d["lookup_tokens"] = s.radix().lookup_tokens();
             d["cached_blocks"] = s.radix().cached_blocks();
             d["nodes"] = s.radix().num_nodes();
             return d;
           })
      .def("alloc_blocks",
           [](Scheduler& s, int n) -> py::object {
             std::vector<int> out;
             for (int i = 0; i < n; ++i) {
               int b = s.pool().allocate();
               if (b < 0) {
                 for (int x : out) s.pool().release(x);
                 return py::none();
               }
               out.push_back(b);
             }
             return py::cast(out);
           })
      .def("release_blocks",
           [](Scheduler& s, const std::vector<int>& blocks) {
             for (int b : blocks) s.pool().release(b);
           })
      .def("radix_insert",
           [](Scheduler& s, const py::array_t<int32_t, py::array::c_style | py::array::forcecast>& t,
              const std::vector<int>& blocks) {
             const int n_blocks = std::min<int>(static_cast<int>(blocks.size()),
                                                static_cast<int>(t.size()) / kTokensPerBlock);
             return s.radix().insert(t.data(), blocks.data(), n_blocks);
           })
      .def("radix_evict", [](Scheduler& s, int want) { return s.radix().evict(want); })
      .def("radix_clear", [](Scheduler& s) { s.radix().clear(); });

  // Step worker: the handler is a Python callable (kind, arg0, arg1) -> int | (int, int); it runs on
  // the worker thread with the GIL held, the waits of the caller release it.
  struct WorkerDeleter {
    void operator()(StepWorker* w) const {
      py::gil_scoped_release rel;  // the worker thread may need the GIL to finish its command
      delete w;
    }
  };
  py::class_<StepWorker, std::unique_ptr<StepWorker, WorkerDeleter>>(m, "StepWorker")
      .def(py::init([](py::function fn, int capacity, int pin_core, int spin_limit, int yield_limit,
                       int park_us) {
             // the callable is reference-counted only under the GIL, wherever the last copy dies
             std::shared_ptr<py::function> fp(new py::function(std::move(fn)), [](py::function* f) {
               py::gil_scoped_acquire gil;
               delete f;
             });
             auto handler = [fp](const StepCommand& c, int* value) -> int {
               py::gil_scoped_acquire gil;
               try {
                 py::object r = (*fp)(c.kind, c.arg0, c.arg1);
                 if (py::isinstance<py::tuple>(r)) {
                   py::tuple t = r.cast<py::tuple>();
                   *value = t[1].cast<int>();
                   return t[0].cast<int>();
                 }
                 return r.is_none() ? 0 : r.cast<int>();
               } catch (py::error_already_set& e) {
                 e.discard_as_unraisable("StepWorker handler");
                 return -1;
               }
             };
             return new StepWorker(handler, capacity, pin_core, spin_limit, yield_limit, park_us);
           }),
           py::arg("handler"), py::arg("capacity") = 64, py::arg("pin_core") = -1,
           py::arg("spin_limit") = 200, py::arg("yield_limit") = 2000, py::arg("park_us") = 50)
      .def("submit",
           [](StepWorker& w, uint64_t seq, int kind, int arg0, int64_t arg1) {
             StepCommand c;
             c.seq = seq;
             c.kind = kind;
             c.arg0 = arg0;
             c.arg1 = arg1;
             return w.submit(c);
           },
           py::arg("seq"), py::arg("kind") = 0, py::arg("arg0") = 0, py::arg("arg1") = 0)
      .def("wait",
           [](StepWorker& w, int timeout_ms) -> py::object {
             StepCompletion c;
             bool ok;
             {
               py::gil_scoped_release rel;
               ok = w.wait(&c, timeout_ms);
             }
             if (!ok) return py::none();
             return py::make_tuple(c.seq, c.status, c.value, c.busy_us);
           },
           py::arg("timeout_ms") = 1000)
      .def("stop",
           [](StepWorker& w) {
             py::gil_scoped_release rel;
             w.stop();
           })
      .def("heartbeat", &StepWorker::heartbeat)
      .def("pinned", &StepWorker::pinned)
      .def("idle_stats", [](const StepWorker& w) {
        WorkerIdleStats s = w.idle_stats();
        py::dict d;
        d["spins"] = s.spins;
        d["yields"] = s.yields;
        d["parks"] = s.parks;
        d["commands"] = s.commands;
        return d;
      });
  m.attr("STEP_COMMAND_BYTES") = sizeof(StepCommand);
  m.attr("STEP_COMPLETION_BYTES") = sizeof(StepCompletion);
}
