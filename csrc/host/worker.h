// Step worker: one host thread per rank that executes step commands handed over through a
// single-producer / single-consumer ring, with the three-phase idle policy of the reference's
// execution worker (spin, then yield, then short timed parks) and an optional core pin.
// Reference: oxide-core/src/worker.rs:10-58 (64-byte command/completion records), :90-138 (idle loop).
#pragma once
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

namespace oxb {

struct alignas(64) StepCommand {
  uint64_t seq = 0;
  int32_t kind = 0;  // 0 = step, 1 = barrier/no-op, 2 = stop
  int32_t arg0 = 0;
  int64_t arg1 = 0;
  uint8_t pad[40] = {0};
};
static_assert(sizeof(StepCommand) == 64, "one cache line per command");

struct alignas(64) StepCompletion {
  uint64_t seq = 0;
  int32_t status = 0;
  int32_t value = 0;
  double busy_us = 0.0;
  uint8_t pad[40] = {0};
};
static_assert(sizeof(StepCompletion) == 64, "one cache line per completion");

struct WorkerIdleStats {
  uint64_t spins = 0, yields = 0, parks = 0, commands = 0;
};

class StepWorker {
 public:
  using Handler = std::function<int(const StepCommand&, int* value)>;
  // capacity: power of two. pin_core < 0: no pinning.
  StepWorker(Handler handler, int capacity = 64, int pin_core = -1, int spin_limit = 200,
             int yield_limit = 2000, int park_us = 50);
  ~StepWorker();
  StepWorker(const StepWorker&) = delete;
  StepWorker& operator=(const StepWorker&) = delete;

  bool submit(const StepCommand& cmd);      // false when the ring is full
  bool poll(StepCompletion* out);           // false when no completion is ready
  bool wait(StepCompletion* out, int timeout_ms);
  void stop();
  uint64_t heartbeat() const { return heartbeat_.load(std::memory_order_relaxed); }
  WorkerIdleStats idle_stats() const;
  bool pinned() const { return pinned_; }

 private:
  void run();
  Handler handler_;
  const uint32_t mask_;
  std::vector<StepCommand> cmds_;
  std::vector<StepCompletion> done_;
  alignas(64) std::atomic<uint64_t> cmd_head_{0};   // written by the producer
  alignas(64) std::atomic<uint64_t> cmd_tail_{0};   // written by the worker
  alignas(64) std::atomic<uint64_t> done_head_{0};  // written by the worker
  alignas(64) std::atomic<uint64_t> done_tail_{0};  // written by the consumer
  alignas(64) std::atomic<uint64_t> heartbeat_{0};
  std::atomic<bool> stop_{false};
  std::atomic<uint64_t> spins_{0}, yields_{0}, parks_{0}, commands_{0};
  std::mutex mu_;
  std::condition_variable cv_;
  std::condition_variable done_cv_;
  const int pin_core_, spin_limit_, yield_limit_, park_us_;
  bool pinned_ = false;
  std::thread thread_;
};

}  // namespace oxb
