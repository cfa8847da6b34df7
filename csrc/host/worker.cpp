#include "worker.h"

#include <pthread.h>
#include <sched.h>

#include <chrono>
#include <stdexcept>

namespace oxb {

StepWorker::StepWorker(Handler handler, int capacity, int pin_core, int spin_limit, int yield_limit,
                       int park_us)
    : handler_(std::move(handler)),
      mask_(static_cast<uint32_t>(capacity) - 1),
      cmds_(capacity),
      done_(capacity),
      pin_core_(pin_core),
      spin_limit_(spin_limit),
      yield_limit_(yield_limit),
      park_us_(park_us) {
  if (capacity <= 0 || (capacity & (capacity - 1)) != 0)
    throw std::invalid_argument("StepWorker: capacity must be a power of two");
  thread_ = std::thread([this] { run(); });
}

StepWorker::~StepWorker() { stop(); }

void StepWorker::stop() {
  bool was = stop_.exchange(true);
  cv_.notify_all();
  if (!was && thread_.joinable()) thread_.join();
}

bool StepWorker::submit(const StepCommand& cmd) {
  const uint64_t head = cmd_head_.load(std::memory_order_relaxed);
  // Every command produces one completion: bounding the commands that were submitted but whose
  // completion has not been taken yet bounds both rings.
  if (head - done_tail_.load(std::memory_order_acquire) > mask_) return false;
  cmds_[head & mask_] = cmd;
  cmd_head_.store(head + 1, std::memory_order_release);
  cv_.notify_one();  // only matters when the worker is parked
  return true;
}

bool StepWorker::poll(StepCompletion* out) {
  const uint64_t tail = done_tail_.load(std::memory_order_relaxed);
  if (tail == done_head_.load(std::memory_order_acquire)) return false;
  *out = done_[tail & mask_];
  done_tail_.store(tail + 1, std::memory_order_release);
  return true;
}

bool StepWorker::wait(StepCompletion* out, int timeout_ms) {
  if (poll(out)) return true;
  std::unique_lock<std::mutex> lk(mu_);
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  while (!poll(out)) {
    if (done_cv_.wait_until(lk, deadline) == std::cv_status::timeout) return poll(out);
  }
  return true;
}

WorkerIdleStats StepWorker::idle_stats() const {
  WorkerIdleStats s;
  s.spins = spins_.load();
  s.yields = yields_.load();
  s.parks = parks_.load();
  s.commands = commands_.load();
  return s;
}

void StepWorker::run() {
  if (pin_core_ >= 0) {
    cpu_set_t set;
    CPU_ZERO(&set);
    CPU_SET(pin_core_, &set);
    pinned_ = pthread_setaffinity_np(pthread_self(), sizeof(set), &set) == 0;
  }
  int idle = 0;
  while (true) {
    heartbeat_.fetch_add(1, std::memory_order_relaxed);
    const uint64_t tail = cmd_tail_.load(std::memory_order_relaxed);
    if (tail != cmd_head_.load(std::memory_order_acquire)) {
      idle = 0;
      const StepCommand cmd = cmds_[tail & mask_];
      cmd_tail_.store(tail + 1, std::memory_order_release);
      if (cmd.kind == 2) break;
      StepCompletion c;
      c.seq = cmd.seq;
      const auto t0 = std::chrono::steady_clock::now();
      int value = 0;
      c.status = cmd.kind == 1 ? 0 : handler_(cmd, &value);
      c.value = value;
      c.busy_us = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count();
      // submit() admits a command only while its completion slot is free
      const uint64_t dh = done_head_.load(std::memory_order_relaxed);
      done_[dh & mask_] = c;
      done_head_.store(dh + 1, std::memory_order_release);
      commands_.fetch_add(1, std::memory_order_relaxed);
      {
        std::lock_guard<std::mutex> lk(mu_);
      }
      done_cv_.notify_all();
      continue;
    }
    if (stop_.load(std::memory_order_acquire)) break;
    ++idle;
    if (idle <= spin_limit_) {
      spins_.fetch_add(1, std::memory_order_relaxed);
#if defined(__x86_64__)
      __builtin_ia32_pause();
#endif
    } else if (idle <= yield_limit_) {
      yields_.fetch_add(1, std::memory_order_relaxed);
      std::this_thread::yield();
    } else {
      parks_.fetch_add(1, std::memory_order_relaxed);
      std::unique_lock<std::mutex> lk(mu_);
      cv_.wait_for(lk, std::chrono::microseconds(park_us_));
    }
  }
}

}  // namespace oxb
