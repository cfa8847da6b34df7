// Multi-thread soak of the host runtime, meant to be built with -fsanitize=thread or
// -fsanitize=address,undefined: many threads allocate / share / release blocks of one pool
// (sequence tables with prefix adoption and copy-on-write), a step worker is fed from another
// thread, and at the end every block must be back in the pool.
// Mirrors the reference's only threaded test, the slot-manager soak
// (oxide-engine/src/slot_manager.rs tests), on the refcounted block pool.
#include <atomic>
#include <cstdio>
#include <random>
#include <thread>
#include <vector>

#include "../block_manager.h"
#include "../worker.h"

using namespace oxb;

int main() {
  const int kBlocks = 512, kThreads = 8, kIters = 4000;
  BlockPool pool(kBlocks);
  std::atomic<long> allocs{0}, failures{0};
  std::vector<std::thread> ts;
  for (int t = 0; t < kThreads; ++t) {
    ts.emplace_back([&, t] {
      std::mt19937 rng(1234 + t);
      for (int it = 0; it < kIters; ++it) {
        SequenceBlockTable a(&pool);
        const int n = 1 + static_cast<int>(rng() % 90);
        std::vector<std::pair<int, int>> cow;
        if (!a.advance(n, &cow)) {
          failures.fetch_add(1);
          a.release_all();
          continue;
        }
        a.commit();
        allocs.fetch_add(static_cast<long>(a.blocks().size()));
        // a second sequence shares the full blocks of the first and then diverges
        SequenceBlockTable b(&pool);
        const int full = n / kTokensPerBlock;
        if (full > 0) {
          std::vector<int> prefix(a.blocks().begin(), a.blocks().begin() + full);
          b.adopt_prefix(prefix, full * kTokensPerBlock);
        }
        cow.clear();
        if (!b.advance(1 + static_cast<int>(rng() % 20), &cow)) failures.fetch_add(1);
        if ((rng() & 3) == 0) b.rollback(); else b.commit();
        a.release_all();
        b.release_all();
      }
    });
  }
  // a step worker driven from the main thread while the pool is being hammered
  std::atomic<long> handled{0};
  StepWorker w([&](const StepCommand& c, int* v) { *v = c.arg0 + 1; handled.fetch_add(1); return 0; }, 16, -1,
               50, 200, 50);
  long completed = 0;
  for (int i = 0; i < 5000; ++i) {
    StepCommand c;
    c.seq = static_cast<uint64_t>(i);
    c.arg0 = i;
    while (!w.submit(c)) {
      StepCompletion d;
      if (w.wait(&d, 100)) ++completed;
    }
  }
  StepCompletion d;
  while (completed < 5000 && w.wait(&d, 1000)) ++completed;
  w.stop();
  for (auto& t : ts) t.join();
  const bool ok = pool.num_free() == kBlocks && completed == 5000 && handled.load() == 5000;
  std::printf("soak: allocs=%ld exhausted=%ld free=%d/%d completed=%ld %s\n", allocs.load(), failures.load(),
              pool.num_free(), kBlocks, completed, ok ? "OK" : "FAILED");
  return ok ? 0 : 1;
}
