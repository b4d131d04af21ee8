// Exercises tib::server::MpscQueue with real producer threads: every item delivered exactly once,
// per-producer order preserved, nothing leaked at destruction (reference server/tests/unit.cpp:17-40
// runs the same kind of check on its queue).  Built by tests/test_server.py, optionally with
// -fsanitize=thread.
#include <atomic>
#include <cstdio>
#include <memory>
#include <thread>
#include <vector>

#include "queue.hpp"

struct Item {
  int producer = -1, sequence = -1;
  std::shared_ptr<int> payload;
};

int main() {
  constexpr int kProducers = 8, kPerProducer = 10000, kRounds = 3;
  for (int round = 0; round < kRounds; ++round) {
    auto live = std::make_shared<int>(0);
    {
      tib::server::MpscQueue<Item> queue;
      std::atomic<bool> go{false};
      std::vector<std::thread> producers;
      for (int p = 0; p < kProducers; ++p)
        producers.emplace_back([&, p] {
          while (!go.load()) std::this_thread::yield();
          for (int i = 0; i < kPerProducer; ++i) queue.push(Item{p, i, live});
        });
      go.store(true);
      std::vector<int> next(kProducers, 0);
      int received = 0;
      Item item;
      while (received < kProducers * kPerProducer) {
        if (!queue.try_pop(item)) { std::this_thread::yield(); continue; }
        if (item.producer < 0 || item.producer >= kProducers || item.sequence != next[item.producer]++) {
          std::printf("order violation: producer %d sequence %d\n", item.producer, item.sequence);
          return 1;
        }
        ++received;
      }
      for (auto& t : producers) t.join();
      if (queue.try_pop(item)) { std::printf("extra item\n"); return 1; }
      for (int p = 0; p < kProducers; ++p) queue.push(Item{p, 0, live});      // left in the queue on purpose
      item = Item();
    }
    if (live.use_count() != 1) { std::printf("leak: %ld payload references alive\n", live.use_count()); return 1; }
  }
  std::printf("ok\n");
  return 0;
}
