// Stress test of the host runtime's plain-C++ parts (WorkerPool, FinishQueue, AgeWatchdog),
// built with -fsanitize=thread or -fsanitize=address,undefined by
// `python -m hipress_b200.build --sanitize thread|address` and run by tests/test_sanitizers.py.
// The reference's equivalents carry known races -- one static stream shared by its five
// threads (ref hp_cuda.cpp:789), an unsynchronised round-robin counter (ref hp_cuda.cpp:930) --
// which is why these paths are exercised from several submitting threads at once.
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <set>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

#include "runtime/finish_queue.h"
#include "runtime/watchdog.h"
#include "runtime/worker_pool.h"

using namespace hipress::runtime;

#define CHECK(cond)                                                          \
  do {                                                                       \
    if (!(cond)) {                                                           \
      std::fprintf(stderr, "CHECK failed at line %d: %s\n", __LINE__, #cond); \
      std::exit(1);                                                          \
    }                                                                        \
  } while (0)

static void pool_and_queue() {
  constexpr int kSubmitters = 4, kPerSubmitter = 2000, kWorkers = 5;
  std::atomic<int> started{0}, ran{0};
  FinishQueue fq;
  std::set<std::string> seen;
  {
    WorkerPool pool(kWorkers, [&](int) { ++started; });
    CHECK(started.load() == kWorkers);
    std::atomic<bool> polling{true};
    std::thread poller([&] {   // the Python side polls while workers push
      while (polling.load()) {
        for (auto& k : fq.drain()) seen.insert(k);
        std::this_thread::yield();
      }
    });
    std::vector<std::thread> submitters;
    for (int s = 0; s < kSubmitters; ++s) {
      submitters.emplace_back([&, s] {
        for (int i = 0; i < kPerSubmitter; ++i) {
          const std::string name = std::to_string(s) + "/" + std::to_string(i);
          auto job = [&, name, i](int) {
            ++ran;
            if (i % 97 == 0) throw std::runtime_error("injected failure " + name);
            fq.push(name);
          };
          if (i % 3 == 0) pool.submit_to(i % kWorkers, job);
          else pool.submit(job);
        }
      });
    }
    for (auto& t : submitters) t.join();
    pool.drain();
    polling = false;
    poller.join();
    for (auto& k : fq.drain()) seen.insert(k);
    CHECK(ran.load() == kSubmitters * kPerSubmitter);
    int failures = 0;
    for (int i = 0; i < kPerSubmitter; ++i) failures += (i % 97 == 0);
    CHECK(pool.error_count() == kSubmitters * failures);
    CHECK(!pool.last_error().empty());
    CHECK(int(seen.size()) == kSubmitters * (kPerSubmitter - failures));
    // shutdown with work still queued: queued jobs run, later submissions are refused
    for (int i = 0; i < 100; ++i) pool.submit([&](int) { ++ran; });
    pool.shutdown();
    CHECK(ran.load() == kSubmitters * kPerSubmitter + 100);
    bool refused = false;
    try {
      pool.submit([](int) {});
    } catch (const std::runtime_error&) {
      refused = true;
    }
    CHECK(refused);
  }
}

static void watchdog() {
  std::mutex mu;
  std::vector<std::string> overdue;
  {
    AgeWatchdog dog(0.05, [&](const std::string& label, double age) {
      std::lock_guard<std::mutex> lk(mu);
      CHECK(age > 0.05);
      overdue.push_back(label);
    });
    // many short tasks from several threads: none may be reported
    std::vector<std::thread> ts;
    for (int t = 0; t < 4; ++t)
      ts.emplace_back([&, t] {
        for (uint64_t i = 0; i < 500; ++i) {
          const uint64_t id = uint64_t(t) * 100000 + i;
          dog.track(id, "short");
          dog.done(id);
        }
      });
    for (auto& t : ts) t.join();
    dog.track(999999, "stuck");
    std::this_thread::sleep_for(std::chrono::milliseconds(200));
    dog.done(999999);
    CHECK(dog.in_flight() == 0);
  }
  std::lock_guard<std::mutex> lk(mu);
  CHECK(overdue.size() == 1 && overdue[0] == "stuck");   // reported exactly once
  // a disabled watchdog starts no thread and tracks nothing
  AgeWatchdog off(0.0, [](const std::string&, double) { std::abort(); });
  off.track(1, "x");
  CHECK(off.in_flight() == 0);
}

int main() {
  pool_and_queue();
  watchdog();
  std::puts("runtime_stress: ok");
  return 0;
}
