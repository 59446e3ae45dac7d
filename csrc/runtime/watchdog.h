// Age limit for in-flight tasks.
//
// In the reference a worker that throws prints and exits, and a task that never finishes is
// never reported: every later poll of getResults spins forever (ref hp_cuda.cpp:805-809,
// 894-902, 1040-1060).  Here every submitted task is tracked from submission to completion; a
// watchdog thread wakes a few times per limit and hands any task older than the limit to a
// callback exactly once (the runtime turns it into a getErrors() entry, so pollers learn of it
// and can stop waiting).  An overdue task is reported, not cancelled: if it finishes later its
// name still reaches the finish queue.  Plain C++ (no torch): stress-tested under sanitizers.
#pragma once
#include <algorithm>
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <functional>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>

namespace hipress {
namespace runtime {

class AgeWatchdog {
 public:
  using Clock = std::chrono::steady_clock;
  using Report = std::function<void(const std::string& label, double age_s)>;

  // limit_s <= 0 disables the watchdog (no thread is started).
  AgeWatchdog(double limit_s, Report report) : limit_s_(limit_s), report_(std::move(report)) {
    if (limit_s_ > 0) thread_ = std::thread([this] { loop(); });
  }
  ~AgeWatchdog() { stop(); }
  AgeWatchdog(const AgeWatchdog&) = delete;
  AgeWatchdog& operator=(const AgeWatchdog&) = delete;

  void track(uint64_t id, const std::string& label) {
    if (limit_s_ <= 0) return;
    std::lock_guard<std::mutex> lk(mu_);
    inflight_[id] = Entry{label, Clock::now(), false};
  }
  void done(uint64_t id) {
    if (limit_s_ <= 0) return;
    std::lock_guard<std::mutex> lk(mu_);
    inflight_.erase(id);
  }
  size_t in_flight() {
    std::lock_guard<std::mutex> lk(mu_);
    return inflight_.size();
  }
  void stop() {
    {
      std::lock_guard<std::mutex> lk(mu_);
      stop_ = true;
    }
    cv_.notify_all();
    if (thread_.joinable()) thread_.join();
  }

 private:
  struct Entry {
    std::string label;
    Clock::time_point since;
    bool reported;
  };

  void loop() {
    const auto period = std::chrono::duration<double>(std::max(0.001, limit_s_ / 4));
    std::unique_lock<std::mutex> lk(mu_);
    while (!stop_) {
      cv_.wait_for(lk, period, [&] { return stop_; });
      if (stop_) break;
      const auto now = Clock::now();
      for (auto& kv : inflight_) {
        Entry& e = kv.second;
        const double age = std::chrono::duration<double>(now - e.since).count();
        if (!e.reported && age > limit_s_) {
          e.reported = true;
          const std::string label = e.label;
          lk.unlock();          // the callback takes the runtime's own locks
          report_(label, age);
          lk.lock();
          break;                // the map may have changed while unlocked: rescan next round
        }
      }
    }
  }

  const double limit_s_;
  Report report_;
  std::mutex mu_;
  std::condition_variable cv_;
  std::unordered_map<uint64_t, Entry> inflight_;
  bool stop_ = false;
  std::thread thread_;
};

}  // namespace runtime
}  // namespace hipress
