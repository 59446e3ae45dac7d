// A small pool of worker threads, each with its own FIFO of closures.
//
// Workers sleep on a condition variable and wake when work arrives (the
// reference's workers poll their queue on a fixed 500 us cycle,
// ref hp_cuda.cpp:174-184).  Submission is round-robin over the queues, or to
// an explicit worker when ordering between tasks matters.  An exception thrown
// by a task is caught, recorded and reported through `last_error()`; the worker
// keeps running (in the reference the thread prints and exits, after which
// every poll hangs: hp_cuda.cpp:805-809).
#pragma once
#include <atomic>
#include <condition_variable>
#include <deque>
#include <functional>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

namespace hipress {
namespace runtime {

class WorkerPool {
 public:
  using Job = std::function<void(int /*worker index*/)>;

  // `on_start` runs once in each worker thread before it takes work (device
  // guard, stream creation).
  WorkerPool(int num_workers, std::function<void(int)> on_start)
      : workers_(static_cast<size_t>(num_workers)) {
    for (int i = 0; i < num_workers; ++i) {
      auto& w = workers_[static_cast<size_t>(i)];
      w = std::make_unique<Worker>();
      w->thread = std::thread([this, i, on_start] { loop(i, on_start); });
    }
    // wait until every worker finished its start-up hook
    for (auto& w : workers_) {
      std::unique_lock<std::mutex> lk(w->mu);
      w->cv_idle.wait(lk, [&] { return w->started; });
    }
  }

  ~WorkerPool() { shutdown(); }

  int size() const { return static_cast<int>(workers_.size()); }

  // Returns the index of the worker that got the job.
  int submit(Job job) {
    const int i = static_cast<int>(next_.fetch_add(1, std::memory_order_relaxed) % workers_.size());
    submit_to(i, std::move(job));
    return i;
  }

  void submit_to(int i, Job job) {
    auto& w = *workers_.at(static_cast<size_t>(i));
    {
      std::lock_guard<std::mutex> lk(w.mu);
      if (w.stop) throw std::runtime_error("hipress runtime: worker pool is shut down");
      w.jobs.push_back(std::move(job));
      ++w.pending;
    }
    w.cv_work.notify_one();
  }

  // Blocks until every job submitted so far has run.
  void drain() {
    for (auto& w : workers_) {
      std::unique_lock<std::mutex> lk(w->mu);
      w->cv_idle.wait(lk, [&] { return w->pending == 0; });
    }
  }

  void shutdown() {
    for (auto& w : workers_) {
      {
        std::lock_guard<std::mutex> lk(w->mu);
        w->stop = true;
      }
      w->cv_work.notify_all();
    }
    for (auto& w : workers_)
      if (w->thread.joinable()) w->thread.join();
  }

  bool alive() const {
    for (auto& w : workers_)
      if (w->stop) return false;
    return !workers_.empty();
  }

  std::string last_error() {
    std::lock_guard<std::mutex> lk(err_mu_);
    return last_error_;
  }
  int error_count() const { return error_count_.load(); }

 private:
  struct Worker {
    std::thread thread;
    std::mutex mu;
    std::condition_variable cv_work, cv_idle;
    std::deque<Job> jobs;
    int pending = 0;
    bool stop = false;
    bool started = false;
  };

  void loop(int index, const std::function<void(int)>& on_start) {
    auto& w = *workers_[static_cast<size_t>(index)];
    try {
      if (on_start) on_start(index);
    } catch (const std::exception& e) {
      record(e.what());
    }
    {
      std::lock_guard<std::mutex> lk(w.mu);
      w.started = true;
    }
    w.cv_idle.notify_all();
    for (;;) {
      Job job;
      {
        std::unique_lock<std::mutex> lk(w.mu);
        w.cv_work.wait(lk, [&] { return w.stop || !w.jobs.empty(); });
        if (w.jobs.empty()) return;  // stop requested and queue drained
        job = std::move(w.jobs.front());
        w.jobs.pop_front();
      }
      try {
        job(index);
      } catch (const std::exception& e) {
        record(e.what());
      } catch (...) {
        record("unknown exception in worker task");
      }
      {
        std::lock_guard<std::mutex> lk(w.mu);
        --w.pending;
      }
      w.cv_idle.notify_all();
    }
  }

  void record(const std::string& what) {
    std::lock_guard<std::mutex> lk(err_mu_);
    last_error_ = what;
    ++error_count_;
  }

  std::vector<std::unique_ptr<Worker>> workers_;
  std::atomic<uint64_t> next_{0};
  std::mutex err_mu_;
  std::string last_error_;
  std::atomic<int> error_count_{0};
};

}  // namespace runtime
}  // namespace hipress
