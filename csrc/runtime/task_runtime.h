// Task runtime with the reference extension's Python-visible contract:
//   init(alg_name, params, device_id, rank_id, size) / end()
//   submit_task(...) in three overloads / getResults(task_id)
// (ref hp_cuda.cpp:829-1060, 1073-1080).  Same task ids, same finish-queue
// mapping, same tensor roles, same root/non-root semantics -- but:
//   * workers sleep on condition variables instead of polling every 500 us,
//   * the submitter's stream is ordered before the worker's stream by an event
//     (the reference synchronises an unrelated stream and hopes),
//   * one pass decodes all peers' payloads for a root task,
//   * a failed task reports through getErrors() and the worker keeps serving; a task still
//     unfinished after `task_age_limit` seconds (an init parameter, default 120, 0 = off) is
//     reported there too, so that pollers do not wait for ever,
//   * end() followed by init() starts a fresh runtime (the reference never
//     restarts its threads: hp_cuda.cpp:814),
//   * tensors may live on the CPU, in which case the CPU codec runs (tests).
#pragma once
#include <torch/extension.h>

#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "finish_queue.h"
#include "watchdog.h"
#include "worker_pool.h"

namespace hipress {
namespace runtime {

constexpr int kCompTask = 10;
constexpr int kDecompTask = 20;
constexpr int kRootDecompCompTask = 30;
constexpr int kPowerSgdEncode1 = 40;
constexpr int kPowerSgdEncode2 = 50;
constexpr int kPowerSgdDecode = 60;
constexpr int kBackThreads = 5;  // ref hp_cuda.h:27

struct CompAlg {
  std::string name;
  int enable_random = 0;
  int bitwidth = 0;
  float threshold = 0.f;
  double sample_rate = 0.0;
  double drop_ratio = 0.0;
  int matrix_approximation_rank = 0;
  uint64_t seed = 0;  // addition: base seed of stochastic rounding / sampling
};

struct Task {
  std::string tensor_name;
  torch::Tensor tensor, residual, B, C, M, P, Q;
  int is_root = 0;
  int task_id = 0;
  uint64_t serial = 0;
};

class TaskRuntime {
 public:
  static TaskRuntime& instance();

  bool init(const std::string& alg_name, std::unordered_map<std::string, double> params,
            int device_id, int rank_id, int size);
  bool end();
  bool running() const { return pool_ != nullptr; }

  bool submit_without_residual(const std::string& name, torch::Tensor tensor, torch::Tensor B,
                               torch::Tensor C, int is_root, int task_id);
  bool submit_with_residual(const std::string& name, torch::Tensor tensor, torch::Tensor residual,
                            torch::Tensor B, torch::Tensor C, int is_root, int task_id);
  bool submit_powersgd(const std::string& name, torch::Tensor tensor, torch::Tensor residual,
                       torch::Tensor M, torch::Tensor P, torch::Tensor Q, int task_id);
  std::vector<std::string> get_results(int task_id);
  std::vector<std::string> get_errors();
  int num_threads() const { return pool_ ? pool_->size() : 0; }
  const CompAlg& algorithm() const { return alg_; }
  // fixed staging size of a GradDrop payload (ref hp_cuda.cpp:230)
  int64_t graddrop_staging_bytes(int64_t n) const;

 private:
  TaskRuntime() = default;
  bool submit(Task t);
  void run(Task& t);
  void run_compress(Task& t);
  void run_decompress(Task& t);
  void run_root(Task& t);
  void run_powersgd(Task& t);
  FinishQueue& queue_for(int task_id);

  CompAlg alg_;
  int device_id_ = 0, rank_ = 0, size_ = 1;
  std::unique_ptr<WorkerPool> pool_;
  std::unique_ptr<AgeWatchdog> watchdog_;
  FinishQueue comp_, decomp_, root_;
  std::mutex err_mu_;
  std::vector<std::string> errors_;
  std::mutex map_mu_;
  // device copies of gathered CPU buffers, per tensor name (ref hp_cuda.cpp:153-161)
  std::unordered_map<std::string, torch::Tensor> gathered_;
  std::atomic<uint64_t> serial_{0};
};

}  // namespace runtime
}  // namespace hipress
