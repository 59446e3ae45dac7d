#include "task_runtime.h"

#include <ATen/cuda/CUDAContext.h>
#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include <cmath>

#include "../common/host_utils.h"
#include "../ops/ops.h"

namespace hipress {
namespace runtime {

TaskRuntime& TaskRuntime::instance() {
  static TaskRuntime* rt = new TaskRuntime();  // leaked: must outlive worker threads at exit
  return *rt;
}

bool TaskRuntime::init(const std::string& alg_name, std::unordered_map<std::string, double> params,
                       int device_id, int rank_id, int size) {
  if (pool_) end();
  CompAlg alg;
  alg.name = alg_name;
  int threads = kBackThreads;
  if (alg_name == "terngrad") {
    alg.enable_random = int(params["enable_random"]);
    alg.bitwidth = int(params["bitwidth"]);
  } else if (alg_name == "tbq") {
    alg.threshold = float(params["threshold"]);
    threads = 1;  // ref hp_cuda.cpp:843: tbq runs single-threaded
  } else if (alg_name == "graddrop") {
    alg.drop_ratio = params["drop_ratio"];
    alg.sample_rate = params["sample_rate"];
  } else if (alg_name == "powersgd") {
    alg.matrix_approximation_rank = int(params["matrix_approximation_rank"]);
  } else {
    return false;  // ref hp_cuda.cpp:851-854
  }
  if (params.count("seed")) alg.seed = uint64_t(params["seed"]);
  if (params.count("num_threads")) threads = std::max(1, int(params["num_threads"]));
  alg_ = alg;
  device_id_ = device_id;
  rank_ = rank_id;
  size_ = size;
  serial_ = 0;
  comp_.drain();
  decomp_.drain();
  root_.drain();
  {
    std::lock_guard<std::mutex> lk(err_mu_);
    errors_.clear();
  }
  pool_ = std::make_unique<WorkerPool>(threads, [](int) {});
  const double age_limit = params.count("task_age_limit") ? params["task_age_limit"] : 120.0;
  watchdog_ = std::make_unique<AgeWatchdog>(age_limit, [this](const std::string& label, double age) {
    std::lock_guard<std::mutex> lk(err_mu_);
    errors_.push_back(label + ": still running after " + std::to_string(age) + " s (task age limit)");
  });
  return true;
}

bool TaskRuntime::end() {
  if (pool_) {
    pool_->drain();
    pool_->shutdown();
    pool_.reset();
  }
  watchdog_.reset();
  std::lock_guard<std::mutex> lk(map_mu_);
  gathered_.clear();
  return true;
}

int64_t TaskRuntime::graddrop_staging_bytes(int64_t n) const {
  return 4 + int64_t(int(2 * std::ceil(double(n) * (1 - alg_.drop_ratio)))) * 4;
}

FinishQueue& TaskRuntime::queue_for(int task_id) {
  switch (task_id) {
    case kCompTask:
    case kPowerSgdEncode1: return comp_;
    case kDecompTask:
    case kPowerSgdDecode: return decomp_;
    default: return root_;  // 30 and 50 (ref hp_cuda.cpp:1040-1060)
  }
}

std::vector<std::string> TaskRuntime::get_results(int task_id) {
  switch (task_id) {
    case kCompTask: case kPowerSgdEncode1:
    case kDecompTask: case kPowerSgdDecode:
    case kRootDecompCompTask: case kPowerSgdEncode2:
      return queue_for(task_id).drain();
    default:
      return {};
  }
}

std::vector<std::string> TaskRuntime::get_errors() {
  std::lock_guard<std::mutex> lk(err_mu_);
  std::vector<std::string> out;
  out.swap(errors_);
  return out;
}

namespace {
void check_input(const torch::Tensor& t, const char* name) {
  TORCH_CHECK(t.defined(), name, " is undefined");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}
}  // namespace

bool TaskRuntime::submit_without_residual(const std::string& name, torch::Tensor tensor,
                                          torch::Tensor B, torch::Tensor C, int is_root,
                                          int task_id) {
  check_input(tensor, "tensor");
  check_input(B, "B");
  check_input(C, "C");
  if (HP_UNLIKELY(is_root != 0 && is_root != 1)) return false;
  if (task_id != kCompTask && task_id != kDecompTask && task_id != kRootDecompCompTask) return false;
  Task t;
  t.tensor_name = name;
  t.tensor = tensor;
  t.B = B;
  t.C = C;
  t.is_root = is_root;
  t.task_id = task_id;
  return submit(std::move(t));
}

bool TaskRuntime::submit_with_residual(const std::string& name, torch::Tensor tensor,
                                       torch::Tensor residual, torch::Tensor B, torch::Tensor C,
                                       int is_root, int task_id) {
  check_input(tensor, "tensor");
  check_input(residual, "residual");
  check_input(B, "B");
  check_input(C, "C");
  if (HP_UNLIKELY(is_root != 0 && is_root != 1)) return false;
  if (task_id != kCompTask && task_id != kDecompTask && task_id != kRootDecompCompTask) return false;
  Task t;
  t.tensor_name = name;
  t.tensor = tensor;
  t.residual = residual;
  t.B = B;
  t.C = C;
  t.is_root = is_root;
  t.task_id = task_id;
  return submit(std::move(t));
}

bool TaskRuntime::submit_powersgd(const std::string& name, torch::Tensor tensor,
                                  torch::Tensor residual, torch::Tensor M, torch::Tensor P,
                                  torch::Tensor Q, int task_id) {
  check_input(tensor, "tensor");
  check_input(residual, "residual");
  check_input(M, "M");
  check_input(P, "P");
  check_input(Q, "Q");
  if (task_id != kPowerSgdEncode1 && task_id != kPowerSgdEncode2 && task_id != kPowerSgdDecode)
    return false;
  Task t;
  t.tensor_name = name;
  t.tensor = tensor;
  t.residual = residual;
  t.M = M;
  t.P = P;
  t.Q = Q;
  t.task_id = task_id;
  return submit(std::move(t));
}

bool TaskRuntime::submit(Task t) {
  TORCH_CHECK(pool_ != nullptr && pool_->alive(), "hipress runtime is not initialised (call init first)");
  t.serial = serial_.fetch_add(1);
  // order the worker's stream after whatever the caller has queued so far
  std::shared_ptr<at::cuda::CUDAEvent> ready;
  if (t.tensor.is_cuda()) {
    ready = std::make_shared<at::cuda::CUDAEvent>();
    ready->record(at::cuda::getCurrentCUDAStream(t.tensor.get_device()));
  }
  const uint64_t serial = t.serial;
  watchdog_->track(serial, t.tensor_name + " (task " + std::to_string(t.task_id) + ")");
  pool_->submit([this, t, ready, serial](int) mutable {
    try {
      if (t.tensor.is_cuda()) {
        c10::cuda::CUDAGuard dev(t.tensor.device());
        // one high-priority stream per worker thread and device, taken from torch's pool
        thread_local std::unordered_map<int, c10::cuda::CUDAStream> streams;
        const int device = t.tensor.get_device();
        auto it = streams.find(device);
        if (it == streams.end())
          it = streams.emplace(device, c10::cuda::getStreamFromPool(/*isHighPriority=*/true, device)).first;
        c10::cuda::CUDAStream stream = it->second;
        c10::cuda::CUDAStreamGuard sg(stream);
        ready->block(stream);
        run(t);
        stream.synchronize();
      } else {
        run(t);
      }
      queue_for(t.task_id).push(t.tensor_name);
    } catch (const std::exception& e) {
      std::lock_guard<std::mutex> lk(err_mu_);
      errors_.push_back(t.tensor_name + ": " + e.what());
    }
    watchdog_->done(serial);
  });
  return true;
}

void TaskRuntime::run(Task& t) {
  switch (t.task_id) {
    case kCompTask: run_compress(t); break;
    case kDecompTask: run_decompress(t); break;
    case kRootDecompCompTask: run_root(t); break;
    default: run_powersgd(t); break;
  }
}

namespace {
uint64_t task_seed(const CompAlg& alg, const Task& t) {
  return alg.seed + 0x9E3779B97F4A7C15ull * (t.serial + 1);
}
// bytes of payload a task moves between B and C
int64_t staged_bytes(const TaskRuntime& rt, const Task& t) {
  if (rt.algorithm().name == "graddrop") return rt.graddrop_staging_bytes(t.tensor.numel());
  if (rt.algorithm().name == "tbq") return ops::tbq_payload_bytes(t.tensor.numel());
  return t.B.numel();  // terngrad: B is sized exactly
}
}  // namespace

void TaskRuntime::run_compress(Task& t) {
  const auto& a = alg_;
  auto g = t.tensor.view(-1);
  if (a.name == "terngrad") {
    ops::terngrad_compress(g, t.B, a.bitwidth, a.enable_random != 0, int64_t(task_seed(a, t)),
                           c10::nullopt);
  } else if (a.name == "tbq") {
    ops::tbq_compress(g, t.residual.view(-1), t.B, a.threshold);
  } else if (a.name == "graddrop") {
    ops::sparse_compress(g, t.residual.view(-1), t.B, a.sample_rate, 1.0 - a.drop_ratio,
                         int64_t(task_seed(a, t)), true);
  } else {
    TORCH_CHECK(false, "task ", t.task_id, " is not valid for algorithm ", a.name);
  }
  const int64_t bytes = std::min<int64_t>(staged_bytes(*this, t), std::min(t.B.numel(), t.C.numel()));
  t.C.slice(0, 0, bytes).copy_(t.B.slice(0, 0, bytes), /*non_blocking=*/true);
}

void TaskRuntime::run_decompress(Task& t) {
  const auto& a = alg_;
  const int64_t bytes = std::min<int64_t>(staged_bytes(*this, t), std::min(t.B.numel(), t.C.numel()));
  t.B.slice(0, 0, bytes).copy_(t.C.slice(0, 0, bytes), /*non_blocking=*/true);
  auto out = t.tensor.view(-1);
  const bool add = t.is_root != 0;  // is_root doubles as "accumulate" (ref hp_cuda.cpp:236, 417, 567)
  if (a.name == "terngrad") {
    ops::terngrad_decompress({t.B}, out, add, 1.0, alg_.bitwidth);
  } else if (a.name == "tbq") {
    ops::tbq_decompress({t.B}, out, a.threshold, add, 1.0);
  } else if (a.name == "graddrop") {
    ops::sparse_decompress({t.B.slice(0, 0, bytes)}, out, add, 1.0);
  } else {
    TORCH_CHECK(false, "task ", t.task_id, " is not valid for algorithm ", a.name);
  }
}

void TaskRuntime::run_root(Task& t) {
  // C holds `size` payload slices of equal length, slice r from rank r.  All
  // slices but this rank's own are decoded into the dense tensor one after
  // another in ascending rank order -- the reference's order of accumulation,
  // own tensor first -- then the dense tensor is compressed into B and copied
  // to C[0:len]  (ref hp_cuda.cpp:241-271, 421-449, 571-601).
  const auto& a = alg_;
  const int64_t len = (a.name == "terngrad") ? t.B.numel() : staged_bytes(*this, t);
  TORCH_CHECK(t.C.numel() >= len * size_, "gathered buffer C holds fewer than size x payload bytes");
  torch::Tensor gathered;
  if (t.tensor.is_cuda() && !t.C.is_cuda()) {
    std::lock_guard<std::mutex> lk(map_mu_);
    auto it = gathered_.find(t.tensor_name);
    if (it == gathered_.end() || it->second.numel() != t.C.numel())
      it = gathered_.insert_or_assign(t.tensor_name, torch::empty_like(t.C, t.tensor.options().dtype(torch::kUInt8))).first;
    gathered = it->second;
    gathered.copy_(t.C, /*non_blocking=*/true);
  } else {
    gathered = t.C;
  }
  std::vector<torch::Tensor> peers;
  for (int r = 0; r < size_; ++r)
    if (r != rank_) peers.push_back(gathered.slice(0, int64_t(r) * len, int64_t(r + 1) * len));
  auto out = t.tensor.view(-1);
  const bool add = t.is_root != 0;
  for (size_t i = 0; i < peers.size(); ++i) {
    // the first peer overwrites unless the task accumulates; every later one adds
    const bool add_to = add || i > 0;
    if (a.name == "terngrad") ops::terngrad_decompress({peers[i]}, out, add_to, 1.0, alg_.bitwidth);
    else if (a.name == "tbq") ops::tbq_decompress({peers[i]}, out, a.threshold, add_to, 1.0);
    else if (a.name == "graddrop") ops::sparse_decompress({peers[i]}, out, add_to, 1.0);
    else TORCH_CHECK(false, "task 30 is not valid for algorithm ", a.name);
  }
  run_compress(t);
}

void TaskRuntime::run_powersgd(Task& t) {
  TORCH_CHECK(alg_.name == "powersgd", "task ", t.task_id, " needs algorithm powersgd");
  switch (t.task_id) {
    case kPowerSgdEncode1: ops::powersgd_encode1(t.tensor, t.residual, t.Q, t.M, t.P); break;
    case kPowerSgdEncode2: ops::powersgd_encode2(t.P, t.M, t.Q); break;
    default: ops::powersgd_decode(t.P, t.Q, t.M, t.residual, t.tensor); break;
  }
}

}  // namespace runtime
}  // namespace hipress
