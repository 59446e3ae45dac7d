// Queue of finished task names, drained whole by the poller (the reference's FinishQueue:
// a mutex around a std::queue of tensor names, ref hp_cuda.h:81-96, hp_cuda.cpp:135-151).
// Plain C++ (no torch) so that the host runtime can be built and stress-tested under
// ThreadSanitizer / AddressSanitizer without a GPU.
#pragma once
#include <mutex>
#include <string>
#include <vector>

namespace hipress {
namespace runtime {

class FinishQueue {
 public:
  void push(const std::string& key) {
    std::lock_guard<std::mutex> lk(mu_);
    keys_.push_back(key);
  }
  std::vector<std::string> drain() {
    std::lock_guard<std::mutex> lk(mu_);
    std::vector<std::string> out;
    out.swap(keys_);
    return out;
  }

 private:
  std::mutex mu_;
  std::vector<std::string> keys_;
};

}  // namespace runtime
}  // namespace hipress
