// Small host-side utilities with counterparts in the reference's support layer.
//
//   HP_LIKELY / HP_UNLIKELY   branch hints (ref ZQ_CPP_LIB/likely.h:4-10)
//   fast_abs                  branch-free |x| for int32 / int64 / float / double by bit
//                             manipulation (ref ZQ_CPP_LIB/high_perf_algo/abs.h:9-33); the
//                             float form is what abs_key() in codec_math.h builds on
//   TimeCost                  wall-clock checkpoint timer: start / record(comment) /
//                             report in us, ms or s (ref ZQ_CPP_LIB/time_cost.hpp:10-60);
//                             uses steady_clock instead of gettimeofday.  Device work is
//                             timed with CUDA events elsewhere, never with this.
#pragma once
#include <stdint.h>

#include <chrono>
#include <cstring>
#include <string>
#include <utility>
#include <vector>

#define HP_LIKELY(x) __builtin_expect(!!(x), 1)
#define HP_UNLIKELY(x) __builtin_expect(!!(x), 0)

namespace hipress {

inline int32_t fast_abs(int32_t v) {
  const int32_t m = v >> 31;
  return (v + m) ^ m;
}
inline int64_t fast_abs(int64_t v) {
  const int64_t m = v >> 63;
  return (v + m) ^ m;
}
inline float fast_abs(float v) {
  uint32_t u;
  std::memcpy(&u, &v, 4);
  u &= 0x7fffffffu;
  std::memcpy(&v, &u, 4);
  return v;
}
inline double fast_abs(double v) {
  uint64_t u;
  std::memcpy(&u, &v, 8);
  u &= 0x7fffffffffffffffull;
  std::memcpy(&v, &u, 8);
  return v;
}

class TimeCost {
 public:
  void start() {
    marks_.clear();
    t0_ = clock::now();
  }
  void record(const std::string& comment) { marks_.emplace_back(comment, clock::now()); }
  // (comment, time since the previous mark) in the given unit: 1e6 = us, 1e3 = ms, 1 = s
  std::vector<std::pair<std::string, double>> intervals(double per_second) const {
    std::vector<std::pair<std::string, double>> out;
    auto prev = t0_;
    for (const auto& m : marks_) {
      out.emplace_back(m.first, std::chrono::duration<double>(m.second - prev).count() * per_second);
      prev = m.second;
    }
    return out;
  }
  std::string print_by(double per_second, const char* unit) const {
    std::string s;
    for (const auto& iv : intervals(per_second)) {
      char buf[64];
      std::snprintf(buf, sizeof(buf), "%.3f%s", iv.second, unit);
      s += "[" + iv.first + "]" + buf + "\t";
    }
    return s;
  }
  std::string print_by_us() const { return print_by(1e6, "us"); }
  std::string print_by_ms() const { return print_by(1e3, "ms"); }
  std::string print_by_s() const { return print_by(1.0, "s"); }

 private:
  using clock = std::chrono::steady_clock;
  clock::time_point t0_ = clock::now();
  std::vector<std::pair<std::string, clock::time_point>> marks_;
};

}  // namespace hipress
