// The threaded CPU codecs (TBQ, TernGrad: csrc/codec_cpu/codec_cpu.cpp) under ThreadSanitizer or
// AddressSanitizer + UBSan: several threads split one tensor, and two caller threads run codecs
// on their own tensors at the same time.  Built by
// `python -m hipress_b200.build --sanitize thread|address` and run by tests/test_sanitizers.py.
// Every result is also compared with the one-thread run.  (The reference's host path has one
// thread and no test.)
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>

#include "codec_cpu/codec_cpu.h"
#include "common/codec_math.h"

using namespace hipress;

#define CHECK(cond)                                                          \
  do {                                                                       \
    if (!(cond)) {                                                           \
      std::fprintf(stderr, "CHECK failed at line %d: %s\n", __LINE__, #cond); \
      std::exit(1);                                                          \
    }                                                                        \
  } while (0)

namespace {

struct Result {
  std::vector<uint8_t> tbq, tern;
  std::vector<float> residual, ef, dense;
};

std::vector<float> make_input(int64_t n, uint32_t seed) {
  std::vector<float> g(static_cast<size_t>(n));
  uint32_t x = seed * 2654435761u + 12345u;
  for (auto& v : g) {
    x = x * 1664525u + 1013904223u;
    v = (float(x >> 8) / float(1 << 24) - 0.5f) * 0.02f;
  }
  return g;
}

Result run(const std::vector<float>& g) {
  const int64_t n = int64_t(g.size());
  Result r;
  r.residual.assign(size_t(n), 0.f);
  r.tbq.assign(size_t(tbq_payload_bytes(n)), 0);
  cpu::tbq_compress(g.data(), r.residual.data(), n, 0.004f, r.tbq.data());
  r.dense.assign(size_t(n), 0.25f);
  cpu::tbq_decompress(r.tbq.data(), n, 0.004f, r.dense.data(), 1);
  r.ef.assign(size_t(n), 0.f);
  r.tern.assign(size_t(tern_payload_bytes(n, 2)), 0);
  CHECK(cpu::terngrad_compress(g.data(), n, 2, 1, 7, r.tern.data(), int64_t(r.tern.size()), r.ef.data()) == 0);
  std::vector<float> d(size_t(n), 0.f);
  CHECK(cpu::terngrad_decompress(r.tern.data(), int64_t(r.tern.size()), d.data(), n, 0) == n);
  r.dense.insert(r.dense.end(), d.begin(), d.end());
  return r;
}

bool same(const Result& a, const Result& b) {
  return a.tbq == b.tbq && a.tern == b.tern &&
         std::memcmp(a.residual.data(), b.residual.data(), a.residual.size() * 4) == 0 &&
         std::memcmp(a.ef.data(), b.ef.data(), a.ef.size() * 4) == 0 &&
         std::memcmp(a.dense.data(), b.dense.data(), a.dense.size() * 4) == 0;
}

}  // namespace

int main() {
  const int64_t n = (int64_t(1) << 20) + 3;
  const std::vector<float> g0 = make_input(n, 1), g1 = make_input(n, 2);
  cpu::set_threads(1);
  const Result ref0 = run(g0), ref1 = run(g1);
  cpu::set_threads(6);
  CHECK(cpu::get_threads() == 6);
  CHECK(same(run(g0), ref0));
  // two callers at once, each splitting its own tensor
  Result a, b;
  std::thread ta([&] { a = run(g0); });
  std::thread tb([&] { b = run(g1); });
  ta.join();
  tb.join();
  CHECK(same(a, ref0));
  CHECK(same(b, ref1));
  cpu::set_threads(1);
  std::printf("codec_threads: ok\n");
  return 0;
}
