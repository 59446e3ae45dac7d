// 32-bit linear congruential generator shared by the CPU codecs and the
// sm_100a kernels (stochastic rounding, threshold sampling).
//
// Same sequence as the reference's naive_random (ZQ_CPP_LIB/naive_random.hpp:14-34):
//   x <- 1103515245 * x + 12345  (mod 2^32)
// seeding stores the seed and throws the first draw away (naive_random.hpp:25-28).
// Seeds are truncated to 32 bits by the caller, as the reference's srand()
// parameter type does.
#pragma once
#include "hd.h"

namespace hipress {

struct Lcg32 {
  uint32_t x;
  HP_HD explicit Lcg32(uint32_t seed) : x(seed) { next(); }
  HP_HD uint32_t next() {
    x = 1103515245u * x + 12345u;
    return x;
  }
  // Uniform float on [0, 1] *inclusive*.  The reference divides in double and
  // rounds to float, float(double(raw) / 4294967295.0), so the top 129 raw
  // values come out as exactly 1.0f (naive_random.hpp:53-69 with bounds (0,1)).
  // Multiplying by the double reciprocal instead gives the same float for every
  // one of the 2^32 raw values (checked exhaustively) and costs one double
  // multiply where the division costs a long instruction sequence on the GPU.
  HP_HD float next_unit() { return unit_from_raw(next()); }
  HP_HD static float unit_from_raw(uint32_t raw) {
    return static_cast<float>(hp_dmul(static_cast<double>(raw), 1.0 / 4294967295.0));
  }
  HP_HD static float unit_from_raw_by_division(uint32_t raw) {
    return static_cast<float>(hp_ddiv(static_cast<double>(raw), 4294967295.0));
  }
  // Uniform integer on [0, range): raw % range (naive_random.hpp:36-51 with
  // lower bound 0 and upper bound range-1).
  HP_HD uint32_t next_below(uint32_t range) { return next() % range; }
};

// After `seed`, the generator state following the discarded draw is affine in
// the seed; kernels that seed one generator per output byte use this to jump
// straight to the first kept draw.
HP_HD uint32_t lcg_step(uint32_t x) { return 1103515245u * x + 12345u; }

}  // namespace hipress
