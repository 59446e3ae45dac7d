// Host/device portability macros and contraction-free fp32 arithmetic.
//
// The packed payloads produced by this library must be bit-identical to the
// reference's *CPU* codec path (the thrust::host instantiation of
// ZQ_CPP_LIB/gradient_compression_body/*.h compiled for baseline x86-64, which
// has no FMA).  nvcc fuses a*b+c into one FMA by default, so every expression
// whose rounding is visible in a payload or a decoded value goes through
// hp_mul/hp_add/hp_sub, which forbid contraction on the device and are plain
// operators on the host (host objects are built with -ffp-contract=off).
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define HP_HD __host__ __device__ __forceinline__
#define HP_DEV __device__ __forceinline__
#else
#define HP_HD inline
#define HP_DEV inline
#endif

namespace hipress {

HP_HD float hp_mul(float a, float b) {
#if defined(__CUDA_ARCH__)
  return __fmul_rn(a, b);
#else
  return a * b;
#endif
}
HP_HD float hp_add(float a, float b) {
#if defined(__CUDA_ARCH__)
  return __fadd_rn(a, b);
#else
  return a + b;
#endif
}
HP_HD float hp_sub(float a, float b) {
#if defined(__CUDA_ARCH__)
  return __fsub_rn(a, b);
#else
  return a - b;
#endif
}
HP_HD double hp_ddiv(double a, double b) {
#if defined(__CUDA_ARCH__)
  return __ddiv_rn(a, b);
#else
  return a / b;
#endif
}
HP_HD double hp_dadd(double a, double b) {
#if defined(__CUDA_ARCH__)
  return __dadd_rn(a, b);
#else
  return a + b;
#endif
}
HP_HD double hp_dmul(double a, double b) {
#if defined(__CUDA_ARCH__)
  return __dmul_rn(a, b);
#else
  return a * b;
#endif
}

// float -> uint8 the way x86 does it for `static_cast<uint8_t>(float)`:
// truncate toward zero into a 32-bit integer, then keep the low byte.  The
// device's native float->u8 conversion saturates instead, which would differ
// for the (rare) value 2^bitwidth produced when the LCG returns exactly 1.0f.
HP_HD uint8_t hp_f2u8_trunc(float v) {
#if defined(__CUDA_ARCH__)
  return static_cast<uint8_t>(__float2int_rz(v));
#else
  return static_cast<uint8_t>(static_cast<int32_t>(v));
#endif
}

// Round-half-even to an integer value (nearbyint under the default FP mode).
HP_HD float hp_rint(float v) {
#if defined(__CUDA_ARCH__)
  return rintf(v);
#else
  return __builtin_nearbyintf(v);
#endif
}

}  // namespace hipress
