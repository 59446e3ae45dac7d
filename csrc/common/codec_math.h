// Scalar codec arithmetic shared, source-for-source, by the CPU codecs and the
// sm_100a kernels.  Each function states the rounding sequence of one element
// so that both sides produce identical bits; vectorisation, packing and data
// movement live with the callers.
//
// Payload layouts (all little-endian; N = number of fp32 elements):
//   TBQ       ceil(N/4) bytes, no header; element k of a byte in bits [2k+1:2k];
//             field 0 -> -t, 1 -> 0, 2 -> +t            (ref tbq_body.h:32-37, 70-87)
//   TernGrad  10-byte header {u8 bitwidth, u8 tail, f32 min, f32 max} then
//             ceil(N/dpb) bytes, dpb = 8/bitwidth       (ref terngrad_body.h:216-224)
//   Sparse    {i32 total_bytes = 4 + 8k} {k x i32 index} {k x f32 value}
//                                                       (ref gd_body.h:193-200, 165, 219)
//   ECQ       {i32 total = 10 + M, f32 max, u8 bitwidth, u8 unused} then M bytes
//                                                       (ref ecq_body.h:212, 266-276)
#pragma once
#include "hd.h"
#include "lcg.h"

namespace hipress {

// ---------------------------------------------------------------- accumulation order
// Canonical order in which the decoded values of W ranks are summed: adjacent pairs, level by
// level -- ((v0+v1)+(v2+v3))+((v4+v5)+(v6+v7)) for eight ranks; a rank without a partner moves
// up a level unchanged, so three ranks give (v0+v1)+v2.  fp32 sums depend on the order; every
// replica, the CPU codec and the kernels use this one, which keeps replicas bit-identical and
// lets the kernels read the sum of a pair of ranks from one table entry.  With one payload the
// sum is the decoded value itself; `decoded + out` of the accumulate mode (ref tbq_body.h:53,
// terngrad_body.h:157) is applied to the finished sum.  Overwrites v; v[0] is also returned.
template <int MAXW>
HP_HD float tree_sum(float (&v)[MAXW], int world) {
#pragma unroll
  for (int width = 1; width < MAXW; width <<= 1) {
#pragma unroll
    for (int i = 0; i + width < MAXW; i += 2 * width)
      if (i + width < world) v[i] = hp_add(v[i], v[i + width]);
  }
  return v[0];
}

// ---------------------------------------------------------------- TBQ
// One element of threshold quantisation with residual feedback
// (ref tbq_body.h:75-85).  Updates `r` in place, returns the 2-bit field.
HP_HD uint32_t tbq_quant(float& r, float g, float t) {
  r = hp_add(r, g);
  if (r >= t) {
    r = hp_sub(r, t);
    return 2u;
  }
  if (r <= -t) {
    r = hp_add(r, t);
    return 0u;
  }
  return 1u;
}
// Decoded value of a field: (float(q) - 1) * t  (ref tbq_body.h:36).
HP_HD float tbq_dequant(uint32_t q, float t) {
  return hp_mul(hp_sub(static_cast<float>(q), 1.0f), t);
}
static constexpr uint8_t kTbqEmptyByte = 0x55;  // four "zero" fields

HP_HD int64_t tbq_payload_bytes(int64_t n) { return (n + 3) >> 2; }

// ---------------------------------------------------------------- TernGrad
static constexpr int kTernHeaderBytes = 10;

HP_HD bool tern_bitwidth_ok(int bw) { return bw == 1 || bw == 2 || bw == 4 || bw == 8; }
HP_HD int tern_dpb(int bw) { return 8 / bw; }
HP_HD int64_t tern_payload_bytes(int64_t n, int bw) {
  const int dpb = tern_dpb(bw);
  return kTernHeaderBytes + (n + dpb - 1) / dpb;
}
// Number of padding slots in the last data byte (ref terngrad_body.h:216-217).
HP_HD int tern_tail(int64_t n, int bw) {
  const int dpb = tern_dpb(bw);
  const int rem = static_cast<int>(n % dpb);
  return rem == 0 ? 0 : dpb - rem;
}
// gap = (max - min) / (2^bw - 1), all in fp32 (ref terngrad_body.h:205, 351).
HP_HD float tern_gap(float mn, float mx, int bw) {
  const float levels = static_cast<float>((1 << bw)) - 1.0f;
#if defined(__CUDA_ARCH__)
  return __fdiv_rn(hp_sub(mx, mn), levels);
#else
  return (mx - mn) / levels;
#endif
}
// Compress-side scale: 1 / (gap + 1e-8) evaluated in double, rounded to float
// once (ref terngrad_body.h:206).  The decode side uses `gap` with no epsilon.
HP_HD float tern_gap_inverse(float gap) {
  return static_cast<float>(hp_ddiv(1.0, hp_dadd(static_cast<double>(gap), 1e-8)));
}
// Deterministic level: nearbyint((x - min) * inv)  (ref terngrad_body.h:51-52).
HP_HD uint8_t tern_quant_det(float x, float mn, float inv) {
  return hp_f2u8_trunc(hp_rint(hp_mul(hp_sub(x, mn), inv)));
}
// Stochastic level: trunc((x - min) * inv + u), u from the per-byte generator
// (ref terngrad_body.h:92-94).  u may be exactly 1.0f, so the level can reach
// 2^bw; callers OR `level << (bw*j)` into a uint8_t without clamping, exactly
// like the reference's integer arithmetic.
HP_HD uint8_t tern_quant_rnd(float x, float mn, float inv, float u) {
  return hp_f2u8_trunc(hp_add(hp_mul(hp_sub(x, mn), inv), u));
}
// Decoded value: q * gap + min  (ref terngrad_body.h:126).
HP_HD float tern_dequant(uint32_t q, float gap, float mn) {
  return hp_add(hp_mul(static_cast<float>(q), gap), mn);
}
// Seed of the generator that rounds data byte `byte_index`
// (ref terngrad_body.h:85: srand(timestamp + i), truncated to 32 bits).
HP_HD uint32_t tern_byte_seed(uint64_t seed, int64_t byte_index) {
  return static_cast<uint32_t>(seed + static_cast<uint64_t>(byte_index));
}

// Quantise up to dpb consecutive elements into one data byte.
//   count   elements available (dpb for full bytes, fewer for the tail byte)
//   random  stochastic rounding; the tail byte is always deterministic
//           (ref terngrad_body.h:287-297)
// When `ef_out` is non-null the error-feedback residual x - decode(level) is
// written for each element (an addition of this library; the reference's
// TernGrad has no residual).
template <int BW>
HP_HD uint8_t tern_pack_byte(const float* x, int count, float mn, float inv, bool random,
                             uint32_t seed32, float gap, float* ef_out) {
  constexpr int DPB = 8 / BW;
  uint8_t qval = 0;
  Lcg32 rng(seed32);
#pragma unroll
  for (int j = 0; j < DPB; ++j) {
    if (j < count) {
      uint8_t t = random ? tern_quant_rnd(x[j], mn, inv, rng.next_unit())
                         : tern_quant_det(x[j], mn, inv);
      qval = static_cast<uint8_t>(qval | (static_cast<int>(t) << (BW * j)));
      if (ef_out) {
        // residual uses the level that survives in the payload for this field
        const uint32_t kept = (static_cast<uint32_t>(t) & ((1u << BW) - 1u));
        ef_out[j] = hp_sub(x[j], tern_dequant(kept, gap, mn));
      }
    }
  }
  return qval;
}

// ---------------------------------------------------------------- sparse (GradDrop / DGC)
HP_HD int64_t sparse_payload_bytes(int64_t k) { return 4 + 8 * k; }
// k a compressor may emit at most: ceil(N * keep_fraction)  (ref gd_body.h:113).
inline int64_t sparse_expected_k(int64_t n, double keep_fraction) {
  double v = static_cast<double>(n) * keep_fraction;
  int64_t k = static_cast<int64_t>(v);
  if (static_cast<double>(k) < v) ++k;
  return k;
}
inline int64_t sparse_sample_count(int64_t n, double sample_rate) {
  return sparse_expected_k(n, sample_rate);
}
// Index of the threshold inside the descending-sorted sample
// (ref gd_body.h:154: (int)(sample_cnt * s_percent)).
inline int64_t sparse_threshold_rank(int64_t sample_cnt, double keep_fraction) {
  return static_cast<int64_t>(static_cast<double>(sample_cnt) * keep_fraction);
}
// Position drawn by sample x (ref gd_body.h:37-41: per-sample generator seeded
// with t + x, one discarded draw, then rand() % N).
HP_HD uint32_t sparse_sample_index(uint64_t seed, int64_t x, uint32_t n) {
  Lcg32 rng(static_cast<uint32_t>(seed + static_cast<uint64_t>(x)));
  return rng.next_below(n);
}
// |v| as an order-preserving unsigned key (sign cleared; NaNs sort high).
HP_HD uint32_t abs_key(float v) {
#if defined(__CUDA_ARCH__)
  return __float_as_uint(v) & 0x7fffffffu;
#else
  union {
    float f;
    uint32_t u;
  } c;
  c.f = v;
  return c.u & 0x7fffffffu;
#endif
}

// ---------------------------------------------------------------- ECQ
static constexpr int kEcqHeaderBytes = 10;
HP_HD bool ecq_bitwidth_ok(int bw) { return bw == 2 || bw == 4 || bw == 8; }
HP_HD int64_t ecq_payload_bytes(int64_t n, int bw) {
  const int dpb = 8 / bw;
  return kEcqHeaderBytes + (n + dpb - 1) / dpb;
}
// Compensated value v = G + alpha*H (signed; the reference takes fabs and loses
// the sign, ecq_body.h:60 -- here the sign is kept so that decode(v) ~ v).
HP_HD float ecq_compensated(float g, float h, float alpha) { return hp_add(g, hp_mul(alpha, h)); }
// Level of v on the grid {-max + q*gap}: trunc((v + max) * inv + u)
// (ref ecq_body.h:115-116).
HP_HD uint8_t ecq_quant(float v, float mx, float inv, float u) {
  return hp_f2u8_trunc(hp_add(hp_mul(hp_add(v, mx), inv), u));
}
// Decoded value q*gap - max (ref ecq_body.h:320).
HP_HD float ecq_dequant(uint32_t q, float gap, float mx) {
  return hp_sub(hp_mul(static_cast<float>(q), gap), mx);
}
// History update H <- beta*H + (v - decode(q)); algebraically the reference's
// beta*H + (f - t)*gap (ecq_body.h:118).
HP_HD float ecq_history(float h, float beta, float v, float decoded) {
  return hp_add(hp_mul(beta, h), hp_sub(v, decoded));
}
HP_HD float ecq_gap(float mx, int bw) {
  const float s = static_cast<float>((1 << (bw - 1)) - 1);
#if defined(__CUDA_ARCH__)
  return __fdiv_rn(mx, s);
#else
  return mx / s;
#endif
}
HP_HD float ecq_gap_inverse(float gap) {
  return static_cast<float>(hp_ddiv(1.0, static_cast<double>(gap)));
}
static constexpr float kEcqZeroCutoff = 1e-6f;  // ref ecq_body.h:212

}  // namespace hipress
