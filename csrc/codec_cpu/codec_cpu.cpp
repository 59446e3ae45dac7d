#include "codec_cpu.h"

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstring>
#include <functional>
#include <thread>
#include <vector>

#include "../common/codec_math.h"

namespace hipress {
namespace cpu {

namespace {
std::atomic<int> g_threads{1};
constexpr int64_t kGrainElems = int64_t(1) << 16;   // smallest piece worth a thread

// body(begin, end) over [0, items) in contiguous pieces, one per thread (the caller runs the
// first piece).  `elems_per_item` scales the grain from elements to items (payload bytes).
template <class F>
void parallel_items(int64_t items, int64_t elems_per_item, const F& body) {
  const int want = g_threads.load(std::memory_order_relaxed);
  const int64_t grain = std::max<int64_t>(1, kGrainElems / std::max<int64_t>(1, elems_per_item));
  int64_t pieces = std::min<int64_t>(want, items / grain);
  if (pieces <= 1) {
    if (items > 0) body(int64_t(0), items);
    return;
  }
  const int64_t per = (items + pieces - 1) / pieces;
  std::vector<std::thread> pool;
  pool.reserve(size_t(pieces - 1));
  for (int64_t p = 1; p < pieces; ++p) {
    const int64_t b = p * per, e = std::min(items, b + per);
    if (b < e) pool.emplace_back([&body, b, e] { body(b, e); });
  }
  body(int64_t(0), std::min(items, per));
  for (auto& t : pool) t.join();
}
}  // namespace

void set_threads(int threads) { g_threads.store(threads < 1 ? 1 : (threads > 256 ? 256 : threads)); }
int get_threads() { return g_threads.load(); }

// ------------------------------------------------------------------ TBQ
namespace {
// tbq_quant without branches: r - t, r - (-t) = r + t and r - 0 = r are the
// same IEEE operations as the branchy form, so fields and residuals are bit-identical.
inline uint32_t tbq_quant_select(float& r, float g, float t) {
  const float s = hp_add(r, g);
  const uint32_t hi = s >= t, lo = s <= -t;
  uint32_t tb;
  std::memcpy(&tb, &t, 4);
  // +t, -t or +0.0 assembled from masks: with data this random a conditional jump mispredicts
  // about once per element, which was three quarters of the encode time
  const uint32_t ab = (tb & (0u - hi)) | ((tb ^ 0x80000000u) & (0u - lo));
  float adj;
  std::memcpy(&adj, &ab, 4);
  r = hp_sub(s, adj);
  return 1u + hi - lo;
}
}  // namespace

void tbq_compress(const float* grad, float* residual, int64_t n, float threshold, uint8_t* out) {
  const int64_t full = n >> 2;
  parallel_items(full, 4, [=](int64_t b0, int64_t b1) {
    for (int64_t b = b0; b < b1; ++b) {  // whole bytes: no bounds checks inside
      const int64_t base = b << 2;
      const uint32_t q = tbq_quant_select(residual[base], grad[base], threshold) |
                         (tbq_quant_select(residual[base + 1], grad[base + 1], threshold) << 2) |
                         (tbq_quant_select(residual[base + 2], grad[base + 2], threshold) << 4) |
                         (tbq_quant_select(residual[base + 3], grad[base + 3], threshold) << 6);
      out[b] = static_cast<uint8_t>(q);
    }
  });
  if (n & 3) {
    uint32_t q = 0;
    for (int k = 0; k < 4; ++k) {
      const int64_t j = (full << 2) + k;
      uint32_t field = 1u;  // padding slots of the last byte decode to zero
      if (j < n) field = tbq_quant(residual[j], grad[j], threshold);
      q |= field << (2 * k);
    }
    out[full] = static_cast<uint8_t>(q);
  }
}

void tbq_decompress(const uint8_t* in, int64_t n, float threshold, float* out, int add) {
  // byte value -> its four decoded elements (same arithmetic as decoding them one by one)
  float lut[256][4];
  for (int v = 0; v < 256; ++v)
    for (int k = 0; k < 4; ++k) lut[v][k] = tbq_dequant((static_cast<uint32_t>(v) >> (2 * k)) & 3u, threshold);
  const int64_t full = n >> 2;
  const float (*table)[4] = lut;
  parallel_items(full, 4, [=](int64_t b0, int64_t b1) {
    if (add) {
      for (int64_t b = b0; b < b1; ++b) {
        const float* e = table[in[b]];
        float* o = out + (b << 2);
        o[0] = hp_add(e[0], o[0]);
        o[1] = hp_add(e[1], o[1]);
        o[2] = hp_add(e[2], o[2]);
        o[3] = hp_add(e[3], o[3]);
      }
    } else {
      for (int64_t b = b0; b < b1; ++b) std::memcpy(out + (b << 2), table[in[b]], 16);
    }
  });
  for (int64_t i = full << 2; i < n; ++i) {
    const float v = lut[in[i >> 2]][i & 3];
    out[i] = add ? hp_add(v, out[i]) : v;
  }
}

// ------------------------------------------------------------------ TernGrad
namespace {

template <int BW>
void tern_compress_impl(const float* grad, const float* res_in, float* res_out, int64_t n, float mn,
                        float inv, float gap, bool random, uint64_t seed, uint8_t* data) {
  constexpr int DPB = 8 / BW;
  const int64_t full = n / DPB;
  const int rem = static_cast<int>(n % DPB);
  parallel_items(full + (rem ? 1 : 0), DPB, [=](int64_t b0, int64_t b1) {
    float x[DPB] = {};
    float ef[DPB] = {};
    for (int64_t b = b0; b < b1; ++b) {
      const int count = b < full ? DPB : rem;
      for (int j = 0; j < count; ++j) {
        const int64_t e = b * DPB + j;
        x[j] = res_in ? hp_add(grad[e], res_in[e]) : grad[e];
      }
      // the tail byte is never stochastic
      const bool rnd = random && b < full;
      data[b] = tern_pack_byte<BW>(x, count, mn, inv, rnd, tern_byte_seed(seed, b), gap,
                                   res_out ? ef : nullptr);
      if (res_out)
        for (int j = 0; j < count; ++j) res_out[b * DPB + j] = ef[j];
    }
  });
}

template <int BW>
void tern_decompress_impl(const uint8_t* data, int64_t count, float gap, float mn, float* out,
                          int add) {
  constexpr int DPB = 8 / BW;
  constexpr uint32_t MASK = (1u << BW) - 1u;
  // byte value -> its DPB decoded elements (same arithmetic as decoding them one by one)
  float lut[256][DPB];
  for (int v = 0; v < 256; ++v)
    for (int k = 0; k < DPB; ++k) lut[v][k] = tern_dequant((static_cast<uint32_t>(v) >> (k * BW)) & MASK, gap, mn);
  const int64_t full = count / DPB;
  const float (*table)[DPB] = lut;
  parallel_items(full, DPB, [=](int64_t b0, int64_t b1) {
    if (add) {
      for (int64_t b = b0; b < b1; ++b) {
        const float* e = table[data[b]];
        float* o = out + b * DPB;
        for (int k = 0; k < DPB; ++k) o[k] = hp_add(e[k], o[k]);
      }
    } else {
      for (int64_t b = b0; b < b1; ++b) std::memcpy(out + b * DPB, table[data[b]], sizeof(float) * DPB);
    }
  });
  for (int64_t i = full * DPB; i < count; ++i) {
    const float v = lut[data[i / DPB]][i % DPB];
    out[i] = add ? hp_add(v, out[i]) : v;
  }
}

}  // namespace

int terngrad_compress(const float* grad, int64_t n, int bitwidth, int enable_random, uint64_t seed,
                      uint8_t* out, int64_t out_size, float* residual) {
  if (!tern_bitwidth_ok(bitwidth)) return -1;
  if (n <= 0 || out_size != tern_payload_bytes(n, bitwidth)) return -1;
  // first minimum / last maximum, like thrust::minmax_element; the distinction
  // is only visible for +-0.0 extremes
  float mn = 0.f, mx = 0.f;
  auto scan = [&](int64_t b, int64_t e, float& lo, float& hi, bool& nan) {
    lo = residual ? hp_add(grad[b], residual[b]) : grad[b];
    hi = lo;
    nan = lo != lo;
    for (int64_t i = b + 1; i < e; ++i) {
      const float v = residual ? hp_add(grad[i], residual[i]) : grad[i];
      nan = nan || v != v;
      if (v < lo) lo = v;
      if (!(v < hi)) hi = v;
    }
  };
  bool done = false;
  const int pieces = int(std::min<int64_t>(get_threads(), n / kGrainElems));
  if (pieces > 1) {
    // per-piece extremes merged in element order with the same comparisons: the first minimum
    // and the last maximum, exactly as the one-thread scan finds them -- for NaN-free input.
    // A NaN makes the running extremes depend on everything before it, so any piece that
    // saw one sends the whole tensor through the one-thread scan below.
    std::vector<float> lo(size_t(pieces), 0.f), hi(size_t(pieces), 0.f);
    std::vector<char> nan(size_t(pieces), 0);
    const int64_t per = (n + pieces - 1) / pieces;
    std::vector<std::thread> pool;
    auto piece = [&](int p) {
      const int64_t b = int64_t(p) * per, e = std::min(n, b + per);
      bool saw = false;
      if (b < e) scan(b, e, lo[size_t(p)], hi[size_t(p)], saw);
      else saw = true;   // empty piece: take the safe path
      nan[size_t(p)] = saw ? 1 : 0;
    };
    for (int p = 1; p < pieces; ++p) pool.emplace_back(piece, p);
    piece(0);
    for (auto& t : pool) t.join();
    bool any_nan = false;
    for (int p = 0; p < pieces; ++p) any_nan = any_nan || nan[size_t(p)] != 0;
    if (!any_nan) {
      mn = lo[0];
      mx = hi[0];
      for (int p = 1; p < pieces; ++p) {
        if (lo[size_t(p)] < mn) mn = lo[size_t(p)];
        if (!(hi[size_t(p)] < mx)) mx = hi[size_t(p)];
      }
      done = true;
    }
  }
  if (!done) {
    bool nan = false;
    scan(0, n, mn, mx, nan);
  }
  const float gap = tern_gap(mn, mx, bitwidth);
  const float inv = tern_gap_inverse(gap);
  out[0] = static_cast<uint8_t>(bitwidth);
  out[1] = static_cast<uint8_t>(tern_tail(n, bitwidth));
  std::memcpy(out + 2, &mn, 4);
  std::memcpy(out + 6, &mx, 4);
  uint8_t* data = out + kTernHeaderBytes;
  const bool rnd = enable_random != 0;
  switch (bitwidth) {
    case 1: tern_compress_impl<1>(grad, residual, residual, n, mn, inv, gap, rnd, seed, data); break;
    case 2: tern_compress_impl<2>(grad, residual, residual, n, mn, inv, gap, rnd, seed, data); break;
    case 4: tern_compress_impl<4>(grad, residual, residual, n, mn, inv, gap, rnd, seed, data); break;
    default: tern_compress_impl<8>(grad, residual, residual, n, mn, inv, gap, rnd, seed, data); break;
  }
  return 0;
}

int64_t terngrad_decompress(const uint8_t* in, int64_t in_size, float* out, int64_t out_capacity,
                            int add) {
  if (in_size < kTernHeaderBytes) return -1;
  const int bw = in[0];
  const int tail = in[1];
  if (!tern_bitwidth_ok(bw)) return -1;
  float mn, mx;
  std::memcpy(&mn, in + 2, 4);
  std::memcpy(&mx, in + 6, 4);
  const int64_t count = (in_size - kTernHeaderBytes) * tern_dpb(bw) - tail;
  if (count < 0 || count > out_capacity) return -1;
  const float gap = tern_gap(mn, mx, bw);
  const uint8_t* data = in + kTernHeaderBytes;
  switch (bw) {
    case 1: tern_decompress_impl<1>(data, count, gap, mn, out, add); break;
    case 2: tern_decompress_impl<2>(data, count, gap, mn, out, add); break;
    case 4: tern_decompress_impl<4>(data, count, gap, mn, out, add); break;
    default: tern_decompress_impl<8>(data, count, gap, mn, out, add); break;
  }
  return count;
}

// ------------------------------------------------------------------ sparse
int64_t sparse_compress(const float* grad, float* R, int64_t n, double sample_rate,
                        double keep_fraction, uint64_t seed, int accumulate, uint8_t* out,
                        int64_t out_capacity) {
  if (n <= 0) return -1;
  const int64_t expected = std::min<int64_t>(n, sparse_expected_k(n, keep_fraction));
  if (out_capacity < sparse_payload_bytes(expected)) return -1;
  if (accumulate)
    for (int64_t i = 0; i < n; ++i) R[i] = hp_add(grad[i], R[i]);

  // threshold from the random sample
  const int64_t sample_cnt = sparse_sample_count(n, sample_rate);
  float thr = 0.0f;
  if (sample_cnt > 0) {
    std::vector<uint32_t> keys(static_cast<size_t>(sample_cnt));
    for (int64_t x = 0; x < sample_cnt; ++x)
      keys[x] = abs_key(R[sparse_sample_index(seed, x, static_cast<uint32_t>(n))]);
    int64_t rank = sparse_threshold_rank(sample_cnt, keep_fraction);
    rank = std::min(rank, sample_cnt - 1);
    std::nth_element(keys.begin(), keys.begin() + rank, keys.end(), std::greater<uint32_t>());
    std::memcpy(&thr, &keys[rank], 4);
  }
  const uint32_t thr_key = abs_key(thr);

  // candidates over the threshold
  int64_t cand = 0;
  for (int64_t i = 0; i < n; ++i) cand += abs_key(R[i]) > thr_key;
  uint32_t cut_key = thr_key;
  int64_t ties_kept = 0;
  if (cand > expected) {
    std::vector<uint32_t> ck;
    ck.reserve(static_cast<size_t>(cand));
    for (int64_t i = 0; i < n; ++i)
      if (abs_key(R[i]) > thr_key) ck.push_back(abs_key(R[i]));
    std::nth_element(ck.begin(), ck.begin() + (expected - 1), ck.end(), std::greater<uint32_t>());
    cut_key = ck[expected - 1];
    int64_t above = 0;
    for (uint32_t k : ck) above += k > cut_key;
    ties_kept = expected - above;
  }

  const int64_t kmax = std::min(cand, expected);
  int32_t* idx_out = reinterpret_cast<int32_t*>(out + 4);
  std::vector<float> vals;
  vals.reserve(static_cast<size_t>(kmax));
  int64_t k = 0, ties_seen = 0;
  for (int64_t i = 0; i < n; ++i) {
    const uint32_t key = abs_key(R[i]);
    bool keep = key > cut_key;
    if (!keep && ties_kept > 0 && key == cut_key && ties_seen < ties_kept) {
      keep = true;
      ++ties_seen;
    }
    if (keep) {
      const int32_t i32 = static_cast<int32_t>(i);
      std::memcpy(idx_out + k, &i32, 4);
      vals.push_back(R[i]);
      R[i] = 0.0f;
      ++k;
    }
  }
  const int32_t total = static_cast<int32_t>(sparse_payload_bytes(k));
  std::memcpy(out, &total, 4);
  if (k) std::memcpy(out + 4 + 4 * k, vals.data(), static_cast<size_t>(4 * k));
  return total;
}

int64_t sparse_decompress(const uint8_t* in, int64_t in_size, float* out, int64_t n, int add) {
  if (in_size < 4) return -1;
  int32_t total;
  std::memcpy(&total, in, 4);
  if (total < 4 || total > in_size) return -1;
  const int64_t k = (total - 4) / 8;
  const uint8_t* idx = in + 4;
  const uint8_t* val = in + 4 + 4 * k;
  for (int64_t x = 0; x < k; ++x) {
    int32_t i;
    std::memcpy(&i, idx + 4 * x, 4);
    if (i < 0 || i >= n) return -1;
  }
  if (!add) std::fill(out, out + n, 0.0f);
  for (int64_t x = 0; x < k; ++x) {
    int32_t i;
    float v;
    std::memcpy(&i, idx + 4 * x, 4);
    std::memcpy(&v, val + 4 * x, 4);
    out[i] = add ? hp_add(out[i], v) : v;
  }
  return k;
}

// ------------------------------------------------------------------ ECQ
int ecq_compress(const float* grad, float* history, int64_t n, float alpha, float beta,
                 int bitwidth, uint64_t seed, uint8_t* out, int64_t out_size) {
  if (!ecq_bitwidth_ok(bitwidth) || n <= 0) return -1;
  if (out_size != ecq_payload_bytes(n, bitwidth)) return -1;
  const int dpb = 8 / bitwidth;
  const int64_t M = (n + dpb - 1) / dpb;
  float mx = 0.0f;
  for (int64_t i = 0; i < n; ++i)
    mx = std::max(mx, std::fabs(ecq_compensated(grad[i], history[i], alpha)));
  uint8_t* Q = out + kEcqHeaderBytes;
  const bool zero = mx < kEcqZeroCutoff;
  // an all-(near-)zero tensor is sent as max = 0 so that it decodes to exact zeros
  const float hmx = zero ? 0.0f : mx;
  const float gap = zero ? 0.0f : ecq_gap(mx, bitwidth);
  const float inv = zero ? 0.0f : ecq_gap_inverse(gap);
  for (int64_t b = 0; b < M; ++b) {
    uint8_t q = 0;
    Lcg32 rng(tern_byte_seed(seed, b));
    for (int j = 0; j < dpb; ++j) {
      const int64_t e = b * dpb + j;
      if (e >= n) break;
      const float v = ecq_compensated(grad[e], history[e], alpha);
      uint8_t t = 0;
      if (!zero) t = ecq_quant(v, mx, inv, rng.next_unit());
      q = static_cast<uint8_t>(q | (static_cast<int>(t) << (bitwidth * j)));
      const uint32_t kept = static_cast<uint32_t>(t) & ((1u << bitwidth) - 1u);
      history[e] = ecq_history(history[e], beta, v, ecq_dequant(kept, gap, hmx));
    }
    Q[b] = q;
  }
  const int32_t total = static_cast<int32_t>(kEcqHeaderBytes + M);
  std::memcpy(out, &total, 4);
  std::memcpy(out + 4, &hmx, 4);
  out[8] = static_cast<uint8_t>(bitwidth);
  out[9] = static_cast<uint8_t>(M * dpb - n);
  return 0;
}

int64_t ecq_decompress(const uint8_t* in, int64_t in_size, float* out, int64_t out_capacity,
                       int add) {
  if (in_size < kEcqHeaderBytes) return -1;
  int32_t total;
  float mx;
  std::memcpy(&total, in, 4);
  std::memcpy(&mx, in + 4, 4);
  const int bw = in[8];
  const int unused = in[9];
  if (!ecq_bitwidth_ok(bw) || total > in_size || total < kEcqHeaderBytes) return -1;
  const int dpb = 8 / bw;
  const int64_t n = static_cast<int64_t>(total - kEcqHeaderBytes) * dpb - unused;
  if (n < 0 || n > out_capacity) return -1;
  const float gap = mx > 0.0f ? ecq_gap(mx, bw) : 0.0f;
  const uint8_t* Q = in + kEcqHeaderBytes;
  const uint32_t mask = (1u << bw) - 1u;
  for (int64_t i = 0; i < n; ++i) {
    const uint32_t q = (Q[i / dpb] >> ((i % dpb) * bw)) & mask;
    const float v = ecq_dequant(q, gap, mx);
    out[i] = add ? hp_add(out[i], v) : v;
  }
  return n;
}

// ------------------------------------------------------------------ PowerSGD
void powersgd_encode1(const float* grad, const float* residual, int64_t N, float* M, int64_t n,
                      int64_t m, const float* Q, int64_t r, float* P) {
  for (int64_t i = 0; i < N; ++i) M[i] = grad[i] + residual[i];
  for (int64_t i = 0; i < n; ++i)
    for (int64_t c = 0; c < r; ++c) {
      double acc = 0.0;
      for (int64_t k = 0; k < m; ++k) acc += static_cast<double>(M[i * m + k]) * Q[k * r + c];
      P[i * r + c] = static_cast<float>(acc);
    }
}

void gram_schmidt(float* P, int64_t n, int64_t r, float eps) {
  for (int64_t j = 0; j < r; ++j) {
    double ss = 0.0;
    for (int64_t i = 0; i < n; ++i) ss += static_cast<double>(P[i * r + j]) * P[i * r + j];
    const double inv = 1.0 / (std::sqrt(ss) + eps);
    for (int64_t i = 0; i < n; ++i) P[i * r + j] = static_cast<float>(P[i * r + j] * inv);
    for (int64_t c = j + 1; c < r; ++c) {
      double dot = 0.0;
      for (int64_t i = 0; i < n; ++i) dot += static_cast<double>(P[i * r + j]) * P[i * r + c];
      for (int64_t i = 0; i < n; ++i)
        P[i * r + c] = static_cast<float>(P[i * r + c] - dot * P[i * r + j]);
    }
  }
}

void powersgd_encode2(float* P, const float* M, int64_t n, int64_t m, int64_t r, float* Q) {
  gram_schmidt(P, n, r, 1e-8f);
  std::vector<double> acc(static_cast<size_t>(m * r), 0.0);
  for (int64_t i = 0; i < n; ++i)
    for (int64_t k = 0; k < m; ++k) {
      const double mv = M[i * m + k];
      for (int64_t c = 0; c < r; ++c) acc[k * r + c] += mv * P[i * r + c];
    }
  for (int64_t x = 0; x < m * r; ++x) Q[x] = static_cast<float>(acc[x]);
}

void powersgd_decode(const float* P, const float* Q, int64_t n, int64_t m, int64_t r, float* M,
                     float* residual, float* grad, int64_t N) {
  for (int64_t i = 0; i < n; ++i)
    for (int64_t k = 0; k < m; ++k) {
      double acc = 0.0;
      for (int64_t c = 0; c < r; ++c) acc += static_cast<double>(P[i * r + c]) * Q[k * r + c];
      M[i * m + k] = static_cast<float>(acc);
    }
  for (int64_t i = 0; i < N; ++i) {
    residual[i] = grad[i] - M[i];
    grad[i] = M[i];
  }
}

}  // namespace cpu
}  // namespace hipress
