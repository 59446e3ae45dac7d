// Sampled-threshold top-k sparsifier (GradDrop / DGC payloads) for sm_100a,
// with no host round-trip.
//
// The reference pipeline is transform(+) -> for_each(sample) -> sort -> D2H+sync
// -> copy_if (implicit sync) -> sort + truncate -> H2D+sync -> for_each(gather)
// (gd_body.h:121-229): four host synchronisations and two sorts.  Here:
//
//   sample x3   The k-th largest |value| of the random sample is found by a
//               3-digit radix select (11+11+10 bits of the order-preserving key).
//               Samples are *recomputed* from the LCG in every round instead of
//               being stored and sorted, so no sample buffer exists.
//   count       One pass: R += G (GradDrop), per-CTA count of |R| > threshold and
//               first-digit histogram of those candidates.
//   trim x2     Only when more than ceil(N*keep) candidates qualified (decided on
//               the device; otherwise the kernels return at once): radix select of
//               the exact cut among the candidates.
//   recount     Per-CTA counts against the cut (only when trimming).
//   scan        One CTA: exclusive offsets per CTA, k, the 4-byte header to every
//               destination, and clearing of the histograms for the next call.
//   write       Ordered compaction: indices ascending, values, residual zeroing,
//               stored into every destination (local and NVLink peers), then the
//               completion flag.
//
// Content rule (identical to the CPU codec): keep |R[i]| > threshold in
// ascending index order; when over-selected keep the largest magnitudes, ties
// toward the lower index.
#include "../common/codec_math.h"
#include "kernels.h"
#include "p2p.cuh"

namespace hipress {
namespace cuda {

namespace {

constexpr int kThreads = 256;
constexpr int kBins = 2048;
constexpr int kMaxBlocks = 148 * 4;
constexpr int kTile = kThreads * 4;  // elements per CTA iteration

struct SparseScratch {
  unsigned int shist[3][kBins];  // sample radix-select rounds
  unsigned int thist[3][kBins];  // trim radix-select rounds
  unsigned int cnt_gt[kMaxBlocks], cnt_eq[kMaxBlocks];
  unsigned int off_gt[kMaxBlocks], off_eq[kMaxBlocks];
  // state words
  // Radix-select progress, one slot per round: a kernel reads the slot of the
  // previous round and writes its own, so no word is read and written by
  // different CTAs of the same launch.
  unsigned int s_prefix[3], s_rank[3];  // sample select
  unsigned int t_prefix[3], t_rank[3];  // trim select
  unsigned int thr_key;                 // threshold (key of a positive float)
  unsigned int cand;                    // candidates over the threshold
  unsigned int cut_key, ties_kept;      // final rule
  unsigned int k;                       // elements emitted
  unsigned int pad[3];
};

__device__ __forceinline__ int digit_of(uint32_t key, int round) {
  return round == 0 ? int(key >> 21) : round == 1 ? int((key >> 10) & 0x7ffu) : int(key & 0x3ffu);
}
__device__ __forceinline__ bool prefix_matches(uint32_t key, int round, uint32_t prefix) {
  return round == 0 ? true : round == 1 ? (key >> 21) == prefix : (key >> 10) == prefix;
}
__device__ __forceinline__ uint32_t extend_prefix(uint32_t prefix, int round, uint32_t digit) {
  return round == 0 ? digit : round == 1 ? (prefix << 11) | digit : (prefix << 10) | digit;
}

// Block-wide: find the bin holding the element of 0-indexed `rank` counted from
// the top bin down.  Every thread returns the same (bin, rank inside bin).
__device__ void pick_from_top(const unsigned int* hist, unsigned int rank, unsigned int& bin,
                              unsigned int& rank_in_bin) {
  __shared__ unsigned int part[kThreads];
  __shared__ unsigned int res[2];
  constexpr int PER = kBins / kThreads;  // 8 bins per thread
  const int t = threadIdx.x;
  unsigned int local[PER];
  unsigned int sum = 0;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    local[j] = hist[kBins - 1 - (t * PER + j)];
    sum += local[j];
  }
  part[t] = sum;
  if (t == 0) {
    res[0] = 0;
    res[1] = 0;
  }
  __syncthreads();
  // serial prefix by warp 0 is enough for 256 entries
  if (t == 0) {
    unsigned int run = 0;
    for (int i = 0; i < kThreads; ++i) {
      const unsigned int v = part[i];
      part[i] = run;
      run += v;
    }
  }
  __syncthreads();
  const unsigned int before = part[t];
  if (rank >= before && rank < before + sum) {
    unsigned int run = before;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      if (rank >= run && rank < run + local[j]) {
        res[0] = kBins - 1 - (t * PER + j);
        res[1] = rank - run;
      }
      run += local[j];
    }
  }
  __syncthreads();
  bin = res[0];
  rank_in_bin = res[1];
  __syncthreads();
}

__device__ __forceinline__ void hist_flush(unsigned int* sh, unsigned int* gh) {
  __syncthreads();
  for (int i = threadIdx.x; i < kBins; i += kThreads) {
    const unsigned int v = sh[i];
    if (v) atomicAdd(gh + i, v);
  }
}

// Visit every element of [begin, end) once with f(value): 16-byte loads, four in flight per
// thread, scalar handling of an unaligned base or a ragged end.  `begin` is a multiple of the
// tile size, so the vector path applies whenever R itself is 16-byte aligned.
template <typename F>
__device__ __forceinline__ void for_each_value(const float* __restrict__ R, int64_t begin, int64_t end, F f) {
  if ((reinterpret_cast<uintptr_t>(R + begin) & 15) == 0) {
    const int64_t nvec = (end - begin) >> 2;
    const float4* v = reinterpret_cast<const float4*>(R + begin);
    int64_t i = threadIdx.x;
    for (; i + 3 * kThreads < nvec; i += 4 * kThreads) {
      const float4 a = v[i], b = v[i + kThreads], c = v[i + 2 * kThreads], d = v[i + 3 * kThreads];
      f(a.x); f(a.y); f(a.z); f(a.w);
      f(b.x); f(b.y); f(b.z); f(b.w);
      f(c.x); f(c.y); f(c.z); f(c.w);
      f(d.x); f(d.y); f(d.z); f(d.w);
    }
    for (; i < nvec; i += kThreads) {
      const float4 a = v[i];
      f(a.x); f(a.y); f(a.z); f(a.w);
    }
    for (int64_t j = begin + (nvec << 2) + threadIdx.x; j < end; j += kThreads) f(R[j]);
  } else {
    for (int64_t j = begin + threadIdx.x; j < end; j += kThreads) f(R[j]);
  }
}

// ---- sample rounds
template <int ROUND>
__global__ void __launch_bounds__(kThreads)
sample_round_kernel(const float* __restrict__ grad, const float* __restrict__ R, int64_t n,
                    int64_t sample_cnt, unsigned int rank0, uint64_t seed, int accumulate,
                    SparseScratch* s, const uint32_t* epoch_dev) {
  if (epoch_dev != nullptr) seed += uint64_t(*epoch_dev) * kEpochSeedStride;  // see PushTargets
  __shared__ unsigned int sh[kBins];
  for (int i = threadIdx.x; i < kBins; i += kThreads) sh[i] = 0;
  uint32_t prefix = 0;
  if (ROUND > 0) {
    const unsigned int rank = ROUND == 1 ? rank0 : s->s_rank[ROUND - 1];
    unsigned int bin, rin;
    pick_from_top(s->shist[ROUND - 1], rank, bin, rin);
    prefix = extend_prefix(ROUND == 1 ? 0u : s->s_prefix[ROUND - 1], ROUND - 1, bin);
    if (blockIdx.x == 0 && threadIdx.x == 0) {
      // consumed by the next kernel in the stream
      s->s_prefix[ROUND] = prefix;
      s->s_rank[ROUND] = rin;
    }
  }
  __syncthreads();
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t x = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; x < sample_cnt; x += stride) {
    const uint32_t idx = sparse_sample_index(seed, x, uint32_t(n));
    const float v = accumulate ? hp_add(grad[idx], R[idx]) : R[idx];
    const uint32_t key = abs_key(v);
    if (prefix_matches(key, ROUND, prefix)) atomicAdd(&sh[digit_of(key, ROUND)], 1u);
  }
  hist_flush(sh, s->shist[ROUND]);
}

// ---- count pass (also performs R += G)
__global__ void __launch_bounds__(kThreads)
count_kernel(const float* __restrict__ grad, float* __restrict__ R, int64_t n, int64_t chunk,
             int64_t sample_cnt, unsigned int rank0, int accumulate, SparseScratch* s) {
  __shared__ unsigned int sh[kBins];
  __shared__ unsigned int blk_cnt;
  for (int i = threadIdx.x; i < kBins; i += kThreads) sh[i] = 0;
  if (threadIdx.x == 0) blk_cnt = 0;
  uint32_t thr_key = 0;
  if (sample_cnt > 0) {
    unsigned int bin, rin;
    pick_from_top(s->shist[2], s->s_rank[2], bin, rin);
    thr_key = extend_prefix(s->s_prefix[2], 2, bin);
  }
  __syncthreads();
  if (blockIdx.x == 0 && threadIdx.x == 0) s->thr_key = thr_key;
  const int64_t begin = int64_t(blockIdx.x) * chunk;
  const int64_t end = begin + chunk < n ? begin + chunk : n;
  unsigned int mine = 0;
  if (!accumulate) {
    // read-only pass (DGC: the velocity was accumulated by its own kernel): 16-byte loads
    for_each_value(R, begin, end, [&](float r) {
      const uint32_t key = abs_key(r);
      if (key > thr_key) {
        ++mine;
        atomicAdd(&sh[digit_of(key, 0)], 1u);
      }
    });
  } else {
    for (int64_t i = begin + threadIdx.x; i < end; i += kThreads) {
      const float r = hp_add(grad[i], R[i]);
      R[i] = r;
      const uint32_t key = abs_key(r);
      if (key > thr_key) {
        ++mine;
        atomicAdd(&sh[digit_of(key, 0)], 1u);
      }
    }
  }
  atomicAdd(&blk_cnt, mine);
  hist_flush(sh, s->thist[0]);
  __syncthreads();
  if (threadIdx.x == 0) {
    s->cnt_gt[blockIdx.x] = blk_cnt;
    s->cnt_eq[blockIdx.x] = 0;
    atomicAdd(&s->cand, blk_cnt);
  }
}

// ---- trim rounds 1 and 2 (return at once when not over-selected)
template <int ROUND>
__global__ void __launch_bounds__(kThreads)
trim_round_kernel(const float* __restrict__ R, int64_t n, int64_t chunk, unsigned int expected,
                  SparseScratch* s) {
  if (s->cand <= expected) return;
  __shared__ unsigned int sh[kBins];
  for (int i = threadIdx.x; i < kBins; i += kThreads) sh[i] = 0;
  const unsigned int rank = ROUND == 1 ? expected - 1 : s->t_rank[ROUND - 1];
  unsigned int bin, rin;
  pick_from_top(s->thist[ROUND - 1], rank, bin, rin);
  const uint32_t prefix = extend_prefix(ROUND == 1 ? 0u : s->t_prefix[ROUND - 1], ROUND - 1, bin);
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    s->t_prefix[ROUND] = prefix;
    s->t_rank[ROUND] = rin;
  }
  const uint32_t thr_key = s->thr_key;
  __syncthreads();
  const int64_t begin = int64_t(blockIdx.x) * chunk;
  const int64_t end = begin + chunk < n ? begin + chunk : n;
  for_each_value(R, begin, end, [&](float x) {
    const uint32_t key = abs_key(x);
    if (key > thr_key && prefix_matches(key, ROUND, prefix))
      atomicAdd(&sh[digit_of(key, ROUND)], 1u);
  });
  hist_flush(sh, s->thist[ROUND]);
}

// ---- final rule + per-CTA counts against the cut
__global__ void __launch_bounds__(kThreads)
recount_kernel(const float* __restrict__ R, int64_t n, int64_t chunk, unsigned int expected,
               SparseScratch* s) {
  if (s->cand <= expected) {
    if (blockIdx.x == 0 && threadIdx.x == 0) {
      s->cut_key = s->thr_key;
      s->ties_kept = 0;
    }
    return;  // counts of the count pass stand
  }
  unsigned int bin, rin;
  pick_from_top(s->thist[2], s->t_rank[2], bin, rin);
  const uint32_t cut = extend_prefix(s->t_prefix[2], 2, bin);
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    s->cut_key = cut;
    s->ties_kept = rin + 1;
  }
  __shared__ unsigned int c_gt, c_eq;
  if (threadIdx.x == 0) {
    c_gt = 0;
    c_eq = 0;
  }
  __syncthreads();
  const int64_t begin = int64_t(blockIdx.x) * chunk;
  const int64_t end = begin + chunk < n ? begin + chunk : n;
  unsigned int g = 0, e = 0;
  for_each_value(R, begin, end, [&](float x) {
    const uint32_t key = abs_key(x);
    g += key > cut;
    e += key == cut;
  });
  atomicAdd(&c_gt, g);
  atomicAdd(&c_eq, e);
  __syncthreads();
  if (threadIdx.x == 0) {
    s->cnt_gt[blockIdx.x] = c_gt;
    s->cnt_eq[blockIdx.x] = c_eq;
  }
}

// ---- one CTA: offsets, k, header, housekeeping
__global__ void __launch_bounds__(1024)
scan_kernel(int blocks, PushTargets dst, SparseScratch* s) {
  resolve_epoch(dst);
  __shared__ unsigned int wa[32], wb[32], tot[2];
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const unsigned int va = t < blocks ? s->cnt_gt[t] : 0u;
  const unsigned int vb = t < blocks ? s->cnt_eq[t] : 0u;
  unsigned int ia = va, ib = vb;  // inclusive scans inside the warp
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned int x = __shfl_up_sync(0xffffffffu, ia, o);
    const unsigned int y = __shfl_up_sync(0xffffffffu, ib, o);
    if (lane >= o) {
      ia += x;
      ib += y;
    }
  }
  if (lane == 31) {
    wa[warp] = ia;
    wb[warp] = ib;
  }
  __syncthreads();
  if (warp == 0) {  // exclusive scan of the 32 warp totals
    const unsigned int xa = wa[lane], xb = wb[lane];
    unsigned int sa = xa, sb = xb;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned int x = __shfl_up_sync(0xffffffffu, sa, o);
      const unsigned int y = __shfl_up_sync(0xffffffffu, sb, o);
      if (lane >= o) {
        sa += x;
        sb += y;
      }
    }
    wa[lane] = sa - xa;
    wb[lane] = sb - xb;
    if (lane == 31) {
      tot[0] = sa;
      tot[1] = sb;
    }
  }
  __syncthreads();
  if (t < blocks) {
    s->off_gt[t] = wa[warp] + ia - va;
    s->off_eq[t] = wb[warp] + ib - vb;
  }
  if (t == 0) {
    const unsigned int ties = s->ties_kept;
    const unsigned int k = tot[0] + (tot[1] < ties ? tot[1] : ties);
    s->k = k;
    const uint32_t total = 4u + 8u * k;
    uint8_t header[4];
    for (int i = 0; i < 4; ++i) header[i] = uint8_t(total >> (8 * i));
    push_bytes(dst, 0, header, 4);
    s->cand = 0;
  }
  unsigned int* h = &s->shist[0][0];
  for (int i = t; i < 6 * kBins; i += 1024) h[i] = 0;
}

// ---- ordered compaction and delivery
// Output order is index order; position of an element = (elements above the cut before it) +
// min(ties kept, elements equal to the cut before it).  The CTA's starting counts come from the
// scan; inside the CTA each warp owns a contiguous part of the chunk: a first walk counts what
// the warp will emit, one barrier turns the counts into per-warp offsets, and a second walk
// (its data now in L1 / L2) emits with warp-level scans only.  99.9 % of the data is below the
// cut, so most 128-element steps are a ballot and nothing else.  (A first version scanned
// across the whole CTA per 1,024-element tile -- five barriers per tile that held a hit -- and
// took 64 us for 64 MB where the reads cost 12.)
__global__ void __launch_bounds__(kThreads)
write_kernel(float* __restrict__ R, int64_t n, int64_t chunk, PushTargets dst,
             const SparseScratch* s) {
  resolve_epoch(dst);
  constexpr int kWarps = kThreads / 32;
  __shared__ unsigned int warp_gt[kWarps], warp_eq[kWarps];
  const uint32_t cut = s->cut_key;
  const unsigned int ties = s->ties_kept;
  const unsigned int k_total = s->k;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t begin = int64_t(blockIdx.x) * chunk;
  const int64_t end = begin + chunk < n ? begin + chunk : n;
  // warp ranges: multiples of 128 elements so that every step is 32 lanes x 4 elements
  int64_t wlen = (end - begin + kWarps - 1) / kWarps;
  wlen = (wlen + 127) / 128 * 128;
  const int64_t wbegin = begin + warp * wlen < end ? begin + warp * wlen : end;
  const int64_t wend = wbegin + wlen < end ? wbegin + wlen : end;
  const bool vec_ok = (reinterpret_cast<uintptr_t>(R) & 15) == 0 && (begin & 3) == 0;

  auto load4 = [&](int64_t e0, float (&v)[4], uint32_t (&key)[4]) {
    if (vec_ok && e0 + 3 < wend) {
      const float4 q = *reinterpret_cast<const float4*>(R + e0);
      v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
#pragma unroll
      for (int j = 0; j < 4; ++j) key[j] = abs_key(v[j]);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[j] = (e0 + j < wend) ? R[e0 + j] : 0.0f;
        key[j] = (e0 + j < wend) ? abs_key(v[j]) : 0u;   // key 0 is below any cut that selects
      }
    }
  };

  // ---- first walk: how many elements above / at the cut does this warp hold
  unsigned int my_gt = 0, my_eq = 0;
  int64_t base = wbegin;
  if (vec_ok) {
    // four steps per iteration with their loads issued together: one load in flight per lane
    // left this walk waiting on DRAM latency
    for (; base + 512 <= wend; base += 512) {
      float4 q[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) q[u] = *reinterpret_cast<const float4*>(R + base + u * 128 + lane * 4);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const uint32_t k0 = abs_key(q[u].x), k1 = abs_key(q[u].y), k2 = abs_key(q[u].z), k3 = abs_key(q[u].w);
        my_gt += (k0 > cut) + (k1 > cut) + (k2 > cut) + (k3 > cut);
        my_eq += (k0 == cut) + (k1 == cut) + (k2 == cut) + (k3 == cut);
      }
    }
  }
  for (; base < wend; base += 128) {
    float v[4];
    uint32_t key[4];
    load4(base + lane * 4, v, key);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const bool in = base + lane * 4 + j < wend;
      my_gt += in && key[j] > cut;
      my_eq += in && key[j] == cut;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    my_gt += __shfl_xor_sync(0xffffffffu, my_gt, o);
    my_eq += __shfl_xor_sync(0xffffffffu, my_eq, o);
  }
  if (lane == 0) {
    warp_gt[warp] = my_gt;
    warp_eq[warp] = my_eq;
  }
  __syncthreads();
  unsigned int run_gt = s->off_gt[blockIdx.x], run_eq = s->off_eq[blockIdx.x];
  for (int w = 0; w < warp; ++w) {
    run_gt += warp_gt[w];
    run_eq += warp_eq[w];
  }

  // ---- second walk: emit
  if (my_gt != 0 || (ties > 0 && my_eq != 0)) {
    for (int64_t step = wbegin; step < wend; step += 128) {
      const int64_t e0 = step + lane * 4;
      float v[4];
      uint32_t key[4];
      load4(e0, v, key);
      unsigned int n_gt = 0, n_eq = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const bool in = e0 + j < wend;
        n_gt += in && key[j] > cut;
        n_eq += in && key[j] == cut;
      }
      if (__ballot_sync(0xffffffffu, (n_gt | n_eq) != 0) == 0) continue;
      unsigned int inc_gt = n_gt, inc_eq = n_eq;   // inclusive scans over the lanes
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const unsigned int a = __shfl_up_sync(0xffffffffu, inc_gt, o);
        const unsigned int b = __shfl_up_sync(0xffffffffu, inc_eq, o);
        if (lane >= o) {
          inc_gt += a;
          inc_eq += b;
        }
      }
      unsigned int gt_before = run_gt + inc_gt - n_gt, eq_before = run_eq + inc_eq - n_eq;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (e0 + j >= wend) break;
        const bool above = key[j] > cut, at = key[j] == cut;
        const bool keep = above || (at && eq_before < ties);
        if (keep) {
          const unsigned int pos = gt_before + (eq_before < ties ? eq_before : ties);
          if (pos < k_total) {
            push_u32(dst, 4 + 4 * int64_t(pos), uint32_t(e0 + j));
            push_u32(dst, 4 + 4 * int64_t(k_total) + 4 * int64_t(pos), __float_as_uint(v[j]));
            R[e0 + j] = 0.0f;
          }
        }
        gt_before += above;
        eq_before += at;
      }
      run_gt += __shfl_sync(0xffffffffu, inc_gt, 31);
      run_eq += __shfl_sync(0xffffffffu, inc_eq, 31);
    }
  }
  publish_when_grid_done(dst);
}

__global__ void __launch_bounds__(kThreads)
scatter_kernel(const uint8_t* __restrict__ payload, int64_t cap, float* __restrict__ out, int64_t n,
               float post_scale, int* status, const uint32_t* epoch_dev, int64_t parity_stride,
               const int* guard) {
  if (status_guarded(guard)) return;
  if (epoch_dev != nullptr && (*epoch_dev & 1u)) payload += parity_stride;  // see UnpackSources
  uint32_t total = 0;
  for (int k = 0; k < 4; ++k) total |= uint32_t(payload[k]) << (8 * k);
  if (total < 4 || int64_t(total) > cap) {
    if (blockIdx.x == 0 && threadIdx.x == 0 && status) atomicExch(status, int(kPayloadBounds));
    return;
  }
  const int64_t k = (int64_t(total) - 4) / 8;
  const uint32_t* idx = reinterpret_cast<const uint32_t*>(payload + 4);
  const uint32_t* val = reinterpret_cast<const uint32_t*>(payload + 4 + 4 * k);
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t x = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; x < k; x += stride) {
    const uint32_t i = idx[x];
    if (int64_t(i) >= n) {
      if (status) atomicExch(status, int(kPayloadBounds));
      continue;
    }
    float v = __uint_as_float(val[x]);
    if (post_scale != 1.0f) v = hp_mul(v, post_scale);
    // indices are unique inside one payload: a plain read-modify-write is race free
    out[i] = hp_add(out[i], v);
  }
}

struct Plan {
  int blocks;
  int64_t chunk;
};
inline Plan plan_for(int64_t n) {
  int64_t blocks = (n + kTile - 1) / kTile;
  if (blocks > kMaxBlocks) blocks = kMaxBlocks;
  if (blocks < 1) blocks = 1;
  int64_t chunk = (n + blocks - 1) / blocks;
  chunk = (chunk + kTile - 1) / kTile * kTile;
  blocks = (n + chunk - 1) / chunk;
  return {int(blocks), chunk};
}

}  // namespace

size_t sparse_scratch_bytes(int64_t) { return sizeof(SparseScratch); }

cudaError_t sparse_compress(const float* grad, float* R, int64_t n, double sample_rate,
                            double keep_fraction, uint64_t seed, int accumulate,
                            const PushTargets& dst, void* scratch, cudaStream_t stream) {
  if (n <= 0 || n > 0x7fffffff || scratch == nullptr) return cudaErrorInvalidValue;
  for (int p = 0; p < dst.world; ++p)
    if (reinterpret_cast<uintptr_t>(dst.payload[p]) & 3) return cudaErrorInvalidValue;
  auto* s = static_cast<SparseScratch*>(scratch);
  const Plan pl = plan_for(n);
  int64_t expected = sparse_expected_k(n, keep_fraction);
  if (expected > n) expected = n;
  const int64_t sample_cnt = sparse_sample_count(n, sample_rate);
  int64_t rank0 = sparse_threshold_rank(sample_cnt, keep_fraction);
  if (sample_cnt > 0 && rank0 > sample_cnt - 1) rank0 = sample_cnt - 1;
  if (sample_cnt > 0) {
    int64_t sb = (sample_cnt + kThreads - 1) / kThreads;
    if (sb > kMaxBlocks) sb = kMaxBlocks;
    sample_round_kernel<0><<<int(sb), kThreads, 0, stream>>>(grad, R, n, sample_cnt, unsigned(rank0), seed, accumulate, s, dst.epoch_dev);
    sample_round_kernel<1><<<int(sb), kThreads, 0, stream>>>(grad, R, n, sample_cnt, unsigned(rank0), seed, accumulate, s, dst.epoch_dev);
    sample_round_kernel<2><<<int(sb), kThreads, 0, stream>>>(grad, R, n, sample_cnt, unsigned(rank0), seed, accumulate, s, dst.epoch_dev);
  }
  count_kernel<<<pl.blocks, kThreads, 0, stream>>>(grad, R, n, pl.chunk, sample_cnt, unsigned(rank0), accumulate, s);
  trim_round_kernel<1><<<pl.blocks, kThreads, 0, stream>>>(R, n, pl.chunk, unsigned(expected), s);
  trim_round_kernel<2><<<pl.blocks, kThreads, 0, stream>>>(R, n, pl.chunk, unsigned(expected), s);
  recount_kernel<<<pl.blocks, kThreads, 0, stream>>>(R, n, pl.chunk, unsigned(expected), s);
  PushTargets hdr = dst;
  hdr.done = nullptr;
  scan_kernel<<<1, 1024, 0, stream>>>(pl.blocks, hdr, s);
  write_kernel<<<pl.blocks, kThreads, 0, stream>>>(R, n, pl.chunk, dst, s);
  return cudaGetLastError();
}

cudaError_t sparse_unpack_accum(const UnpackSources& src, float* out, int64_t n, int add,
                                float post_scale, int* status, cudaStream_t stream) {
  if (n <= 0 || src.world < 1 || src.world > kMaxWorld) return cudaErrorInvalidValue;
  if (!add) {
    cudaError_t e = cudaMemsetAsync(out, 0, size_t(n) * sizeof(float), stream);
    if (e != cudaSuccess) return e;
  }
  for (int r = 0; r < src.world; ++r) {
    if (reinterpret_cast<uintptr_t>(src.payload[r]) & 3) return cudaErrorInvalidValue;
    // worst-case k is bounded by the slot capacity
    const int64_t kmax = (src.payload_bytes[r] - 4) / 8;
    int64_t blocks = (kmax + kThreads - 1) / kThreads;
    if (blocks < 1) blocks = 1;
    if (blocks > 148 * 8) blocks = 148 * 8;
    scatter_kernel<<<int(blocks), kThreads, 0, stream>>>(src.payload[r], src.payload_bytes[r], out,
                                                        n, post_scale, status, src.epoch_dev,
                                                        src.parity_stride, src.guard);
  }
  return cudaGetLastError();
}

}  // namespace cuda
}  // namespace hipress
