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
//
// Two forms of everything after the sampling.  The passes above ("scan form") read the whole
// tensor up to five times.  For keep fractions up to 1 % the "list form" reads it ONCE:
//
//   count+collect  the one pass over the tensor.  It applies the codec's state update (R += G
//               for GradDrop; u = m*u + s*g, v += u and g = 0 for DGC with momentum correction;
//               nothing for plain DGC) and appends every candidate |value| > threshold, as
//               (index, value), to a per-warp list in index order.  A warp owns a contiguous
//               part of its CTA's chunk, so the lists, taken in order, are sorted by index.
//               Lists grow in blocks of 16 entries taken from a pool with one atomic.
//   cut         One CTA, only when more than ceil(N*keep) candidates qualified: their keys
//               (35 K for a 128 MB bucket at 0.1 %) are gathered into shared memory with batched
//               loads and the exact cut is found by a radix select there.
//   count+scan  One warp per list counts what it keeps against the cut; the last CTA to finish
//               turns the per-CTA totals into exclusive offsets, k and the header.
//   emit        One warp per list: indices and values to every destination, residual (and
//               DGC's momentum u) cleared at the emitted positions, then the completion flag.
//
// The sample keys are stored by the first sampling round and re-read by the other two (the
// scan form recomputes them, three random gathers per sample and round with momentum
// correction).  The pool is sized for many times the expected number of candidates (see
// list_plan); should it still run out, the candidates that did not fit stay in the residual
// and are sent in a later step (counted in SparseScratch::dropped).
#include "../common/codec_math.h"
#include "kernels.h"
#include "p2p.cuh"

#include <algorithm>
#include <cmath>

namespace hipress {
namespace cuda {

namespace {

constexpr int kThreads = 256;
constexpr int kBins = 2048;
constexpr int kMaxBlocks = 148 * 4;
constexpr int kTile = kThreads * 4;  // elements per CTA iteration
constexpr int kMaxLists = kMaxBlocks * (kThreads / 32);
constexpr int kBlockEntries = 16;
constexpr unsigned int kNoBlock = 0xffffffffu;
constexpr double kListMaxKeep = 0.01;   // the list form serves keep fractions up to this

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
  // list form
  unsigned int pool_used;               // blocks handed out (reset by select)
  unsigned int dropped;                 // candidates that found no block (cumulative)
  unsigned int last_cand;               // candidates seen by the last call (metrics)
  unsigned int lists_done;              // CTA arrival counter of the count+scan kernel (left at zero)
  unsigned int list_head[kMaxLists];    // first block of each warp's list, kNoBlock when empty
  unsigned int list_gt[kMaxLists], list_eq[kMaxLists];   // kept counts per list (above / at the cut)
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

// ---- the value the selection looks at, for one element, by mode
// mode 0: R as it is (plain DGC); mode 1: G + R (GradDrop's accumulation); mode 2: DGC with
// momentum correction, v + (m*u + s*g), rounded exactly as the collect pass rounds it.
struct SparseFuseDev {
  const float* grad;   // modes 1, 2
  float* u;            // mode 2: momentum
  float momentum;      // mode 2
  float clip;          // mode 2: > 0 = scale g by min(1, clip / |g|)
  const float* sumsq;  // mode 2 with clipping: |g|^2 of the bucket
  int zero_grad;       // mode 2: leave zeros in grad (the dense gradient is rebuilt from the payloads)
  int mode;
};
__device__ __forceinline__ float dgc_clip_scale(const SparseFuseDev& f) {
  if (f.mode != 2 || f.clip <= 0.f) return 1.0f;
  return fminf(1.0f, f.clip / (sqrtf(*f.sumsq) + 1e-6f));
}
__device__ __forceinline__ float dgc_new_u(float u, float g, float momentum, float scale) {
  return __fmaf_rn(momentum, u, __fmul_rn(scale, g));
}
__device__ __forceinline__ float fused_value(const SparseFuseDev& f, const float* R, uint32_t i, float scale) {
  if (f.mode == 0) return R[i];
  if (f.mode == 1) return hp_add(f.grad[i], R[i]);
  return __fadd_rn(R[i], dgc_new_u(f.u[i], f.grad[i], f.momentum, scale));
}

// ---- sample rounds
// keys: when non-null, round 0 stores every sample's key there and rounds 1 and 2 read them
// back instead of drawing and gathering again.
template <int ROUND>
__global__ void __launch_bounds__(kThreads)
sample_round_kernel(SparseFuseDev fuse, const float* __restrict__ R, int64_t n,
                    int64_t sample_cnt, unsigned int rank0, uint64_t seed,
                    SparseScratch* s, uint32_t* __restrict__ keys, const uint32_t* epoch_dev) {
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
  const float scale = dgc_clip_scale(fuse);
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  // whole warps iterate together; sampled magnitudes share their leading bits, so the lanes that
  // hit the same bin are counted by one of them (one shared-memory atomic per bin and warp)
  const int64_t padded = (sample_cnt + 31) & ~int64_t(31);
  for (int64_t x = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; x < padded; x += stride) {
    uint32_t key = 0;
    bool live = x < sample_cnt;
    if (live) {
      if (ROUND > 0 && keys != nullptr) {
        key = keys[x];
      } else {
        const uint32_t idx = sparse_sample_index(seed, x, uint32_t(n));
        key = abs_key(fused_value(fuse, R, idx, scale));
        if (keys != nullptr) keys[x] = key;
      }
      live = prefix_matches(key, ROUND, prefix);
    }
    const int bin = live ? digit_of(key, ROUND) : -1;
    const unsigned int same = __match_any_sync(0xffffffffu, bin);
    if (live && int(threadIdx.x & 31) == __ffs(same) - 1) atomicAdd(&sh[bin], unsigned(__popc(same)));
  }
  hist_flush(sh, s->shist[ROUND]);
}

// ---- count pass (also performs R += G)
__global__ void __launch_bounds__(kThreads)
count_kernel(const float* __restrict__ grad, float* __restrict__ R, int64_t n, int64_t chunk,
             int64_t sample_cnt, unsigned int rank0, int accumulate, int zero_grad, SparseScratch* s) {
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
      if (zero_grad) const_cast<float*>(grad)[i] = 0.f;
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
// thread t scans the totals of CTA t: the count / write kernels may not have more CTAs than this
// kernel has threads
static_assert(kMaxBlocks <= 1024, "scan_kernel scans one per-CTA total per thread");
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
    s->last_cand = s->cand;
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
write_kernel(float* __restrict__ R, float* __restrict__ u_mask, float* sumsq_to_clear, int64_t n,
             int64_t chunk, PushTargets dst, const SparseScratch* s) {
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
            if (u_mask != nullptr) u_mask[e0 + j] = 0.0f;   // DGC's momentum factor masking
          }
        }
        gt_before += above;
        eq_before += at;
      }
      run_gt += __shfl_sync(0xffffffffu, inc_gt, 31);
      run_eq += __shfl_sync(0xffffffffu, inc_eq, 31);
    }
  }
  if (sumsq_to_clear != nullptr && blockIdx.x == 0 && threadIdx.x == 0) *sumsq_to_clear = 0.f;
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

// Scan form, DGC with momentum correction: the state update as a pass of its own
// (u = m*u + s*g, v += u, g = 0), with the same rounding as the list form's collect pass.
__global__ void __launch_bounds__(kThreads)
dgc_update_kernel(SparseFuseDev fuse, float* __restrict__ R, int64_t n) {
  const float scale = dgc_clip_scale(fuse);
  float* gw = const_cast<float*>(fuse.grad);
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float u = dgc_new_u(fuse.u[i], fuse.grad[i], fuse.momentum, scale);
    fuse.u[i] = u;
    R[i] = __fadd_rn(R[i], u);
    if (fuse.zero_grad) gw[i] = 0.f;
  }
}

// ================================================================ list form
// Pool of list blocks, behind the sample keys in the scratch: block b holds count[b] (index,
// value bits) pairs in entry[b * 16 ..] and continues in block next[b].  Three flat arrays, so
// that the cut kernel can sweep all entries with coalesced, independent loads.
struct ListPool {
  unsigned int* count;
  unsigned int* next;
  uint2* entry;
  uint32_t* dense;        // the candidates' keys once more, densely packed in no particular order
  unsigned int capacity;  // blocks
};

// Cursor of a warp's list; only lane 0's copy is used.
struct ListCursor {
  unsigned int block = kNoBlock, fill = 0, lost = 0, total = 0;
  bool exhausted = false;
};

// Appends this step's candidates of the calling warp to the warp's list, in lane order and,
// within a lane, element order.  count: candidates of this lane (0..4); idx / val: their
// indices and values.  Candidates are rare (0.1 % of the elements), so the entries are handed
// to lane 0 by shuffle and appended one at a time; a list grows by one block of the pool when
// its last block is full.
__device__ __forceinline__ void list_append(SparseScratch* s, const ListPool& pool, int list, int lane,
                                            unsigned int count, const uint32_t (&idx)[4], const float (&val)[4],
                                            ListCursor& cur) {
  unsigned int mask = __ballot_sync(0xffffffffu, count != 0);
  while (mask != 0) {
    const int src = __ffs(mask) - 1;
    mask &= mask - 1;
    const unsigned int c = __shfl_sync(0xffffffffu, count, src);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t i = __shfl_sync(0xffffffffu, idx[j], src);
      const float v = __shfl_sync(0xffffffffu, val[j], src);
      if (lane != 0 || j >= int(c)) continue;
      if (cur.exhausted) {
        ++cur.lost;
        continue;
      }
      if (cur.block == kNoBlock || cur.fill == kBlockEntries) {
        const unsigned int id = atomicAdd(&s->pool_used, 1u);
        if (id >= pool.capacity) {
          cur.exhausted = true;
          ++cur.lost;
          continue;
        }
        pool.count[id] = 0;
        pool.next[id] = kNoBlock;
        if (cur.block == kNoBlock) s->list_head[list] = id;
        else pool.next[cur.block] = id;
        cur.block = id;
        cur.fill = 0;
      }
      pool.entry[size_t(cur.block) * kBlockEntries + cur.fill] = make_uint2(i, __float_as_uint(v));
      pool.count[cur.block] = ++cur.fill;
      ++cur.total;
    }
  }
}

// ---- the one pass over the tensor
// MODE = fuse.mode as a template parameter (no registers for arrays a mode does not read); four
// CTAs per SM, so that the whole grid of 4 x 148 CTAs is resident at once.
template <int MODE>
__global__ void __launch_bounds__(kThreads, 4)
collect_kernel(SparseFuseDev fuse, float* __restrict__ R, int64_t n, int64_t chunk, int64_t sample_cnt,
               SparseScratch* s, ListPool pool) {
  fuse.mode = MODE;
  constexpr int kWarps = kThreads / 32;
  constexpr int U = MODE == 2 ? 2 : 4;   // steps whose loads are issued together
  uint32_t thr_key = 0;
  if (sample_cnt > 0) {
    unsigned int bin, rin;
    pick_from_top(s->shist[2], s->s_rank[2], bin, rin);
    thr_key = extend_prefix(s->s_prefix[2], 2, bin);
  }
  __syncthreads();
  if (blockIdx.x == 0 && threadIdx.x == 0) s->thr_key = thr_key;
  const float scale = dgc_clip_scale(fuse);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int list = blockIdx.x * kWarps + warp;
  const int64_t begin = int64_t(blockIdx.x) * chunk;
  const int64_t end = begin + chunk < n ? begin + chunk : n;
  // warp ranges: multiples of 128 elements so that every step is 32 lanes x 4 elements
  int64_t wlen = (end - begin + kWarps - 1) / kWarps;
  wlen = (wlen + 127) / 128 * 128;
  const int64_t wbegin = begin + warp * wlen < end ? begin + warp * wlen : end;
  const int64_t wend = wbegin + wlen < end ? wbegin + wlen : end;
  uintptr_t bits = reinterpret_cast<uintptr_t>(R);
  if (MODE >= 1) bits |= reinterpret_cast<uintptr_t>(fuse.grad);
  if (MODE == 2) bits |= reinterpret_cast<uintptr_t>(fuse.u);
  const bool vec_ok = (bits & 15) == 0 && (begin & 3) == 0;
  float* gw = const_cast<float*>(fuse.grad);   // mode 2 leaves zeros behind

  ListCursor cur;
  if (lane == 0) s->list_head[list] = kNoBlock;

  // state update + candidate test of the 4 elements at e0 (e0 + 3 < wend, 16-byte aligned)
  auto step4 = [&](int64_t e0, float4 r4, float4 g4, float4 u4, uint32_t (&idx)[4], float (&val)[4]) -> unsigned int {
    float r[4] = {r4.x, r4.y, r4.z, r4.w};
    if (MODE == 1) {
      const float g[4] = {g4.x, g4.y, g4.z, g4.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) r[j] = hp_add(g[j], r[j]);
      *reinterpret_cast<float4*>(R + e0) = make_float4(r[0], r[1], r[2], r[3]);
      if (fuse.zero_grad) *reinterpret_cast<float4*>(gw + e0) = make_float4(0.f, 0.f, 0.f, 0.f);
    } else if (MODE == 2) {
      const float g[4] = {g4.x, g4.y, g4.z, g4.w};
      float u[4] = {u4.x, u4.y, u4.z, u4.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        u[j] = dgc_new_u(u[j], g[j], fuse.momentum, scale);
        r[j] = __fadd_rn(r[j], u[j]);
      }
      *reinterpret_cast<float4*>(fuse.u + e0) = make_float4(u[0], u[1], u[2], u[3]);
      *reinterpret_cast<float4*>(R + e0) = make_float4(r[0], r[1], r[2], r[3]);
      if (fuse.zero_grad) *reinterpret_cast<float4*>(gw + e0) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    unsigned int count = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (abs_key(r[j]) > thr_key) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {   // compile-time indices keep idx / val in registers
          if (c == int(count)) {
            idx[c] = uint32_t(e0 + j);
            val[c] = r[j];
          }
        }
        ++count;
      }
    }
    return count;
  };

  int64_t base = wbegin;
  if (vec_ok) {
    // U steps per iteration with their loads issued together
    for (; base + U * 128 <= wend; base += U * 128) {
      float4 r4[U], g4[MODE >= 1 ? U : 1] = {}, u4[MODE == 2 ? U : 1] = {};
#pragma unroll
      for (int q = 0; q < U; ++q) {
        const int64_t e0 = base + q * 128 + lane * 4;
        r4[q] = *reinterpret_cast<const float4*>(R + e0);
        if (MODE >= 1) g4[MODE >= 1 ? q : 0] = __ldg(reinterpret_cast<const float4*>(fuse.grad + e0));
        if (MODE == 2) u4[MODE == 2 ? q : 0] = *reinterpret_cast<const float4*>(fuse.u + e0);
      }
#pragma unroll
      for (int q = 0; q < U; ++q) {
        uint32_t idx[4] = {0u, 0u, 0u, 0u};
        float val[4] = {0.f, 0.f, 0.f, 0.f};
        const unsigned int count = step4(base + q * 128 + lane * 4, r4[q], g4[MODE >= 1 ? q : 0], u4[MODE == 2 ? q : 0], idx, val);
        if (__ballot_sync(0xffffffffu, count != 0) != 0) list_append(s, pool, list, lane, count, idx, val, cur);
      }
    }
  }
  // the rest of the warp's range, element by element within steps of 128
  for (; base < wend; base += 128) {
    uint32_t idx[4] = {0u, 0u, 0u, 0u};
    float val[4] = {0.f, 0.f, 0.f, 0.f};
    unsigned int count = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t e = base + lane * 4 + j;
      if (e < wend) {
        float r = R[e];
        if (MODE == 1) {
          r = hp_add(fuse.grad[e], r);
          R[e] = r;
          if (fuse.zero_grad) gw[e] = 0.f;
        } else if (MODE == 2) {
          const float u = dgc_new_u(fuse.u[e], fuse.grad[e], fuse.momentum, scale);
          r = __fadd_rn(r, u);
          fuse.u[e] = u;
          R[e] = r;
          if (fuse.zero_grad) gw[e] = 0.f;
        }
        if (abs_key(r) > thr_key) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            if (c == int(count)) {
              idx[c] = uint32_t(e);
              val[c] = r;
            }
          }
          ++count;
        }
      }
    }
    if (__ballot_sync(0xffffffffu, count != 0) != 0) list_append(s, pool, list, lane, count, idx, val, cur);
  }
  // The cut kernel wants all candidate keys in one flat array (it is a single CTA: a sweep over
  // the half-empty list blocks cost it 70 us).  Each warp copies the keys of its own list, which
  // it has just written, to a range it reserves with one atomic.
  if (lane == 0 && cur.lost != 0) atomicAdd(&s->dropped, cur.lost);
  const unsigned int total = __shfl_sync(0xffffffffu, cur.total, 0);
  if (total != 0) {
    unsigned int base = 0;
    if (lane == 0) base = atomicAdd(&s->cand, total);
    base = __shfl_sync(0xffffffffu, base, 0);
    __syncwarp();   // lane 0's list writes are visible to the other lanes
    unsigned int done = 0;
    for (unsigned int b = s->list_head[list]; b != kNoBlock && b < pool.capacity; b = pool.next[b]) {
      const unsigned int c = pool.count[b];
      if (lane < int(c)) pool.dense[base + done + lane] = pool.entry[size_t(b) * kBlockEntries + lane].y & 0x7fffffffu;
      done += c;
    }
  }
}

// ---- one CTA: the exact cut among the candidates, when there are more than wanted
constexpr int kCutThreads = 1024;
constexpr int kCutSmemKeys = 48 * 1024;   // keys held in shared memory (192 KB)

// Block-wide over kCutThreads threads: the bin holding the element of 0-indexed `rank` counted
// from the top bin down, and the rank inside that bin.  Every thread returns the same pair.
__device__ void pick_from_top_1024(const unsigned int* hist, unsigned int rank, unsigned int& bin,
                                   unsigned int& rank_in_bin, unsigned int* part /* [kCutThreads] */,
                                   unsigned int* res /* [2] */) {
  constexpr int PER = kBins / kCutThreads;  // 2 bins per thread
  const int t = threadIdx.x;
  unsigned int local[PER];
  unsigned int sum = 0;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    local[j] = hist[kBins - 1 - (t * PER + j)];
    sum += local[j];
  }
  // inclusive scan of the per-thread sums: warp scans, then a scan of the 32 warp totals
  const int lane = t & 31, warp = t >> 5;
  unsigned int inc = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned int a = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += a;
  }
  if (lane == 31) part[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    const unsigned int x = part[lane];
    unsigned int sx = x;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned int a = __shfl_up_sync(0xffffffffu, sx, o);
      if (lane >= o) sx += a;
    }
    part[lane] = sx - x;   // exclusive
  }
  __syncthreads();
  const unsigned int before = part[warp] + inc - sum;
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

__global__ void __launch_bounds__(kCutThreads)
cut_kernel(unsigned int expected, SparseScratch* s, ListPool pool) {
  extern __shared__ uint32_t keys[];   // kCutSmemKeys
  __shared__ unsigned int sh[kBins];
  __shared__ unsigned int part[kCutThreads];
  __shared__ unsigned int res[2];
  const unsigned int cand = s->cand;
  if (cand <= expected) {
    if (threadIdx.x == 0) {
      s->cut_key = s->thr_key;
      s->ties_kept = 0;
    }
    return;
  }
  const bool in_smem = cand <= unsigned(kCutSmemKeys);
  if (in_smem) {
    // eight independent loads per thread and iteration
    for (unsigned int base = 0; base < cand; base += kCutThreads * 8) {
      uint32_t k[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const unsigned int i = base + u * kCutThreads + threadIdx.x;
        k[u] = i < cand ? pool.dense[i] : 0u;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const unsigned int i = base + u * kCutThreads + threadIdx.x;
        if (i < cand) keys[i] = k[u];
      }
    }
    __syncthreads();
  }
  const unsigned int count = cand;
  uint32_t prefix = 0;
  unsigned int rank = expected - 1;   // 0-based from the top
  for (int round = 0; round < 3; ++round) {
    for (int i = threadIdx.x; i < kBins; i += kCutThreads) sh[i] = 0;
    __syncthreads();
    // whole warps iterate together: candidate keys share their leading bits (same exponent), so
    // the lanes that hit the same bin are counted by one of them (one atomic per bin and warp)
    const unsigned int count_padded = (count + 31u) & ~31u;
    for (unsigned int i = threadIdx.x; i < count_padded; i += kCutThreads) {
      uint32_t key = 0;
      bool live = i < count;
      if (live) {
        key = in_smem ? keys[i] : pool.dense[i];   // more candidates than shared memory holds: from L2
      }
      live = live && prefix_matches(key, round, prefix);
      const int bin = live ? digit_of(key, round) : -1;
      const unsigned int same = __match_any_sync(0xffffffffu, bin);
      if (live && (threadIdx.x & 31) == __ffs(same) - 1) atomicAdd(&sh[bin], unsigned(__popc(same)));
    }
    __syncthreads();
    unsigned int bin, rin;
    pick_from_top_1024(sh, rank, bin, rin, part, res);
    prefix = extend_prefix(prefix, round, bin);
    rank = rin;
  }
  if (threadIdx.x == 0) {
    s->cut_key = prefix;
    s->ties_kept = rank + 1;
  }
}

// ---- one warp per list: kept counts against the cut; the last CTA: offsets, k, header, housekeeping
__global__ void __launch_bounds__(kThreads)
count_scan_kernel(int lists, PushTargets dst, SparseScratch* s, ListPool pool, float* sumsq_to_clear) {
  resolve_epoch(dst);
  constexpr int kWarps = kThreads / 32;
  __shared__ unsigned int w_gt[kWarps], w_eq[kWarps];
  __shared__ bool is_last;
  __shared__ unsigned int part_gt[kThreads], part_eq[kThreads];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int list = blockIdx.x * kWarps + warp;
  const uint32_t cut = s->cut_key;
  unsigned int gt = 0, eq = 0;
  if (list < lists) {
    for (unsigned int b = s->list_head[list]; b != kNoBlock && b < pool.capacity; b = pool.next[b]) {
      const unsigned int c = pool.count[b];
      const uint32_t key = lane < int(c) ? (pool.entry[size_t(b) * kBlockEntries + lane].y & 0x7fffffffu) : 0u;
      gt += __popc(__ballot_sync(0xffffffffu, lane < int(c) && key > cut));
      eq += __popc(__ballot_sync(0xffffffffu, lane < int(c) && key == cut));
    }
    if (lane == 0) {
      s->list_gt[list] = gt;
      s->list_eq[list] = eq;
    }
  }
  if (lane == 0) {
    w_gt[warp] = gt;
    w_eq[warp] = eq;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned int a = 0, b = 0;
    for (int w = 0; w < kWarps; ++w) {
      a += w_gt[w];
      b += w_eq[w];
    }
    s->cnt_gt[blockIdx.x] = a;
    s->cnt_eq[blockIdx.x] = b;
    __threadfence();
    is_last = atomicAdd(&s->lists_done, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  // exclusive scan of the per-CTA totals (at most kMaxBlocks of them)
  const int ctas = gridDim.x;
  const int per = (ctas + kThreads - 1) / kThreads;
  const int c0 = threadIdx.x * per, c1 = (c0 + per < ctas) ? c0 + per : ctas;
  unsigned int a = 0, b = 0;
  for (int c = c0; c < c1; ++c) {
    const unsigned int x = reinterpret_cast<volatile unsigned int*>(s->cnt_gt)[c];
    const unsigned int y = reinterpret_cast<volatile unsigned int*>(s->cnt_eq)[c];
    s->off_gt[c] = a;   // exclusive within this thread's run; the run's base is added below
    s->off_eq[c] = b;
    a += x;
    b += y;
  }
  part_gt[threadIdx.x] = a;
  part_eq[threadIdx.x] = b;
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned int rg = 0, re = 0;
    for (int i = 0; i < kThreads; ++i) {
      const unsigned int x = part_gt[i], y = part_eq[i];
      part_gt[i] = rg;
      part_eq[i] = re;
      rg += x;
      re += y;
    }
    const unsigned int ties = s->ties_kept;
    const unsigned int k = rg + (re < ties ? re : ties);
    s->k = k;
    s->last_cand = s->cand;
    const uint32_t total = 4u + 8u * k;
    uint8_t header[4];
    for (int i = 0; i < 4; ++i) header[i] = uint8_t(total >> (8 * i));
    push_bytes(dst, 0, header, 4);
    s->pool_used = 0;
    s->cand = 0;
    s->lists_done = 0;
    if (sumsq_to_clear != nullptr) *sumsq_to_clear = 0.f;
  }
  __syncthreads();
  for (int c = c0; c < c1; ++c) {
    s->off_gt[c] += part_gt[threadIdx.x];
    s->off_eq[c] += part_eq[threadIdx.x];
  }
  unsigned int* h = &s->shist[0][0];
  for (int i = threadIdx.x; i < 3 * kBins; i += kThreads) h[i] = 0;
}

// ---- one warp per list: deliver, clear the emitted positions, publish
__global__ void __launch_bounds__(kThreads)
emit_kernel(float* __restrict__ R, float* __restrict__ u_mask, int lists, PushTargets dst,
            const SparseScratch* s, ListPool pool) {
  resolve_epoch(dst);
  constexpr int kWarps = kThreads / 32;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int list = blockIdx.x * kWarps + warp;
  const uint32_t cut = s->cut_key;
  const unsigned int ties = s->ties_kept, k_total = s->k;
  if (list < lists) {
    // what the lists before this one keep: the CTA's offset plus the earlier warps of the CTA
    unsigned int run_gt = s->off_gt[blockIdx.x], run_eq = s->off_eq[blockIdx.x];
    for (int w = 0; w < warp; ++w) {
      run_gt += s->list_gt[blockIdx.x * kWarps + w];
      run_eq += s->list_eq[blockIdx.x * kWarps + w];
    }
    for (unsigned int b = s->list_head[list]; b != kNoBlock && b < pool.capacity; b = pool.next[b]) {
      const unsigned int c = pool.count[b];
      uint2 en = make_uint2(0u, 0u);
      if (lane < int(c)) en = pool.entry[size_t(b) * kBlockEntries + lane];
      const uint32_t key = en.y & 0x7fffffffu;
      const bool above = lane < int(c) && key > cut, at = lane < int(c) && key == cut;
      const unsigned int ma = __ballot_sync(0xffffffffu, above), me = __ballot_sync(0xffffffffu, at);
      const unsigned int lt = (1u << lane) - 1u;
      const unsigned int gt_before = run_gt + __popc(ma & lt), eq_before = run_eq + __popc(me & lt);
      if (above || (at && eq_before < ties)) {
        const unsigned int pos = gt_before + (eq_before < ties ? eq_before : ties);
        if (pos < k_total) {
          push_u32(dst, 4 + 4 * int64_t(pos), en.x);
          push_u32(dst, 4 + 4 * int64_t(k_total) + 4 * int64_t(pos), en.y);
          R[en.x] = 0.0f;
          if (u_mask != nullptr) u_mask[en.x] = 0.0f;
        }
      }
      run_gt += __popc(ma);
      run_eq += __popc(me);
    }
  }
  publish_when_grid_done(dst);
}

// out[idx] = 0 for every index of every payload: puts a dense buffer that only holds scattered
// payload entries back to all zeros without a pass over the whole buffer.
struct ClearSources {
  const uint8_t* payload[kMaxWorld];
  int64_t cap[kMaxWorld];
};
__global__ void __launch_bounds__(kThreads)
clear_kernel(ClearSources src, float* __restrict__ out, int64_t n, const uint32_t* epoch_dev, int64_t parity_stride,
             const int* guard) {
  if (status_guarded(guard)) return;
  const uint8_t* payload = src.payload[0];
  int64_t cap = src.cap[0];
#pragma unroll
  for (int r = 1; r < kMaxWorld; ++r) {
    if (r == int(blockIdx.y)) {
      payload = src.payload[r];
      cap = src.cap[r];
    }
  }
  if (epoch_dev != nullptr && (*epoch_dev & 1u)) payload += parity_stride;
  uint32_t total = 0;
  for (int k = 0; k < 4; ++k) total |= uint32_t(payload[k]) << (8 * k);
  if (total < 4 || int64_t(total) > cap) return;   // reported by the scatter kernel
  const int64_t k = (int64_t(total) - 4) / 8;
  const uint32_t* idx = reinterpret_cast<const uint32_t*>(payload + 4);
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t x = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; x < k; x += stride) {
    const uint32_t i = idx[x];
    if (int64_t(i) < n) out[i] = 0.0f;
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

namespace {

// Layout of the scratch behind SparseScratch: sample keys, then the pool of list blocks.  Both
// are sized from n alone, so that one allocation serves every keep fraction and sample rate a
// caller may pick later; a call whose sample or expected candidate count does not fit takes the
// scan form, which needs neither.
struct ListPlan {
  int64_t key_capacity;    // sample keys
  int64_t pool_blocks;
  size_t keys_offset, pool_offset, total_bytes;
};
inline ListPlan list_plan(int64_t n) {
  ListPlan p;
  p.key_capacity = n / 100 + 1024;
  // candidates: 6 % of n (six times the largest expectation the list form serves) plus a floor
  // that covers thresholds drawn from a handful of samples, plus one partly filled block per list
  const int64_t entries = n / 100 * 6 + 65536;
  p.pool_blocks = entries / kBlockEntries + kMaxLists;
  p.keys_offset = (sizeof(SparseScratch) + 255) / 256 * 256;
  p.pool_offset = (p.keys_offset + size_t(p.key_capacity) * 4 + 255) / 256 * 256;
  // count[blocks], next[blocks], entry[blocks][16], dense[blocks * 16]
  p.total_bytes = p.pool_offset + size_t(p.pool_blocks) * (8 + kBlockEntries * (sizeof(uint2) + 4)) + 512;
  return p;
}

}  // namespace

size_t sparse_scratch_bytes(int64_t n) { return list_plan(n < 1 ? 1 : n).total_bytes; }

cudaError_t sparse_compress_fused(const SparseFuse& fuse, float* R, int64_t n, double sample_rate,
                                  double keep_fraction, uint64_t seed, const PushTargets& dst, void* scratch,
                                  cudaStream_t stream) {
  if (n <= 0 || n > 0x7fffffff || scratch == nullptr || R == nullptr) return cudaErrorInvalidValue;
  if (fuse.mode < 0 || fuse.mode > 2 || (fuse.mode >= 1 && fuse.grad == nullptr) || (fuse.mode == 2 && fuse.u == nullptr))
    return cudaErrorInvalidValue;
  for (int p = 0; p < dst.world; ++p)
    if (reinterpret_cast<uintptr_t>(dst.payload[p]) & 3) return cudaErrorInvalidValue;
  auto* s = static_cast<SparseScratch*>(scratch);
  const Plan pl = plan_for(n);
  int64_t expected = sparse_expected_k(n, keep_fraction);
  if (expected > n) expected = n;
  const int64_t sample_cnt = sparse_sample_count(n, sample_rate);
  int64_t rank0 = sparse_threshold_rank(sample_cnt, keep_fraction);
  if (sample_cnt > 0 && rank0 > sample_cnt - 1) rank0 = sample_cnt - 1;
  const ListPlan lp = list_plan(n);
  SparseFuseDev f{fuse.grad, fuse.u, fuse.momentum, fuse.clip, fuse.sumsq, fuse.zero_grad, fuse.mode};
  uint32_t* keys = sample_cnt <= lp.key_capacity
                       ? reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(scratch) + lp.keys_offset) : nullptr;
  // the list form: keep fractions up to 1 %, and a pool that holds the candidates with a wide
  // margin: their number is about n (rank0+1) / (samples+1) with a relative spread of
  // 1 / sqrt(rank0+1); without sampling every non-zero element is a candidate
  bool lists = keep_fraction <= kListMaxKeep && sample_cnt > 0;
  if (lists) {
    const double mean = double(n) * double(rank0 + 1) / double(sample_cnt + 1);
    const double need = mean * (1.0 + 40.0 / std::sqrt(double(rank0 + 1)));
    lists = need <= double(lp.pool_blocks - kMaxLists) * kBlockEntries;
  }
  if (fuse.mode == 2 && fuse.clip > 0.f) {
    if (fuse.sumsq == nullptr) return cudaErrorInvalidValue;
    cudaError_t e = dgc_sumsq(fuse.grad, n, const_cast<float*>(fuse.sumsq), stream);
    if (e != cudaSuccess) return e;
  }
  if (sample_cnt > 0) {
    int64_t sb = (sample_cnt + kThreads - 1) / kThreads;
    if (sb > kMaxBlocks) sb = kMaxBlocks;
    sample_round_kernel<0><<<int(sb), kThreads, 0, stream>>>(f, R, n, sample_cnt, unsigned(rank0), seed, s, keys, dst.epoch_dev);
    sample_round_kernel<1><<<int(sb), kThreads, 0, stream>>>(f, R, n, sample_cnt, unsigned(rank0), seed, s, keys, dst.epoch_dev);
    sample_round_kernel<2><<<int(sb), kThreads, 0, stream>>>(f, R, n, sample_cnt, unsigned(rank0), seed, s, keys, dst.epoch_dev);
  }
  PushTargets hdr = dst;
  hdr.done = nullptr;
  if (lists) {
    uint8_t* pool_base = static_cast<uint8_t*>(scratch) + lp.pool_offset;
    ListPool pool;
    pool.capacity = static_cast<unsigned int>(lp.pool_blocks);
    pool.count = reinterpret_cast<unsigned int*>(pool_base);
    pool.next = pool.count + lp.pool_blocks;
    pool.entry = reinterpret_cast<uint2*>((reinterpret_cast<uintptr_t>(pool.next + lp.pool_blocks) + 127) & ~uintptr_t(127));
    pool.dense = reinterpret_cast<uint32_t*>(pool.entry + size_t(lp.pool_blocks) * kBlockEntries);
    const int nlists = pl.blocks * (kThreads / 32);
    if (fuse.mode == 2) collect_kernel<2><<<pl.blocks, kThreads, 0, stream>>>(f, R, n, pl.chunk, sample_cnt, s, pool);
    else if (fuse.mode == 1) collect_kernel<1><<<pl.blocks, kThreads, 0, stream>>>(f, R, n, pl.chunk, sample_cnt, s, pool);
    else collect_kernel<0><<<pl.blocks, kThreads, 0, stream>>>(f, R, n, pl.chunk, sample_cnt, s, pool);
    {
      cudaError_t e = cudaFuncSetAttribute(cut_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           kCutSmemKeys * int(sizeof(uint32_t)));
      if (e != cudaSuccess) return e;
    }
    cut_kernel<<<1, kCutThreads, kCutSmemKeys * sizeof(uint32_t), stream>>>(unsigned(expected), s, pool);
    count_scan_kernel<<<pl.blocks, kThreads, 0, stream>>>(
        nlists, hdr, s, pool, fuse.mode == 2 && fuse.clip > 0.f ? const_cast<float*>(fuse.sumsq) : nullptr);
    emit_kernel<<<pl.blocks, kThreads, 0, stream>>>(R, fuse.mode == 2 ? fuse.u : nullptr, nlists, dst, s, pool);
    return cudaGetLastError();
  }
  // scan form
  if (fuse.mode == 2) {
    dgc_update_kernel<<<pl.blocks, kThreads, 0, stream>>>(f, R, n);
  }
  count_kernel<<<pl.blocks, kThreads, 0, stream>>>(fuse.grad, R, n, pl.chunk, sample_cnt, unsigned(rank0),
                                                   fuse.mode == 1 ? 1 : 0, fuse.zero_grad, s);
  trim_round_kernel<1><<<pl.blocks, kThreads, 0, stream>>>(R, n, pl.chunk, unsigned(expected), s);
  trim_round_kernel<2><<<pl.blocks, kThreads, 0, stream>>>(R, n, pl.chunk, unsigned(expected), s);
  recount_kernel<<<pl.blocks, kThreads, 0, stream>>>(R, n, pl.chunk, unsigned(expected), s);
  scan_kernel<<<1, 1024, 0, stream>>>(pl.blocks, hdr, s);
  write_kernel<<<pl.blocks, kThreads, 0, stream>>>(R, fuse.mode == 2 ? fuse.u : nullptr,
                                                   fuse.mode == 2 && fuse.clip > 0.f ? const_cast<float*>(fuse.sumsq) : nullptr,
                                                   n, pl.chunk, dst, s);
  return cudaGetLastError();
}

cudaError_t sparse_compress(const float* grad, float* R, int64_t n, double sample_rate,
                            double keep_fraction, uint64_t seed, int accumulate,
                            const PushTargets& dst, void* scratch, cudaStream_t stream) {
  SparseFuse fuse;
  fuse.mode = accumulate ? 1 : 0;
  fuse.grad = accumulate ? grad : nullptr;
  return sparse_compress_fused(fuse, R, n, sample_rate, keep_fraction, seed, dst, scratch, stream);
}

// Counters of the last compress call that used `scratch`: {elements emitted, candidates over the
// sampled threshold (list form; 0 otherwise), threshold as the bit pattern of a float, candidates
// dropped so far because the pool was full}.  Copied to the host on `stream`.
cudaError_t sparse_read_stats(const void* scratch, unsigned int* host4, cudaStream_t stream) {
  const auto* s = static_cast<const SparseScratch*>(scratch);
  cudaError_t e = cudaMemcpyAsync(host4 + 0, &s->k, 4, cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaMemcpyAsync(host4 + 1, &s->last_cand, 4, cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaMemcpyAsync(host4 + 2, &s->thr_key, 4, cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaMemcpyAsync(host4 + 3, &s->dropped, 4, cudaMemcpyDeviceToHost, stream);
  return e;
}

cudaError_t sparse_clear(const UnpackSources& src, float* out, int64_t n, cudaStream_t stream) {
  if (n <= 0 || src.world < 1 || src.world > kMaxWorld) return cudaErrorInvalidValue;
  ClearSources cs{};
  int64_t kmax = 1;
  for (int r = 0; r < src.world; ++r) {
    if (reinterpret_cast<uintptr_t>(src.payload[r]) & 3) return cudaErrorInvalidValue;
    cs.payload[r] = src.payload[r];
    cs.cap[r] = src.payload_bytes[r];
    kmax = std::max<int64_t>(kmax, (src.payload_bytes[r] - 4) / 8);
  }
  int64_t blocks = (kmax + kThreads - 1) / kThreads;
  if (blocks > 148 * 2) blocks = 148 * 2;
  clear_kernel<<<dim3(unsigned(blocks), unsigned(src.world), 1), kThreads, 0, stream>>>(cs, out, n, src.epoch_dev,
                                                                                          src.parity_stride, src.guard);
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
