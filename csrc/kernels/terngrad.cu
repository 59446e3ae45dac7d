// Min-max k-bit quantiser ("TernGrad" codec of the reference) for sm_100a.
//
// Compress is two kernels and no host synchronisation:
//   1. minmax_header_kernel  grid reduction of min/max over grad (+ residual);
//      the last CTA derives gap and 1/(gap+1e-8) (in double, as the reference's
//      host code does: terngrad_body.h:205-206), stores them for kernel 2 and
//      writes the 10-byte header into every destination.
//   2. tern_quant_kernel     quantises with per-byte LCG stochastic rounding
//      (or round-half-even), packs, stores the bytes into every destination,
//      optionally writes the error-feedback residual, handles the always
//      deterministic partial last byte in-kernel, then publishes the flag.
// The reference needs minmax_element + D2H + sync, a header H2D, a transform,
// and a second D2H/sync/H2D for the tail (terngrad_body.h:186-298).
//
// Unpack-accumulate decodes the payloads of all ranks in one pass, each with
// its own header, in ascending rank order.
#include "../common/codec_math.h"
#include "kernels.h"
#include "p2p.cuh"
#include "reduce.cuh"
#include "unpack_lut.cuh"

#include <algorithm>

namespace hipress {
namespace cuda {

namespace {

constexpr int kThreads = 256;

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
inline int grid_for(int64_t items, int threads, int max_blocks) {
  int64_t blocks = (items + threads - 1) / threads;
  if (blocks < 1) blocks = 1;
  if (blocks > max_blocks) blocks = max_blocks;
  return int(blocks);
}

template <bool VEC, bool EF>
__global__ void __launch_bounds__(kThreads)
minmax_header_kernel(const float* __restrict__ grad, const float* __restrict__ residual, int64_t n,
                     int bw, PushTargets dst, MinMaxScratch* scratch) {
  if (push_guarded(dst)) return;
  resolve_epoch(dst);
  // scatter mode: blockIdx.y is the shard; each shard has its own reduction state and header
  PushCursor cur{nullptr};
  if (dst.shard_elems > 0) {
    const int j = blockIdx.y;
    const int64_t cnt = shard_len(n, dst.shard_elems, j);
    if (cnt == 0) return;
    grad += int64_t(j) * dst.shard_elems;
    if (EF) residual += int64_t(j) * dst.shard_elems;
    n = cnt;
    scratch += j;
    cur.one = select_dest(dst, j);
  }
  float mn = INFINITY, mx = -INFINITY;
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  const int64_t tid = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (VEC) {
    const int64_t nv = n >> 2;
    for (int64_t i = tid; i < nv; i += stride) {
      float4 g = __ldg(reinterpret_cast<const float4*>(grad) + i);
      if (EF) {
        const float4 r = __ldg(reinterpret_cast<const float4*>(residual) + i);
        g.x = hp_add(g.x, r.x); g.y = hp_add(g.y, r.y);
        g.z = hp_add(g.z, r.z); g.w = hp_add(g.w, r.w);
      }
      mn = fminf(mn, fminf(fminf(g.x, g.y), fminf(g.z, g.w)));
      mx = fmaxf(mx, fmaxf(fmaxf(g.x, g.y), fmaxf(g.z, g.w)));
    }
    for (int64_t i = (nv << 2) + tid; i < n; i += stride) {
      const float v = EF ? hp_add(grad[i], residual[i]) : grad[i];
      mn = fminf(mn, v);
      mx = fmaxf(mx, v);
    }
  } else {
    for (int64_t i = tid; i < n; i += stride) {
      const float v = EF ? hp_add(grad[i], residual[i]) : grad[i];
      mn = fminf(mn, v);
      mx = fmaxf(mx, v);
    }
  }
  float gmn, gmx;
  if (!grid_minmax_last_block<kThreads>(scratch, mn, mx, gmn, gmx)) return;
  if (threadIdx.x == 0) {
    const float gap = tern_gap(gmn, gmx, bw);
    scratch->mn = gmn;
    scratch->mx = gmx;
    scratch->gap = gap;
    scratch->inv = tern_gap_inverse(gap);
    uint8_t header[kTernHeaderBytes];
    header[0] = uint8_t(bw);
    header[1] = uint8_t(tern_tail(n, bw));
    const uint32_t a = __float_as_uint(gmn), b = __float_as_uint(gmx);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      header[2 + k] = uint8_t(a >> (8 * k));
      header[6 + k] = uint8_t(b >> (8 * k));
    }
    put_bytes(dst, cur, 0, header, kTernHeaderBytes);
  }
}

// Elements handled by one thread and bytes it produces.
template <int BW> struct Unit {
  static constexpr int DPB = 8 / BW;
  static constexpr int EPT = DPB > 4 ? DPB : 4;  // elements per thread
  static constexpr int BPT = EPT / DPB;          // bytes per thread: 1,1,2,4
};

constexpr int kStageBytes = 512;  // payload bytes a warp gathers before it stores them

// Quantise the EPT elements of one unit; returns its BPT payload bytes (little-endian).
template <int BW, bool EF>
__device__ __forceinline__ uint32_t tern_quant_unit(float (&x)[Unit<BW>::EPT], int64_t first_byte, float mn,
                                                    float inv, float gap, int random, uint64_t seed,
                                                    float (&ef)[Unit<BW>::EPT]) {
  constexpr int DPB = Unit<BW>::DPB, BPT = Unit<BW>::BPT;
  uint32_t bytes = 0;
#pragma unroll
  for (int b = 0; b < BPT; ++b) {
    const uint8_t q = tern_pack_byte<BW>(x + b * DPB, DPB, mn, inv, random != 0,
                                         tern_byte_seed(seed, first_byte + b), gap,
                                         EF ? ef + b * DPB : nullptr);
    bytes |= uint32_t(q) << (8 * b);
  }
  return bytes;
}

// wide: large tensors with 16-byte aligned destinations.  A warp then works on chunks of
// 512 payload bytes: in each of J = 16/BPT sub-steps lane L quantises unit j*32+L of the chunk
// (coalesced 16-byte loads), the bytes are gathered in shared memory, and every lane stores
// 16 of them to each destination -- 512 contiguous bytes per warp and destination, against the
// 32 bytes per warp of the word path, which is what NVLink peer stores need to run near link
// speed.  The rest of the tensor (less than one chunk) takes the word path.
template <int BW, bool VEC, bool EF>
__global__ void __launch_bounds__(kThreads)
tern_quant_kernel(const float* __restrict__ grad, float* __restrict__ residual, int64_t n,
                  int random, uint64_t seed, PushTargets dst, const MinMaxScratch* scratch, int wide) {
  if (push_guarded(dst)) return;
  resolve_epoch(dst);
  if (dst.epoch_dev != nullptr) seed += uint64_t(dst.epoch) * kEpochSeedStride;
  constexpr int DPB = Unit<BW>::DPB, EPT = Unit<BW>::EPT, BPT = Unit<BW>::BPT;
  const int64_t S = dst.shard_elems;
  // state of the shard in hand (the whole tensor unless in scatter mode)
  int cur_j = -1;
  PushCursor cur{nullptr};
  float mn = 0.f, inv = 0.f, gap = 0.f;
  uint64_t cur_seed = seed;
  auto enter = [&](int j) {   // (re)load what depends on the shard
    if (j == cur_j) return;
    cur_j = j;
    const MinMaxScratch* s = scratch + (S > 0 ? j : 0);
    mn = s->mn; inv = s->inv; gap = s->gap;
    if (S > 0) {
      cur.one = select_dest(dst, j);
      cur_seed = seed + uint64_t(j) * kShardSeedStride;
    }
  };
  if (S == 0) enter(0);

  // ---- chunks of 512 payload bytes
  constexpr int64_t CH = int64_t(kStageBytes) * DPB;
  int64_t chunks = 0;
  if (VEC && wide) {
    __shared__ __align__(16) uint8_t stage[kThreads / 32][kStageBytes];
    constexpr int J = 16 / BPT;           // sub-steps per chunk
    constexpr int U = EPT == 8 ? 2 : 4;   // sub-steps whose loads are issued together
    chunks = n / CH;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t warps = int64_t(gridDim.x) * (blockDim.x >> 5);
    for (int64_t c = int64_t(blockIdx.x) * (blockDim.x >> 5) + warp; c < chunks; c += warps) {
      int64_t ebase = c * CH;        // first element of the chunk in the tensor
      int64_t lbase = ebase;         // ... and relative to its shard
      if (S > 0) {
        const int j = int(ebase / S);
        enter(j);
        lbase = ebase - int64_t(j) * S;
      }
      const int64_t bbase = lbase / DPB;  // first payload byte of the chunk
#pragma unroll 1
      for (int j0 = 0; j0 < J; j0 += U) {
        float x[U][EPT], ef[U][EPT];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int64_t e0 = ebase + int64_t((j0 + u) * 32 + lane) * EPT;
#pragma unroll
          for (int v = 0; v < EPT / 4; ++v) {
            float4 g = __ldg(reinterpret_cast<const float4*>(grad + e0) + v);
            if (EF) {
              const float4 r = reinterpret_cast<const float4*>(residual + e0)[v];
              g.x = hp_add(g.x, r.x); g.y = hp_add(g.y, r.y);
              g.z = hp_add(g.z, r.z); g.w = hp_add(g.w, r.w);
            }
            x[u][4 * v] = g.x; x[u][4 * v + 1] = g.y; x[u][4 * v + 2] = g.z; x[u][4 * v + 3] = g.w;
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int unit = (j0 + u) * 32 + lane;
          const uint32_t bytes = tern_quant_unit<BW, EF>(x[u], bbase + int64_t(unit) * BPT, mn, inv, gap, random,
                                                         cur_seed, ef[u]);
          if (EF) {
            const int64_t e0 = ebase + int64_t(unit) * EPT;
#pragma unroll
            for (int v = 0; v < EPT / 4; ++v)
              reinterpret_cast<float4*>(residual + e0)[v] =
                  make_float4(ef[u][4 * v], ef[u][4 * v + 1], ef[u][4 * v + 2], ef[u][4 * v + 3]);
          }
          if (BPT == 1) stage[warp][unit] = uint8_t(bytes);
          else if (BPT == 2) reinterpret_cast<uint16_t*>(stage[warp])[unit] = uint16_t(bytes);
          else reinterpret_cast<uint32_t*>(stage[warp])[unit] = bytes;
        }
      }
      __syncwarp();
      const uint4 v = reinterpret_cast<const uint4*>(stage[warp])[lane];
      put_u128(dst, cur, kTernHeaderBytes + bbase + lane * 16, v);
      __syncwarp();
    }
  }

  // ---- the rest, one unit per thread: lanes combine their bytes into 32-bit words
  const int64_t rest_begin = chunks * CH;         // element
  int64_t rest_local = rest_begin;                // relative to its shard
  int64_t rest_n = n;                             // end of the rest, relative to its shard
  if (S > 0 && rest_begin < n) {
    const int j = int(rest_begin / S);
    enter(j);
    rest_local = rest_begin - int64_t(j) * S;
    rest_n = rest_local + (n - rest_begin);
  }
  const float* g_rest = grad + (rest_begin - rest_local);      // shard base
  float* r_rest = EF ? residual + (rest_begin - rest_local) : nullptr;
  const int64_t unit0 = rest_local / EPT;
  const int64_t units = rest_n / EPT;             // complete units of the shard
  const int64_t span = units - unit0;
  const int64_t span_padded = (span + 31) & ~int64_t(31);
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t k = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; k < span_padded; k += stride) {
    const int64_t u = unit0 + k;
    uint32_t bytes = 0;
    if (u < units) {
      float x[EPT], ef[EPT];
      const int64_t e0 = u * EPT;
      if (VEC) {
#pragma unroll
        for (int v = 0; v < EPT / 4; ++v) {
          float4 g = __ldg(reinterpret_cast<const float4*>(g_rest + e0) + v);
          if (EF) {
            const float4 r = reinterpret_cast<const float4*>(r_rest + e0)[v];
            g.x = hp_add(g.x, r.x); g.y = hp_add(g.y, r.y);
            g.z = hp_add(g.z, r.z); g.w = hp_add(g.w, r.w);
          }
          x[4 * v] = g.x; x[4 * v + 1] = g.y; x[4 * v + 2] = g.z; x[4 * v + 3] = g.w;
        }
      } else {
#pragma unroll
        for (int i = 0; i < EPT; ++i)
          x[i] = EF ? hp_add(g_rest[e0 + i], r_rest[e0 + i]) : g_rest[e0 + i];
      }
      bytes = tern_quant_unit<BW, EF>(x, u * BPT, mn, inv, gap, random, cur_seed, ef);
      if (EF) {
        if (VEC) {
#pragma unroll
          for (int v = 0; v < EPT / 4; ++v)
            reinterpret_cast<float4*>(r_rest + e0)[v] =
                make_float4(ef[4 * v], ef[4 * v + 1], ef[4 * v + 2], ef[4 * v + 3]);
        } else {
#pragma unroll
          for (int i = 0; i < EPT; ++i) r_rest[e0 + i] = ef[i];
        }
      }
    }
    // combine lanes into 32-bit words and store them (k and u differ by a multiple of 32 units
    // only when unit0 is one; the lane pattern below depends on the lane, not on u)
    if (BPT == 1) {
      const uint32_t word = gather4_bytes(bytes);
      if ((threadIdx.x & 3) == 0 && u < units) {
        if (u + 3 < units) {
          put_u32(dst, cur, kTernHeaderBytes + u, word);
        } else {
          for (int64_t b = u; b < units; ++b)
            put_u8(dst, cur, kTernHeaderBytes + b, uint8_t(word >> (8 * (b - u))));
        }
      }
    } else if (BPT == 2) {
      const uint32_t word = gather2_halves(bytes);
      if ((threadIdx.x & 1) == 0 && u < units) {
        if (u + 1 < units) {
          put_u32(dst, cur, kTernHeaderBytes + 2 * u, word);
        } else {
          put_u8(dst, cur, kTernHeaderBytes + 2 * u, uint8_t(word));
          put_u8(dst, cur, kTernHeaderBytes + 2 * u + 1, uint8_t(word >> 8));
        }
      }
    } else {
      if (u < units) put_u32(dst, cur, kTernHeaderBytes + 4 * u, bytes);
    }
  }
  // leftover elements (fewer than EPT): whole bytes keep the requested rounding
  // mode, the partial last byte is always deterministic
  const int64_t done_elems = units * EPT;
  if (done_elems < rest_n && blockIdx.x == 0 && threadIdx.x == 0) {
    int64_t byte_index = done_elems / DPB;
    for (int64_t e = done_elems; e < rest_n; e += DPB, ++byte_index) {
      const int count = (rest_n - e) >= DPB ? DPB : int(rest_n - e);
      float x[DPB], ef[DPB];
      for (int j = 0; j < count; ++j)
        x[j] = EF ? hp_add(g_rest[e + j], r_rest[e + j]) : g_rest[e + j];
      const bool rnd = random != 0 && count == DPB;
      const uint8_t q = tern_pack_byte<BW>(x, count, mn, inv, rnd,
                                           tern_byte_seed(cur_seed, byte_index), gap,
                                           EF ? ef : nullptr);
      put_u8(dst, cur, kTernHeaderBytes + byte_index, q);
      if (EF)
        for (int j = 0; j < count; ++j) r_rest[e + j] = ef[j];
    }
  }
  publish_when_grid_done(dst);
}

struct TernHeader {
  float mn, gap;
  int bw, ok;
};

__device__ __forceinline__ TernHeader read_header(const uint8_t* p, int64_t cap, int64_t n) {
  TernHeader h;
  h.bw = p[0];
  const int tail = p[1];
  uint32_t a = 0, b = 0;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    a |= uint32_t(p[2 + k]) << (8 * k);
    b |= uint32_t(p[6 + k]) << (8 * k);
  }
  h.mn = __uint_as_float(a);
  h.ok = tern_bitwidth_ok(h.bw) && tern_payload_bytes(n, h.bw) <= cap && tail == tern_tail(n, h.bw);
  h.gap = h.ok ? tern_gap(h.mn, __uint_as_float(b), h.bw) : 0.f;
  return h;
}

// Table-driven unpack (see unpack_lut.cuh).  All payloads of one call must
// carry the same bitwidth; it is read from the headers, so the host never has
// to look at a payload.  BW > 0 compiles the decode loop for that bitwidth only
// (fewer registers, more resident CTAs); BW == 0 dispatches on the header at
// run time for callers that do not know the bitwidth.
// MODE (chosen by the launcher, so that each form is its own kernel with its own register
// budget): kPair = pair tables (2 bits, aligned), kConcat = concatenated shards (2 bits,
// aligned), kGeneric = nibble or byte tables.
enum UnpackMode : int { kGeneric = 0, kPair = 1, kConcat = 2 };

template <int BW, bool APPLY, int MODE, int WORLD>
__global__ void __launch_bounds__(kUnpackThreads, MODE == kGeneric ? 1 : 4)
tern_unpack_lut_kernel(UnpackSources src, float* __restrict__ out, int64_t n, int add,
                       float post_scale, SgdApply apply, int* status) {
  if (unpack_guarded(src)) return;
  resolve_epoch(src);
  extern __shared__ __align__(16) float lut[];  // [world][256][dpb], byte-table path only
  // BW == 2: pair tables [slots][256][2] (8 KB), whose first 1 KB doubles as the per-rank nibble
  // tables of the unaligned and concatenated forms; BW == 1, 4: nibble tables only
  __shared__ __align__(128) float tab[MODE == kPair ? (kMaxWorld / 2) * kPairRows * 2
                                                   : ((BW == 1 || BW == 2 || BW == 4) ? kMaxWorld * 16 * (4 / (BW ? BW : 1)) : 1)];
  __shared__ TernHeader hdr[kMaxWorld];
  __shared__ int all_ok;
  constexpr bool concat = MODE == kConcat;
  uint32_t first[kMaxWorld];
  if constexpr ((BW == 1 || BW == 2 || BW == 4) && !concat)
    unpack_nibble_prefetch<BW>(src, kTernHeaderBytes, src.parity_off, n, first);
  if (threadIdx.x == 0) all_ok = 1;
  __syncthreads();
#pragma unroll
  for (int r = 0; r < kMaxWorld; ++r) {   // thread r reads header r; compile-time index into src
    if (int(threadIdx.x) == r && r < src.world) {
      // concatenated shards: payload r holds shard r only (possibly nothing)
      const int64_t count = concat ? shard_count(n, src.shard_elems, r) : n;
      if (count > 0) {
        hdr[r] = read_header(src.payload[r] + src.parity_off, src.payload_bytes[r], count);
        if (!hdr[r].ok) all_ok = 0;
      } else {
        hdr[r].ok = 1; hdr[r].bw = 0; hdr[r].mn = 0.f; hdr[r].gap = 0.f;
      }
    }
  }
  __syncthreads();
  int bw = BW;
  if (all_ok) {
    for (int r = 0; r < src.world; ++r) {  // every thread computes the same verdict
      if (hdr[r].bw == 0) continue;        // empty shard
      if (bw == 0) bw = hdr[r].bw;
      if (hdr[r].bw != bw) all_ok = 0;
    }
  }
  __syncthreads();
  if (!all_ok || bw == 0) {
    if (!all_ok && blockIdx.x == 0 && threadIdx.x == 0 && status) atomicExch(status, int(kBadHeader));
    return;
  }
  const int64_t data_offset = kTernHeaderBytes + src.parity_off;
  if constexpr (MODE == kPair) {
    build_pair_tables<false>(tab, src.world, [&](int r, int nibble, int which) {
      return tern_dequant((uint32_t(nibble) >> (2 * which)) & 3u, hdr[r].gap, hdr[r].mn);
    });
    __syncthreads();
    unpack_pair_body<APPLY, false, (WORLD > 0 ? WORLD : 1)>(tab, 0u, first, src, data_offset, out, n, add, post_scale, apply);
    return;
  } else if constexpr (BW == 1 || BW == 2 || BW == 4) {
    // nibble tables (see unpack_lut.cuh): entry (rank, nibble, slot)
    constexpr int DPN = 4 / BW;
    for (int i = threadIdx.x; i < src.world * 16 * DPN; i += blockDim.x) {
      const int r = i / (16 * DPN), v = (i / DPN) & 15, j = i % DPN;
      tab[i] = tern_dequant((uint32_t(v) >> (BW * j)) & ((1u << BW) - 1u), hdr[r].gap, hdr[r].mn);
    }
    __syncthreads();
    if constexpr (concat)
      unpack_concat_body<APPLY, false>(tab, src, data_offset, out, n, add, post_scale, apply);
    else
      unpack_nibble_body<BW, APPLY, false>(tab, first, src, data_offset, out, n, add, post_scale, apply);
    return;
  } else {
  const int dpb = 8 / bw;
  const uint32_t mask = (1u << bw) - 1u;
  for (int i = threadIdx.x; i < src.world * 256; i += blockDim.x) {
    const int r = i >> 8, v = i & 255;
    for (int j = 0; j < dpb; ++j)
      lut[(r * 256 + int(lut_row(uint32_t(v)))) * dpb + j] =
          tern_dequant((uint32_t(v) >> (bw * j)) & mask, hdr[r].gap, hdr[r].mn);
  }
  __syncthreads();
  if (BW > 0) {
    unpack_lut_body<8 / (BW > 0 ? BW : 1), APPLY>(lut, src, data_offset, out, n, add, post_scale, apply);
  } else {
    switch (bw) {
      case 1: unpack_lut_body<8, APPLY>(lut, src, data_offset, out, n, add, post_scale, apply); break;
      case 2: unpack_lut_body<4, APPLY>(lut, src, data_offset, out, n, add, post_scale, apply); break;
      case 4: unpack_lut_body<2, APPLY>(lut, src, data_offset, out, n, add, post_scale, apply); break;
      default: unpack_lut_body<1, APPLY>(lut, src, data_offset, out, n, add, post_scale, apply); break;
    }
  }
  }
}

template <int BW, bool APPLY>
cudaError_t launch_tern_unpack(const UnpackSources& src, float* out, int64_t n, int add, float post_scale,
                               const SgdApply& apply, int* status, cudaStream_t stream) {
  // table size: world x 256 x dpb floats; without a known bitwidth, room for 1-bit payloads (dpb = 8)
  const int dpb = BW > 0 ? 8 / BW : 8;
  const bool nibble = BW == 1 || BW == 2 || BW == 4;
  const size_t smem = nibble ? 0 : size_t(src.world) * 256 * dpb * sizeof(float);
  if (!nibble) {
    // per device, and cheap: set on every launch rather than remembered per process
    cudaError_t e = cudaFuncSetAttribute(tern_unpack_lut_kernel<BW, APPLY, kGeneric, 0>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 256 * 8 * 4);
    if (e != cudaSuccess) return e;
  }
  // a CTA decodes many groups so that building its tables stays small against the decode work
  const int64_t groups = (n + 4 * dpb - 1) / (4 * dpb);
  const int grid = grid_for(groups, kUnpackThreads, nibble ? 148 * 4 : 148 * 8);
  bool aligned = aligned16(out);
  if (APPLY) aligned = aligned && aligned16(apply.param) && aligned16(apply.momentum);
  if constexpr (BW == 2) {
    if (src.shard_elems > 0) {
      tern_unpack_lut_kernel<2, APPLY, kConcat, 0><<<grid, kUnpackThreads, 0, stream>>>(src, out, n, add, post_scale, apply, status);
      return cudaGetLastError();
    }
    if (aligned) {
#define HP_PAIR(W) \
  case W: tern_unpack_lut_kernel<2, APPLY, kPair, W><<<grid, kUnpackThreads, 0, stream>>>(src, out, n, add, post_scale, apply, status); break
      switch (src.world) {
        HP_PAIR(1); HP_PAIR(2); HP_PAIR(3); HP_PAIR(4); HP_PAIR(5); HP_PAIR(6); HP_PAIR(7); HP_PAIR(8);
        default: return cudaErrorInvalidValue;
      }
#undef HP_PAIR
      return cudaGetLastError();
    }
  }
  tern_unpack_lut_kernel<BW, APPLY, kGeneric, 0><<<grid, kUnpackThreads, smem, stream>>>(src, out, n, add, post_scale, apply, status);
  return cudaGetLastError();
}

}  // namespace

size_t minmax_scratch_bytes() { return sizeof(MinMaxScratch); }

cudaError_t terngrad_compress(const float* grad, float* residual, int64_t n, int bitwidth,
                              int enable_random, uint64_t seed, const PushTargets& dst,
                              void* scratch, cudaStream_t stream) {
  if (n <= 0 || !tern_bitwidth_ok(bitwidth) || scratch == nullptr) return cudaErrorInvalidValue;
  auto* s = static_cast<MinMaxScratch*>(scratch);
  const bool ef = residual != nullptr;
  const bool vec = aligned16(grad) && (!ef || aligned16(residual));
  const int64_t S = dst.shard_elems;
  bool dst16 = (dst.parity_stride & 15) == 0;
  for (int p = 0; p < dst.world; ++p) dst16 = dst16 && aligned16(dst.payload[p] + kTernHeaderBytes);
  if (dst.mc != nullptr) dst16 = dst16 && aligned16(dst.mc + kTernHeaderBytes);
  // scatter mode runs on the chunked path only (see tern_quant_kernel)
  if (S > 0 && (!vec || !dst16 || S % 4096 != 0 || (n + S - 1) / S > dst.world)) return cudaErrorInvalidValue;
  const int shards = S > 0 ? int((n + S - 1) / S) : 1;
  PushTargets hdr_dst = dst;
  hdr_dst.done = nullptr;  // only the quantising kernel publishes
  {
    const int64_t per = S > 0 ? (S < n ? S : n) : n;
    int gx = grid_for((per + 3) >> 2, kThreads, 148 * 4);
    if (shards > 1) gx = std::min(gx, std::max(1, (148 * 4 + shards - 1) / shards));
    const dim3 grid(gx, shards);
#define LAUNCH(V, E) \
  minmax_header_kernel<V, E><<<grid, kThreads, 0, stream>>>(grad, residual, n, bitwidth, hdr_dst, s)
    if (vec && ef) LAUNCH(true, true);
    else if (vec) LAUNCH(true, false);
    else if (ef) LAUNCH(false, true);
    else LAUNCH(false, false);
#undef LAUNCH
  }
  {
    // chunked path with 16-byte stores once there is a chunk per warp of a half-filled GPU
    const int dpb = 8 / bitwidth;
    const int64_t chunks = n / (int64_t(kStageBytes) * dpb);
    const int wide = (vec && dst16 && (S > 0 || chunks >= 148 * 2)) ? 1 : 0;
    const int threads = wide ? 128 : kThreads;
    const int grid = wide ? grid_for(chunks * 32, threads, 148 * 16)
                          : grid_for(n / (dpb > 4 ? dpb : 4), kThreads, 148 * 8);
#define LAUNCH2(BW, V, E) \
  tern_quant_kernel<BW, V, E><<<grid, threads, 0, stream>>>(grad, residual, n, enable_random, seed, dst, s, wide)
#define LAUNCH_BW(BW)                         \
  do {                                        \
    if (vec && ef) LAUNCH2(BW, true, true);   \
    else if (vec) LAUNCH2(BW, true, false);   \
    else if (ef) LAUNCH2(BW, false, true);    \
    else LAUNCH2(BW, false, false);           \
  } while (0)
    switch (bitwidth) {
      case 1: LAUNCH_BW(1); break;
      case 2: LAUNCH_BW(2); break;
      case 4: LAUNCH_BW(4); break;
      default: LAUNCH_BW(8); break;
    }
#undef LAUNCH_BW
#undef LAUNCH2
  }
  return cudaGetLastError();
}

cudaError_t terngrad_unpack_accum(const UnpackSources& src, float* out, int64_t n, int add,
                                  float post_scale, const SgdApply& apply, int* status,
                                  cudaStream_t stream, int bitwidth_hint) {
  if (n <= 0 || src.world < 1 || src.world > kMaxWorld) return cudaErrorInvalidValue;
  if (bitwidth_hint != 0 && !tern_bitwidth_ok(bitwidth_hint)) return cudaErrorInvalidValue;
  if (src.shard_elems > 0) {
    // concatenated shards: 2-bit payloads and 16-byte aligned dense arrays only
    bool ok = bitwidth_hint == 2 && src.shard_elems % 2048 == 0 && aligned16(out) &&
              (n + src.shard_elems - 1) / src.shard_elems <= src.world;
    if (apply.param != nullptr) ok = ok && aligned16(apply.param) && aligned16(apply.momentum);
    if (!ok) return cudaErrorInvalidValue;
  }
  const bool ap = apply.param != nullptr;
#define HP_UNPACK(BW) \
  (ap ? launch_tern_unpack<BW, true>(src, out, n, add, post_scale, apply, status, stream) \
      : launch_tern_unpack<BW, false>(src, out, n, add, post_scale, apply, status, stream))
  switch (bitwidth_hint) {
    case 1: return HP_UNPACK(1);
    case 2: return HP_UNPACK(2);
    case 4: return HP_UNPACK(4);
    case 8: return HP_UNPACK(8);
    default: return HP_UNPACK(0);
  }
#undef HP_UNPACK
}

}  // namespace cuda
}  // namespace hipress
