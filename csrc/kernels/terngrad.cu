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
  resolve_epoch(dst);
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
    push_bytes(dst, 0, header, kTernHeaderBytes);
  }
}

// Elements handled by one thread and bytes it produces.
template <int BW> struct Unit {
  static constexpr int DPB = 8 / BW;
  static constexpr int EPT = DPB > 4 ? DPB : 4;  // elements per thread
  static constexpr int BPT = EPT / DPB;          // bytes per thread: 1,1,2,4
};

template <int BW, bool VEC, bool EF>
__global__ void __launch_bounds__(kThreads)
tern_quant_kernel(const float* __restrict__ grad, float* __restrict__ residual, int64_t n,
                  int random, uint64_t seed, PushTargets dst, const MinMaxScratch* scratch) {
  resolve_epoch(dst);
  if (dst.epoch_dev != nullptr) seed += uint64_t(dst.epoch) * kEpochSeedStride;
  constexpr int DPB = Unit<BW>::DPB, EPT = Unit<BW>::EPT, BPT = Unit<BW>::BPT;
  const float mn = scratch->mn, inv = scratch->inv, gap = scratch->gap;
  const int64_t units = n / EPT;
  const int64_t units_padded = (units + 31) & ~int64_t(31);
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t u = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; u < units_padded; u += stride) {
    uint32_t bytes = 0;
    if (u < units) {
      float x[EPT], ef[EPT];
      const int64_t e0 = u * EPT;
      if (VEC) {
#pragma unroll
        for (int v = 0; v < EPT / 4; ++v) {
          float4 g = __ldg(reinterpret_cast<const float4*>(grad + e0) + v);
          if (EF) {
            const float4 r = reinterpret_cast<const float4*>(residual + e0)[v];
            g.x = hp_add(g.x, r.x); g.y = hp_add(g.y, r.y);
            g.z = hp_add(g.z, r.z); g.w = hp_add(g.w, r.w);
          }
          x[4 * v] = g.x; x[4 * v + 1] = g.y; x[4 * v + 2] = g.z; x[4 * v + 3] = g.w;
        }
      } else {
#pragma unroll
        for (int k = 0; k < EPT; ++k)
          x[k] = EF ? hp_add(grad[e0 + k], residual[e0 + k]) : grad[e0 + k];
      }
#pragma unroll
      for (int b = 0; b < BPT; ++b) {
        const int64_t byte_index = u * BPT + b;
        const uint8_t q = tern_pack_byte<BW>(x + b * DPB, DPB, mn, inv, random != 0,
                                             tern_byte_seed(seed, byte_index), gap,
                                             EF ? ef + b * DPB : nullptr);
        bytes |= uint32_t(q) << (8 * b);
      }
      if (EF) {
        if (VEC) {
#pragma unroll
          for (int v = 0; v < EPT / 4; ++v)
            reinterpret_cast<float4*>(residual + e0)[v] =
                make_float4(ef[4 * v], ef[4 * v + 1], ef[4 * v + 2], ef[4 * v + 3]);
        } else {
#pragma unroll
          for (int k = 0; k < EPT; ++k) residual[e0 + k] = ef[k];
        }
      }
    }
    // combine lanes into 32-bit words and store them to every destination
    if (BPT == 1) {
      const uint32_t word = gather4_bytes(bytes);
      if ((threadIdx.x & 3) == 0 && u < units) {
        if (u + 3 < units) {
          push_u32(dst, kTernHeaderBytes + u, word);
        } else {
          for (int64_t b = u; b < units; ++b)
            push_u8(dst, kTernHeaderBytes + b, uint8_t(word >> (8 * (b - u))));
        }
      }
    } else if (BPT == 2) {
      const uint32_t word = gather2_halves(bytes);
      if ((threadIdx.x & 1) == 0 && u < units) {
        if (u + 1 < units) {
          push_u32(dst, kTernHeaderBytes + 2 * u, word);
        } else {
          push_u8(dst, kTernHeaderBytes + 2 * u, uint8_t(word));
          push_u8(dst, kTernHeaderBytes + 2 * u + 1, uint8_t(word >> 8));
        }
      }
    } else {
      if (u < units) push_u32(dst, kTernHeaderBytes + 4 * u, bytes);
    }
  }
  // leftover elements (fewer than EPT): whole bytes keep the requested rounding
  // mode, the partial last byte is always deterministic
  const int64_t done_elems = units * EPT;
  if (done_elems < n && blockIdx.x == 0 && threadIdx.x == 0) {
    int64_t byte_index = done_elems / DPB;
    for (int64_t e = done_elems; e < n; e += DPB, ++byte_index) {
      const int count = (n - e) >= DPB ? DPB : int(n - e);
      float x[DPB], ef[DPB];
      for (int j = 0; j < count; ++j)
        x[j] = EF ? hp_add(grad[e + j], residual[e + j]) : grad[e + j];
      const bool rnd = random != 0 && count == DPB;
      const uint8_t q = tern_pack_byte<BW>(x, count, mn, inv, rnd,
                                           tern_byte_seed(seed, byte_index), gap,
                                           EF ? ef : nullptr);
      push_u8(dst, kTernHeaderBytes + byte_index, q);
      if (EF)
        for (int j = 0; j < count; ++j) residual[e + j] = ef[j];
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
template <int BW, bool APPLY>
__global__ void __launch_bounds__(kUnpackThreads)
tern_unpack_lut_kernel(UnpackSources src, float* __restrict__ out, int64_t n, int add,
                       float post_scale, SgdApply apply, int* status) {
  resolve_epoch(src);
  extern __shared__ __align__(16) float lut[];  // [world][256][dpb], byte-table path only
  __shared__ __align__(128) float nib[(BW == 1 || BW == 2 || BW == 4) ? kMaxWorld * 16 * (4 / (BW ? BW : 1)) : 1];
  __shared__ TernHeader hdr[kMaxWorld];
  __shared__ int all_ok;
  uint32_t first[kMaxWorld];
  if constexpr (BW == 1 || BW == 2 || BW == 4) unpack_nibble_prefetch<BW>(src, kTernHeaderBytes, src.parity_off, n, first);
  if (threadIdx.x == 0) all_ok = 1;
  __syncthreads();
#pragma unroll
  for (int r = 0; r < kMaxWorld; ++r) {   // thread r reads header r; compile-time index into src
    if (int(threadIdx.x) == r && r < src.world) {
      hdr[r] = read_header(src.payload[r] + src.parity_off, src.payload_bytes[r], n);
      if (!hdr[r].ok) all_ok = 0;
    }
  }
  __syncthreads();
  const int bw = BW > 0 ? BW : hdr[0].bw;
  if (all_ok) {
    for (int r = 0; r < src.world; ++r)
      if (hdr[r].bw != bw) all_ok = 0;  // every thread computes the same verdict
  }
  __syncthreads();
  if (!all_ok) {
    if (blockIdx.x == 0 && threadIdx.x == 0 && status) atomicExch(status, int(kBadHeader));
    return;
  }
  if constexpr (BW == 1 || BW == 2 || BW == 4) {
    // nibble tables (see unpack_lut.cuh): entry (rank, nibble, slot)
    constexpr int DPN = 4 / BW;
    for (int i = threadIdx.x; i < src.world * 16 * DPN; i += blockDim.x) {
      const int r = i / (16 * DPN), v = (i / DPN) & 15, j = i % DPN;
      nib[i] = tern_dequant((uint32_t(v) >> (BW * j)) & ((1u << BW) - 1u), hdr[r].gap, hdr[r].mn);
    }
    __syncthreads();
    if constexpr (BW == 2) {
      if (unpack_coalesced_ok(src, out, APPLY, apply)) {
        unpack_nibble_body_coalesced2<APPLY, false>(nib, first, src, kTernHeaderBytes + src.parity_off, out, n, add, post_scale, apply);
        return;
      }
    }
    unpack_nibble_body<BW, APPLY, false>(nib, first, src, kTernHeaderBytes + src.parity_off, out, n, add, post_scale, apply);
    return;
  }
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
    unpack_lut_body<8 / (BW > 0 ? BW : 1), APPLY>(lut, 256, src, kTernHeaderBytes + src.parity_off, out, n, add, post_scale, apply);
  } else {
    switch (bw) {
      case 1: unpack_lut_body<8, APPLY>(lut, 256, src, kTernHeaderBytes + src.parity_off, out, n, add, post_scale, apply); break;
      case 2: unpack_lut_body<4, APPLY>(lut, 256, src, kTernHeaderBytes + src.parity_off, out, n, add, post_scale, apply); break;
      case 4: unpack_lut_body<2, APPLY>(lut, 256, src, kTernHeaderBytes + src.parity_off, out, n, add, post_scale, apply); break;
      default: unpack_lut_body<1, APPLY>(lut, 256, src, kTernHeaderBytes + src.parity_off, out, n, add, post_scale, apply); break;
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
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(tern_unpack_lut_kernel<BW, APPLY>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 256 * 8 * 4);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  // one thread decodes 4 payload bytes per rank and iteration; a CTA covers at least 4 K
  // elements so that building the table stays small against the decode work
  const int64_t groups = (n + 4 * dpb - 1) / (4 * dpb);
  const int grid = grid_for(groups, kUnpackThreads, nibble ? 148 * 4 : 148 * 8);
  tern_unpack_lut_kernel<BW, APPLY><<<grid, kUnpackThreads, smem, stream>>>(src, out, n, add, post_scale, apply, status);
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
  PushTargets hdr_dst = dst;
  hdr_dst.done = nullptr;  // only the quantising kernel publishes
  {
    const int grid = grid_for((n + 3) >> 2, kThreads, 148 * 4);
#define LAUNCH(V, E) \
  minmax_header_kernel<V, E><<<grid, kThreads, 0, stream>>>(grad, residual, n, bitwidth, hdr_dst, s)
    if (vec && ef) LAUNCH(true, true);
    else if (vec) LAUNCH(true, false);
    else if (ef) LAUNCH(false, true);
    else LAUNCH(false, false);
#undef LAUNCH
  }
  {
#define LAUNCH2(BW, V, E)                                                                   \
  tern_quant_kernel<BW, V, E><<<grid_for(n / Unit<BW>::EPT, kThreads, 148 * 8), kThreads, 0, \
                                stream>>>(grad, residual, n, enable_random, seed, dst, s)
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
