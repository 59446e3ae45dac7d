// One-pass decode + accumulate of up to 8 packed payloads through shared-memory tables.
//
// A payload byte holds DPB = 8/bitwidth quantised elements.  Instead of extracting and
// dequantising every field with integer and floating-point instructions (which made the first
// version of these kernels issue-bound at ~136 instructions per element for 8 ranks), each CTA
// first builds decode tables with the same contraction-free arithmetic as the CPU codec, and
// the main loop needs one 32-bit payload load per 4 bytes and rank plus table reads and adds.
//
// The decoded values of the ranks are summed in the canonical pairwise order (tree_sum in
// codec_math.h), so the result is bit-identical to the CPU codec on every replica.  Three table
// forms, fastest first:
//   pair tables     2-bit payloads, 16-byte aligned dense arrays: ranks (2s, 2s+1) share a table
//                   indexed by one nibble of each, whose entry already holds the pair's sum
//                   (the first level of the canonical order), so eight ranks cost four
//                   shared-memory reads and three adds per two elements
//   nibble tables   bitwidths 1, 2, 4 at any alignment
//   byte tables     bitwidth 8 or unknown
#pragma once
#include "../common/codec_math.h"
#include "kernels.h"
#include "p2p.cuh"

namespace hipress {
namespace cuda {

constexpr int kUnpackThreads = 256;

__device__ __forceinline__ uint32_t load_u32_any(const uint8_t* p) {
  if ((reinterpret_cast<uintptr_t>(p) & 3) == 0) return *reinterpret_cast<const uint32_t*>(p);
  return uint32_t(p[0]) | (uint32_t(p[1]) << 8) | (uint32_t(p[2]) << 16) | (uint32_t(p[3]) << 24);
}

__device__ __forceinline__ void sgd_update4(const SgdApply& a, int64_t i, const float* g) {
  const float4 p4 = *reinterpret_cast<const float4*>(a.param + i);
  float4 b4 = a.first_step ? make_float4(0, 0, 0, 0) : *reinterpret_cast<const float4*>(a.momentum + i);
  float p[4] = {p4.x, p4.y, p4.z, p4.w};
  float b[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float d = g[k] + a.weight_decay * p[k];
    b[k] = a.first_step ? d : a.mu * b[k] + d;
    p[k] -= a.lr * b[k];
  }
  *reinterpret_cast<float4*>(a.momentum + i) = make_float4(b[0], b[1], b[2], b[3]);
  *reinterpret_cast<float4*>(a.param + i) = make_float4(p[0], p[1], p[2], p[3]);
}

// True when an earlier kernel of the step recorded a failure: the caller returns without writing.
__device__ __forceinline__ bool unpack_guarded(const UnpackSources& src) {
  return src.guard != nullptr && *reinterpret_cast<const volatile int*>(src.guard) != 0;
}

// payload[j] for a run-time j without indexing the kernel-parameter array dynamically (which
// would move the whole struct into local memory): a chain of selects over compile-time indices.
__device__ __forceinline__ const uint8_t* select_payload(const UnpackSources& src, int j) {
  const uint8_t* p = src.payload[0];
#pragma unroll
  for (int r = 1; r < kMaxWorld; ++r)
    if (r == j) p = src.payload[r];
  return p;
}
__device__ __forceinline__ int64_t select_payload_bytes(const UnpackSources& src, int j) {
  int64_t b = src.payload_bytes[0];
#pragma unroll
  for (int r = 1; r < kMaxWorld; ++r)
    if (r == j) b = src.payload_bytes[r];
  return b;
}

// Elements of shard j when a tensor of n elements is cut into shards of S.
__device__ __forceinline__ int64_t shard_count(int64_t n, int64_t S, int j) {
  const int64_t left = n - int64_t(j) * S;
  return left <= 0 ? 0 : (left < S ? left : S);
}

// Finish one group of 4 consecutive elements: accumulate mode, scale, store, fused update.
// The group lives at o[off .. off+3]; e is its index in the tensor (for the fused update).
template <bool APPLY>
__device__ __forceinline__ void unpack_finish4(float (&acc)[4], float* __restrict__ o, int off, int add,
                                               float post_scale, const SgdApply& apply, int64_t e) {
  if (add) {
    const float4 x = *reinterpret_cast<const float4*>(o + off);
    acc[0] = hp_add(acc[0], x.x); acc[1] = hp_add(acc[1], x.y);
    acc[2] = hp_add(acc[2], x.z); acc[3] = hp_add(acc[3], x.w);
  }
  if (post_scale != 1.0f) {
#pragma unroll
    for (int k = 0; k < 4; ++k) acc[k] = hp_mul(acc[k], post_scale);
  }
  const bool clear = APPLY && apply.clear_grad;
  *reinterpret_cast<float4*>(o + off) =
      clear ? make_float4(0.f, 0.f, 0.f, 0.f) : make_float4(acc[0], acc[1], acc[2], acc[3]);
  if (APPLY) sgd_update4(apply, e, acc);
}
template <bool APPLY>
__device__ __forceinline__ void unpack_finish4(float (&acc)[4], float* __restrict__ out, int64_t e, int add,
                                               float post_scale, const SgdApply& apply) {
  unpack_finish4<APPLY>(acc, out + e, 0, add, post_scale, apply, e);
}
template <bool APPLY>
__device__ __forceinline__ void unpack_finish1(float acc, float* __restrict__ out, int64_t e, int add,
                                               float post_scale, const SgdApply& apply) {
  if (add) acc = hp_add(acc, out[e]);
  if (post_scale != 1.0f) acc = hp_mul(acc, post_scale);
  out[e] = (APPLY && apply.clear_grad) ? 0.f : acc;
  if (APPLY) sgd_update(apply, e, acc);
}

// Table row of byte value v.  Gradient payloads are dominated by a few byte values (fields
// near the middle levels); with rows stored in natural order those values fall on only four
// of the eight 16-byte bank groups and every table read is a multi-way bank conflict.  XOR-ing
// two higher bits into the low bits spreads them over all eight groups (a bijection on 0..255).
__device__ __forceinline__ uint32_t lut_row(uint32_t v) { return v ^ ((v >> 3) & 5u); }

// ---------------------------------------------------------------- byte tables
// lut: shared memory, entry (rank r, byte v, slot j) at lut[(r*256 + lut_row(v))*DPB + j].
// data_offset: bytes to skip at the start of each payload (header size + slot shift).
template <int DPB, bool APPLY>
__device__ __forceinline__ void unpack_lut_body(const float* lut, const UnpackSources& src, int64_t data_offset,
                                                float* __restrict__ out, int64_t n, int add,
                                                float post_scale, const SgdApply& apply) {
  constexpr int EPG = 4 * DPB;  // elements per group of 4 payload bytes
  constexpr int VW = DPB >= 4 ? 4 : DPB;  // values fetched per table read
  const int64_t full_groups = n / EPG;
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  const bool vec = ((reinterpret_cast<uintptr_t>(out) |
                     (APPLY ? (reinterpret_cast<uintptr_t>(apply.param) |
                               reinterpret_cast<uintptr_t>(apply.momentum)) : uintptr_t(0))) & 15) == 0;
  int64_t grp = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  // payload words of the group being decoded; the next group's words are requested before
  // the current ones are used, so their latency hides behind the decode
  uint32_t w[kMaxWorld];
#pragma unroll
  for (int r = 0; r < kMaxWorld; ++r)
    w[r] = (r < src.world && grp < full_groups) ? load_u32_any(src.payload[r] + data_offset + grp * 4) : 0u;
  for (; grp < full_groups; grp += stride) {
    const int64_t e0 = grp * EPG;
    const int64_t nxt = grp + stride;
    uint32_t wn[kMaxWorld];
#pragma unroll
    for (int r = 0; r < kMaxWorld; ++r)
      wn[r] = (r < src.world && nxt < full_groups) ? load_u32_any(src.payload[r] + data_offset + nxt * 4) : 0u;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
#pragma unroll
      for (int q = 0; q < DPB / VW; ++q) {
        float v[VW][kMaxWorld];
#pragma unroll
        for (int r = 0; r < kMaxWorld; ++r) {
          if (r < src.world) {
            const float* e = lut + (size_t(r) * 256 + lut_row((w[r] >> (8 * b)) & 255u)) * DPB + q * VW;
            if (VW == 4) {
              const float4 t = *reinterpret_cast<const float4*>(e);
              v[0][r] = t.x; v[1][r] = t.y; v[2][r] = t.z; v[3][r] = t.w;
            } else if (VW == 2) {
              const float2 t = *reinterpret_cast<const float2*>(e);
              v[0][r] = t.x; v[1][r] = t.y;
            } else {
              v[0][r] = e[0];
            }
          }
        }
        float acc[VW];
#pragma unroll
        for (int k = 0; k < VW; ++k) acc[k] = tree_sum(v[k], src.world);
        const int64_t e = e0 + b * DPB + q * VW;
        if (VW == 4 && vec) {
          if constexpr (VW == 4) unpack_finish4<APPLY>(acc, out, e, add, post_scale, apply);
        } else {
#pragma unroll
          for (int k = 0; k < VW; ++k) unpack_finish1<APPLY>(acc[k], out, e + k, add, post_scale, apply);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < kMaxWorld; ++r) w[r] = wn[r];
  }
  // fewer than EPG leftover elements: one thread, element by element
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    for (int64_t e = full_groups * EPG; e < n; ++e) {
      float v[kMaxWorld];
#pragma unroll
      for (int r = 0; r < kMaxWorld; ++r) {
        if (r < src.world) {
          const uint32_t byte = src.payload[r][data_offset + e / DPB];
          v[r] = lut[(size_t(r) * 256 + lut_row(byte)) * DPB + int(e % DPB)];
        }
      }
      unpack_finish1<APPLY>(tree_sum(v, src.world), out, e, add, post_scale, apply);
    }
  }
}

// ---------------------------------------------------------------- nibble tables
// The byte table above costs one 16-byte shared-memory read per payload byte, and because a
// rank's table spans 4 KB, rows of different bytes collide on banks (measured: 2.2 wavefronts
// per quarter-warp read for 2-bit gradient payloads).  For bitwidths 1, 2 and 4 the table can
// instead be indexed by a 4-bit nibble: 16 rows of 4/BW floats.  At 2 bits a rank's table is
// exactly 128 bytes -- one row of all 32 banks -- so any two lanes either read the same row
// (a broadcast) or different banks: the reads are conflict free whatever the data.
//
// lut: entry (rank r, nibble v, slot j) at lut[(r*16 + v)*DPN + j], DPN = 4/BW (r = 0 when shared).
//
// The first payload words of a thread are requested by unpack_nibble_prefetch *before* the
// kernel reads headers and builds its tables, so that the DRAM latency of the first loads and
// the dependent loads of the prologue overlap instead of adding up.  A word is only requested
// when it lies inside the slot (payload_bytes), whatever the header will turn out to say.
// header_bytes: bytes before the packed data inside a slot; slot_shift: where this step's slot
// starts relative to src.payload[r] (the epoch-parity offset; 0 unless the epoch lives on the device).
template <int BW>
__device__ __forceinline__ void unpack_nibble_prefetch(const UnpackSources& src, int header_bytes,
                                                       int64_t slot_shift, int64_t n,
                                                       uint32_t (&w)[kMaxWorld]) {
  constexpr int EPG = 8 * (4 / BW);
  const int64_t grp = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
#pragma unroll
  for (int r = 0; r < kMaxWorld; ++r)
    w[r] = (r < src.world && grp < n / EPG && header_bytes + (grp + 1) * 4 <= src.payload_bytes[r])
               ? load_u32_any(src.payload[r] + slot_shift + header_bytes + grp * 4)
               : 0u;
}

// SHARED: all ranks decode through one table (TBQ); otherwise rank r's table starts 16 rows
// after rank r-1's.  w: the words unpack_nibble_prefetch returned for this thread.
template <int BW, bool APPLY, bool SHARED>
__device__ __forceinline__ void unpack_nibble_body(const float* lut, uint32_t (&w)[kMaxWorld],
                                                   const UnpackSources& src, int64_t data_offset,
                                                   float* __restrict__ out, int64_t n, int add,
                                                   float post_scale, const SgdApply& apply) {
  static_assert(BW == 1 || BW == 2 || BW == 4, "nibble tables cover bitwidths 1, 2 and 4");
  constexpr int DPN = 4 / BW;                                  // elements per nibble
  constexpr int EPG = 8 * DPN;                                 // elements per 32-bit payload word
  constexpr int ROW_SHIFT = DPN == 4 ? 4 : (DPN == 2 ? 3 : 2);  // log2(bytes per table row)
  constexpr int rank_stride = SHARED ? 0 : 16;
  const int64_t full_groups = n / EPG;
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  int64_t grp = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  for (; grp < full_groups; grp += stride) {
    const int64_t e0 = grp * EPG;
    const int64_t nxt = grp + stride;
    uint32_t wn[kMaxWorld];
#pragma unroll
    for (int r = 0; r < kMaxWorld; ++r)
      wn[r] = (r < src.world && nxt < full_groups) ? load_u32_any(src.payload[r] + data_offset + nxt * 4) : 0u;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float v[DPN][kMaxWorld];
#pragma unroll
      for (int r = 0; r < kMaxWorld; ++r) {
        if (r < src.world) {
          const char* table = reinterpret_cast<const char*>(lut) + r * rank_stride * DPN * 4;
          // byte offset of the row of nibble k: ((w >> 4k) & 15) << ROW_SHIFT in one shift + mask
          const uint32_t off = (4 * k >= ROW_SHIFT ? (w[r] >> (4 * k - ROW_SHIFT)) : (w[r] << (ROW_SHIFT - 4 * k))) &
                               (15u << ROW_SHIFT);
          if (DPN == 4) {
            const float4 t = *reinterpret_cast<const float4*>(table + off);
            v[0][r] = t.x; v[1 % DPN][r] = t.y; v[2 % DPN][r] = t.z; v[3 % DPN][r] = t.w;
          } else if (DPN == 2) {
            const float2 t = *reinterpret_cast<const float2*>(table + off);
            v[0][r] = t.x; v[1 % DPN][r] = t.y;
          } else {
            v[0][r] = *reinterpret_cast<const float*>(table + off);
          }
        }
      }
#pragma unroll
      for (int j = 0; j < DPN; ++j)
        unpack_finish1<APPLY>(tree_sum(v[j], src.world), out, e0 + k * DPN + j, add, post_scale, apply);
    }
#pragma unroll
    for (int r = 0; r < kMaxWorld; ++r) w[r] = wn[r];
  }
  // fewer than EPG leftover elements: one thread, element by element
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    constexpr int DPB = 8 / BW;
    for (int64_t e = full_groups * EPG; e < n; ++e) {
      const int in_byte = int(e % DPB);
      float v[kMaxWorld];
#pragma unroll
      for (int r = 0; r < kMaxWorld; ++r) {
        if (r < src.world) {
          const uint32_t byte = src.payload[r][data_offset + e / DPB];
          const uint32_t nib = (byte >> (4 * (in_byte / DPN))) & 15u;
          v[r] = lut[(size_t(r) * rank_stride + nib) * DPN + in_byte % DPN];
        }
      }
      unpack_finish1<APPLY>(tree_sum(v, src.world), out, e, add, post_scale, apply);
    }
  }
}

// ---------------------------------------------------------------- pair tables, 2 bits
// Slot s covers ranks (2s, 2s+1).  Its table has 256 rows of two floats: row (b << 4) | a holds
// decode_{2s}(a) + decode_{2s+1}(b) for the two elements of nibbles a and b, i.e. the first
// level of the canonical sum is read, not computed.  A last rank without a partner uses rows
// 0..15 of its slot (b = 0), which hold its decoded values alone.
//
// Index words: for payload words wa, wb of the two ranks, lo = (wa & 0x0f0f0f0f) | ((wb << 4) &
// 0xf0f0f0f0) packs the four row numbers of the even nibbles into the bytes of one register and
// hi = ((wa >> 4) & 0x0f0f0f0f) | (wb & 0xf0f0f0f0) those of the odd nibbles: eight look-ups
// cost four logic instructions to prepare.  Rows are stored swizzled, row ^ ((row >> 4) & 5):
// gradient nibbles are mostly 5, 6, 9 or 10 (both fields on a middle level), and without the
// swizzle two lanes that agree in a and differ in b hit the same bank on different rows.
//
// Mapping: lane L of a warp handles payload byte j*32 + L (j = 0..3) of the warp's 128-byte
// chunk, i.e. elements (j*32 + L)*4 .. +3 of the chunk's 512: every dense access is a 512-byte
// contiguous run across the warp.  Payloads are loaded one 32-bit word per lane and rank; index
// words reach their lanes by shuffle.
constexpr int kPairRows = 256;
__device__ __forceinline__ uint32_t pair_swizzle(uint32_t packed_rows) {
  return packed_rows ^ ((packed_rows >> 4) & 0x05050505u);
}

// value(r, nibble, which): decoded value of element `which` (0/1) of a nibble of rank r.
// tables: [slots][256][2] floats; slots = (world + 1) / 2, or one table when SHARED (all ranks
// decode alike, and the lone rank of an odd world reads the pair rows of a partner that decodes
// to zero: lone_nibble is that partner's nibble).
template <bool SHARED, typename Value>
__device__ __forceinline__ void build_pair_tables(float* tables, int world, Value value) {
  const int slots = SHARED ? 1 : (world + 1) / 2;
  for (int i = threadIdx.x; i < slots * kPairRows; i += blockDim.x) {
    const int s = i >> 8, row = i & 255, a = row & 15, b = row >> 4;
    const int ra = 2 * s, rb = 2 * s + 1;
    const bool lone = !SHARED && rb >= world;
    if (lone && b != 0) continue;
    float x = value(ra, a, 0), y = value(ra, a, 1);
    if (!lone) {
      x = hp_add(x, value(rb, b, 0));
      y = hp_add(y, value(rb, b, 1));
    }
    const int at = row ^ ((row >> 4) & 5);
    reinterpret_cast<float2*>(tables)[s * kPairRows + at] = make_float2(x, y);
  }
}

// WORLD is a template parameter: with the rank count known at compile time the loops below are
// straight-line code (a first version that tested `r < src.world` everywhere spent 60 % of its
// instructions on those tests and their branches).
template <bool APPLY, bool SHARED, int WORLD>
__device__ __forceinline__ void unpack_pair_body(const float* tables, uint32_t lone_word, uint32_t (&w)[kMaxWorld],
                                                 const UnpackSources& src, int64_t data_offset,
                                                 float* __restrict__ out, int64_t n, int add,
                                                 float post_scale, const SgdApply& apply) {
  constexpr int kSlots = (WORLD + 1) / 2;
  const int64_t full_chunks = n / 512;  // complete 128-byte warp chunks
  const int lane = threadIdx.x & 31;
  const uint32_t sel = 0x4440u | uint32_t(lane & 3);  // byte (lane & 3) of a register, zero-extended
  const int64_t warps = int64_t(gridDim.x) * (blockDim.x >> 5);
  int64_t chunk = int64_t(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  for (; chunk < full_chunks; chunk += warps) {
    const int64_t nxt = (chunk + warps) * 32 + lane;
    const bool more = chunk + warps < full_chunks;
    uint32_t wn[WORLD];
#pragma unroll
    for (int r = 0; r < WORLD; ++r)
      wn[r] = more ? load_u32_any(src.payload[r] + data_offset + nxt * 4) : 0u;
    uint32_t lo[kSlots], hi[kSlots];
#pragma unroll
    for (int s = 0; s < kSlots; ++s) {
      const uint32_t wa = w[2 * s];
      const uint32_t wb = (2 * s + 1 < WORLD) ? w[2 * s + 1] : lone_word;
      lo[s] = pair_swizzle((wa & 0x0f0f0f0fu) | ((wb << 4) & 0xf0f0f0f0u));
      hi[s] = pair_swizzle(((wa >> 4) & 0x0f0f0f0fu) | (wb & 0xf0f0f0f0u));
    }
    float* const o = out + chunk * 512 + lane * 4;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int from = j * 8 + (lane >> 2);
      float v[4][kSlots];
#pragma unroll
      for (int s = 0; s < kSlots; ++s) {
        const uint32_t l = __shfl_sync(0xffffffffu, lo[s], from);
        const uint32_t h = __shfl_sync(0xffffffffu, hi[s], from);
        const char* table = reinterpret_cast<const char*>(tables) + (SHARED ? 0 : s * kPairRows * 8);
        const float2 a = *reinterpret_cast<const float2*>(table + (__byte_perm(l, 0u, sel) << 3));
        const float2 b = *reinterpret_cast<const float2*>(table + (__byte_perm(h, 0u, sel) << 3));
        v[0][s] = a.x; v[1][s] = a.y; v[2][s] = b.x; v[3][s] = b.y;
      }
      float acc[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) acc[k] = tree_sum(v[k], kSlots);
      unpack_finish4<APPLY>(acc, o, j * 128, add, post_scale, apply, chunk * 512 + lane * 4 + j * 128);
    }
#pragma unroll
    for (int r = 0; r < WORLD; ++r) w[r] = wn[r];
  }
  // elements past the last complete chunk (fewer than 512): block 0, element by element,
  // through the same tables (rank pairs, then the canonical order over the slots)
  if (blockIdx.x == 0) {
    const uint32_t lone_nib = lone_word & 15u;
    for (int64_t e = full_chunks * 512 + threadIdx.x; e < n; e += blockDim.x) {
      float v[kSlots];
#pragma unroll
      for (int s = 0; s < kSlots; ++s) {
        const int sh = 4 * int((e & 3) >> 1);
        const uint32_t a = (uint32_t(src.payload[2 * s][data_offset + (e >> 2)]) >> sh) & 15u;
        uint32_t b = lone_nib;
        if (2 * s + 1 < WORLD) b = (uint32_t(src.payload[(2 * s + 1) % kMaxWorld][data_offset + (e >> 2)]) >> sh) & 15u;
        const uint32_t row = (b << 4) | a;
        v[s] = tables[((SHARED ? 0 : s) * kPairRows + (row ^ ((row >> 4) & 5u))) * 2 + (e & 1)];
      }
      unpack_finish1<APPLY>(tree_sum(v, kSlots), out, e, add, post_scale, apply);
    }
  }
}

// ---------------------------------------------------------------- concatenated shards, 2 bits
// Sharded exchange, last phase: payload[j] encodes shard j alone.  nib: [world or 1][16][2]
// nibble tables (rank j's at nib + j*32 floats; one table when SHARED).  Same lane mapping as
// the pair body; a 512-element chunk never straddles two shards (shard_elems % 2048 == 0).
// header_bytes + slot_shift: where the packed data starts inside payload[j].
template <bool APPLY, bool SHARED>
__device__ __forceinline__ void unpack_concat_body(const float* nib, const UnpackSources& src, int64_t data_offset,
                                                   float* __restrict__ out, int64_t n, int add,
                                                   float post_scale, const SgdApply& apply) {
  const int64_t S = src.shard_elems;
  const int64_t full_chunks = n / 512;
  const int lane = threadIdx.x & 31;
  const int64_t warps = int64_t(gridDim.x) * (blockDim.x >> 5);
  for (int64_t chunk = int64_t(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); chunk < full_chunks;
       chunk += warps) {
    const int64_t e_chunk = chunk * 512;
    const int j = int(e_chunk / S);
    const uint8_t* p = select_payload(src, j) + data_offset + ((e_chunk - int64_t(j) * S) >> 2);
    const uint32_t word = *reinterpret_cast<const uint32_t*>(p + lane * 4);
    const char* table = reinterpret_cast<const char*>(nib) + (SHARED ? 0 : j * 128);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint32_t wq = __shfl_sync(0xffffffffu, word, q * 8 + (lane >> 2));
      const uint32_t byte = (wq >> (8 * (lane & 3))) & 255u;
      const float2 lo = *reinterpret_cast<const float2*>(table + ((byte & 15u) << 3));
      const float2 hi = *reinterpret_cast<const float2*>(table + ((byte >> 4) << 3));
      float acc[4] = {lo.x, lo.y, hi.x, hi.y};
      unpack_finish4<APPLY>(acc, out, e_chunk + int64_t(q * 32 + lane) * 4, add, post_scale, apply);
    }
  }
  if (blockIdx.x == 0) {
    for (int64_t e = full_chunks * 512 + threadIdx.x; e < n; e += blockDim.x) {
      const int j = int(e / S);
      const int64_t le = e - int64_t(j) * S;
      const uint32_t byte = select_payload(src, j)[data_offset + (le >> 2)];
      const uint32_t nb = (byte >> (4 * ((le & 3) >> 1))) & 15u;
      unpack_finish1<APPLY>(nib[((SHARED ? 0 : j) * 16 + nb) * 2 + (le & 1)], out, e, add, post_scale, apply);
    }
  }
}

// True when the dense arrays allow the 16-byte accesses of the pair and concat bodies.
__device__ __forceinline__ bool unpack_coalesced_ok(const float* out, bool apply_on, const SgdApply& apply) {
  uintptr_t bits = reinterpret_cast<uintptr_t>(out);
  if (apply_on) bits |= reinterpret_cast<uintptr_t>(apply.param) | reinterpret_cast<uintptr_t>(apply.momentum);
  return (bits & 15) == 0;
}

}  // namespace cuda
}  // namespace hipress
