// One-pass decode + accumulate of up to 8 packed payloads through a
// shared-memory byte table.
//
// A payload byte holds DPB = 8/bitwidth quantised elements.  Instead of
// extracting and dequantising every field with integer and floating-point
// instructions (which made the first version of these kernels issue-bound at
// ~136 instructions per element for 8 ranks), each CTA first builds, per rank,
// a table  byte value -> DPB decoded floats  (256 x DPB entries, computed with
// the same contraction-free arithmetic as the CPU codec), and the main loop
// then needs one 32-bit payload load per 4 bytes and one vector shared-memory
// load per byte, plus the adds.  Accumulation order is the canonical one
// (ascending rank, acc = decoded + acc), so results are bit-identical to
// decoding the payloads one after another.
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

// Table row of byte value v.  Gradient payloads are dominated by a few byte values (fields
// near the middle levels); with rows stored in natural order those values fall on only four
// of the eight 16-byte bank groups and every table read is a multi-way bank conflict.  XOR-ing
// two higher bits into the low bits spreads them over all eight groups (a bijection on 0..255).
__device__ __forceinline__ uint32_t lut_row(uint32_t v) { return v ^ ((v >> 3) & 5u); }

// lut: shared memory, entry (rank r, byte v, slot j) at lut[(r*rank_stride + lut_row(v))*DPB + j];
// rank_stride is 256 for per-rank tables and 0 when all ranks share one table.
// data_offset: bytes to skip at the start of each payload (header size).
template <int DPB, bool APPLY>
__device__ __forceinline__ void unpack_lut_body(const float* lut, int rank_stride,
                                                const UnpackSources& src, int64_t data_offset,
                                                float* __restrict__ out, int64_t n, int add,
                                                float post_scale, const SgdApply& apply) {
  constexpr int EPG = 4 * DPB;  // elements per group of 4 payload bytes
  const int64_t full_groups = n / EPG;
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  const bool out_vec = (reinterpret_cast<uintptr_t>(out) & 15) == 0;
  const bool apply_vec = APPLY && ((reinterpret_cast<uintptr_t>(apply.param) |
                                    reinterpret_cast<uintptr_t>(apply.momentum)) & 15) == 0;
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
    float acc[EPG];
    if (add) {
#pragma unroll
      for (int k = 0; k < EPG; ++k) acc[k] = out[e0 + k];
    }
#pragma unroll
    for (int r = 0; r < kMaxWorld; ++r) {
      if (r < src.world) {
        const float* table = lut + size_t(r) * rank_stride * DPB;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const float* e = table + lut_row((w[r] >> (8 * b)) & 255u) * DPB;
          float v[DPB];
          if (DPB % 4 == 0) {
#pragma unroll
            for (int q = 0; q < DPB / 4; ++q) {
              const float4 t = reinterpret_cast<const float4*>(e)[q];
              v[4 * q] = t.x; v[4 * q + 1] = t.y; v[4 * q + 2] = t.z; v[4 * q + 3] = t.w;
            }
          } else if (DPB == 2) {
            const float2 t = *reinterpret_cast<const float2*>(e);
            v[0] = t.x; v[1] = t.y;
          } else {
            v[0] = e[0];
          }
#pragma unroll
          for (int j = 0; j < DPB; ++j)
            acc[b * DPB + j] = (r == 0 && !add) ? v[j] : hp_add(v[j], acc[b * DPB + j]);
        }
      }
    }
    if (post_scale != 1.0f) {
#pragma unroll
      for (int k = 0; k < EPG; ++k) acc[k] = hp_mul(acc[k], post_scale);
    }
    const bool clear = APPLY && apply.clear_grad;
    if (out_vec) {
#pragma unroll
      for (int q = 0; q < EPG / 4; ++q)
        reinterpret_cast<float4*>(out + e0)[q] =
            clear ? make_float4(0.f, 0.f, 0.f, 0.f)
                  : make_float4(acc[4 * q], acc[4 * q + 1], acc[4 * q + 2], acc[4 * q + 3]);
    } else {
#pragma unroll
      for (int k = 0; k < EPG; ++k) out[e0 + k] = clear ? 0.f : acc[k];
    }
    if (APPLY) {
      if (apply_vec) {
#pragma unroll
        for (int q = 0; q < EPG / 4; ++q) sgd_update4(apply, e0 + 4 * q, acc + 4 * q);
      } else {
#pragma unroll
        for (int k = 0; k < EPG; ++k) sgd_update(apply, e0 + k, acc[k]);
      }
    }
#pragma unroll
    for (int r = 0; r < kMaxWorld; ++r) w[r] = wn[r];
  }
  // fewer than EPG leftover elements: one thread, element by element
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    for (int64_t e = full_groups * EPG; e < n; ++e) {
      float acc = add ? out[e] : 0.f;
#pragma unroll
      for (int r = 0; r < kMaxWorld; ++r) {
        if (r >= src.world) break;
        const uint32_t byte = src.payload[r][data_offset + e / DPB];
        const float v = lut[(size_t(r) * rank_stride + lut_row(byte)) * DPB + int(e % DPB)];
        acc = (r == 0 && !add) ? v : hp_add(v, acc);
      }
      if (post_scale != 1.0f) acc = hp_mul(acc, post_scale);
      out[e] = (APPLY && apply.clear_grad) ? 0.f : acc;
      if (APPLY) sgd_update(apply, e, acc);
    }
  }
}

// ---------------------------------------------------------------- nibble tables
// The byte table above costs one 16-byte shared-memory read per payload byte, and because a
// rank's table spans 4 KB, rows of different bytes collide on banks (measured: 2.2 wavefronts
// per quarter-warp read for 2-bit gradient payloads).  For bitwidths 1, 2 and 4 the table can
// instead be indexed by a 4-bit nibble: 16 rows of 4/BW floats.  At 2 bits a rank's table is
// exactly 128 bytes -- one row of all 32 banks -- so any two lanes either read the same row
// (a broadcast) or different banks: the reads are conflict free whatever the data, the table
// needs no swizzle, and building it is 16 entries per rank instead of 256.
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
  const bool out_vec = (reinterpret_cast<uintptr_t>(out) & 15) == 0;
  const bool apply_vec = APPLY && ((reinterpret_cast<uintptr_t>(apply.param) |
                                    reinterpret_cast<uintptr_t>(apply.momentum)) & 15) == 0;
  int64_t grp = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  for (; grp < full_groups; grp += stride) {
    const int64_t e0 = grp * EPG;
    const int64_t nxt = grp + stride;
    uint32_t wn[kMaxWorld];
#pragma unroll
    for (int r = 0; r < kMaxWorld; ++r)
      wn[r] = (r < src.world && nxt < full_groups) ? load_u32_any(src.payload[r] + data_offset + nxt * 4) : 0u;
    float acc[EPG];
    if (add) {
#pragma unroll
      for (int k = 0; k < EPG; ++k) acc[k] = out[e0 + k];
    }
#pragma unroll
    for (int r = 0; r < kMaxWorld; ++r) {
      if (r < src.world) {
        const char* table = reinterpret_cast<const char*>(lut) + r * rank_stride * DPN * 4;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          // byte offset of the row of nibble k: ((w >> 4k) & 15) << ROW_SHIFT in one shift + mask
          const uint32_t off = (4 * k >= ROW_SHIFT ? (w[r] >> (4 * k - ROW_SHIFT)) : (w[r] << (ROW_SHIFT - 4 * k))) &
                               (15u << ROW_SHIFT);
          float v[DPN];
          if (DPN == 4) {
            const float4 t = *reinterpret_cast<const float4*>(table + off);
            v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
          } else if (DPN == 2) {
            const float2 t = *reinterpret_cast<const float2*>(table + off);
            v[0] = t.x; v[1] = t.y;
          } else {
            v[0] = *reinterpret_cast<const float*>(table + off);
          }
#pragma unroll
          for (int j = 0; j < DPN; ++j)
            acc[k * DPN + j] = (r == 0 && !add) ? v[j] : hp_add(v[j], acc[k * DPN + j]);
        }
      }
    }
    if (post_scale != 1.0f) {
#pragma unroll
      for (int k = 0; k < EPG; ++k) acc[k] = hp_mul(acc[k], post_scale);
    }
    const bool clear = APPLY && apply.clear_grad;
    if (out_vec) {
#pragma unroll
      for (int q = 0; q < EPG / 4; ++q)
        reinterpret_cast<float4*>(out + e0)[q] =
            clear ? make_float4(0.f, 0.f, 0.f, 0.f)
                  : make_float4(acc[4 * q], acc[4 * q + 1], acc[4 * q + 2], acc[4 * q + 3]);
    } else {
#pragma unroll
      for (int k = 0; k < EPG; ++k) out[e0 + k] = clear ? 0.f : acc[k];
    }
    if (APPLY) {
      if (apply_vec) {
#pragma unroll
        for (int q = 0; q < EPG / 4; ++q) sgd_update4(apply, e0 + 4 * q, acc + 4 * q);
      } else {
#pragma unroll
        for (int k = 0; k < EPG; ++k) sgd_update(apply, e0 + k, acc[k]);
      }
    }
#pragma unroll
    for (int r = 0; r < kMaxWorld; ++r) w[r] = wn[r];
  }
  // fewer than EPG leftover elements: one thread, element by element
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    constexpr int DPB = 8 / BW;
    for (int64_t e = full_groups * EPG; e < n; ++e) {
      float acc = add ? out[e] : 0.f;
      const int in_byte = int(e % DPB);
#pragma unroll
      for (int r = 0; r < kMaxWorld; ++r) {
        if (r >= src.world) break;
        const uint32_t byte = src.payload[r][data_offset + e / DPB];
        const uint32_t nib = (byte >> (4 * (in_byte / DPN))) & 15u;
        const float v = lut[(size_t(r) * rank_stride + nib) * DPN + in_byte % DPN];
        acc = (r == 0 && !add) ? v : hp_add(v, acc);
      }
      if (post_scale != 1.0f) acc = hp_mul(acc, post_scale);
      out[e] = (APPLY && apply.clear_grad) ? 0.f : acc;
      if (APPLY) sgd_update(apply, e, acc);
    }
  }
}

// ---------------------------------------------------------------- one or two payloads, 2 bits
// With one or two payloads the kernel is bound by the dense traffic (gradient out, parameters
// and momentum in and out), not by the decode, and the mapping above -- a thread owning 64
// contiguous bytes of every dense array -- makes each 16-byte access of a warp touch 32
// different sectors.  Here lane L of a warp handles payload byte j*32 + L (j = 0..3) of the
// warp's 128-byte payload chunk, i.e. elements (j*32 + L)*4 .. +3 of the chunk's 512: every
// dense access is a 512-byte contiguous run across the warp.  The payload is still loaded one
// 32-bit word per lane; bytes reach their lanes by shuffle.
template <bool APPLY, bool SHARED>
__device__ __forceinline__ void unpack_nibble_body_coalesced2(const float* lut, uint32_t (&w)[kMaxWorld],
                                                              const UnpackSources& src, int64_t data_offset,
                                                              float* __restrict__ out, int64_t n, int add,
                                                              float post_scale, const SgdApply& apply) {
  constexpr int rank_stride_bytes = SHARED ? 0 : 16 * 2 * 4;
  const int64_t full_groups = n / 16;            // complete 32-bit payload words
  const int64_t full_chunks = full_groups / 32;  // complete 128-byte warp chunks
  const int lane = threadIdx.x & 31;
  const int64_t warps = int64_t(gridDim.x) * (blockDim.x >> 5);
  const bool clear = APPLY && apply.clear_grad;
  int64_t chunk = int64_t(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  for (; chunk < full_chunks; chunk += warps) {
    const int64_t nxt = (chunk + warps) * 32 + lane;
    uint32_t wn[kMaxWorld];
#pragma unroll
    for (int r = 0; r < kMaxWorld; ++r)
      wn[r] = (r < src.world && chunk + warps < full_chunks) ? load_u32_any(src.payload[r] + data_offset + nxt * 4) : 0u;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t e = chunk * 512 + int64_t(j * 32 + lane) * 4;
      float acc[4];
      if (add) {
        const float4 o = *reinterpret_cast<const float4*>(out + e);
        acc[0] = o.x; acc[1] = o.y; acc[2] = o.z; acc[3] = o.w;
      }
#pragma unroll
      for (int r = 0; r < kMaxWorld; ++r) {
        if (r < src.world) {
          const uint32_t word = __shfl_sync(0xffffffffu, w[r], j * 8 + (lane >> 2));
          const uint32_t byte = (word >> (8 * (lane & 3))) & 255u;
          const char* table = reinterpret_cast<const char*>(lut) + r * rank_stride_bytes;
          const float2 lo = *reinterpret_cast<const float2*>(table + ((byte & 15u) << 3));
          const float2 hi = *reinterpret_cast<const float2*>(table + ((byte >> 4) << 3));
          const float v[4] = {lo.x, lo.y, hi.x, hi.y};
#pragma unroll
          for (int k = 0; k < 4; ++k) acc[k] = (r == 0 && !add) ? v[k] : hp_add(v[k], acc[k]);
        }
      }
      if (post_scale != 1.0f) {
#pragma unroll
        for (int k = 0; k < 4; ++k) acc[k] = hp_mul(acc[k], post_scale);
      }
      *reinterpret_cast<float4*>(out + e) =
          clear ? make_float4(0.f, 0.f, 0.f, 0.f) : make_float4(acc[0], acc[1], acc[2], acc[3]);
      if (APPLY) sgd_update4(apply, e, acc);
    }
#pragma unroll
    for (int r = 0; r < kMaxWorld; ++r) w[r] = wn[r];
  }
  // payload words past the last complete chunk (fewer than 32) and the elements past the last
  // complete word (fewer than 16): block 0, element by element
  if (blockIdx.x == 0) {
    for (int64_t e = full_chunks * 512 + threadIdx.x; e < n; e += blockDim.x) {
      float acc = add ? out[e] : 0.f;
#pragma unroll
      for (int r = 0; r < kMaxWorld; ++r) {
        if (r >= src.world) break;
        const uint32_t byte = src.payload[r][data_offset + (e >> 2)];
        const uint32_t nib = (byte >> (4 * ((e & 3) >> 1))) & 15u;
        const float v = lut[(size_t(SHARED ? 0 : r) * 16 + nib) * 2 + (e & 1)];
        acc = (r == 0 && !add) ? v : hp_add(v, acc);
      }
      if (post_scale != 1.0f) acc = hp_mul(acc, post_scale);
      out[e] = clear ? 0.f : acc;
      if (APPLY) sgd_update(apply, e, acc);
    }
  }
}

// True when unpack_nibble_body_coalesced2 applies: 2-bit payloads of at most two ranks and
// 16-byte aligned dense arrays.
__device__ __forceinline__ bool unpack_coalesced_ok(const UnpackSources& src, const float* out, bool apply_on,
                                                    const SgdApply& apply) {
  uintptr_t bits = reinterpret_cast<uintptr_t>(out);
  if (apply_on) bits |= reinterpret_cast<uintptr_t>(apply.param) | reinterpret_cast<uintptr_t>(apply.momentum);
  return src.world <= 2 && (bits & 15) == 0;
}

}  // namespace cuda
}  // namespace hipress
