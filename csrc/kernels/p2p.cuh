// Device-side helpers for kernels that store into peer GPUs' memory and for
// the flag protocol that tells receivers a payload is complete.
#pragma once
#include "kernels.h"

namespace hipress {
namespace cuda {

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Stores of arbitrary alignment: pick the widest store the address allows.
__device__ __forceinline__ void store_u32_any(uint8_t* p, uint32_t v) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(p);
  if ((a & 3) == 0) {
    *reinterpret_cast<uint32_t*>(p) = v;
  } else if ((a & 1) == 0) {
    reinterpret_cast<uint16_t*>(p)[0] = static_cast<uint16_t>(v);
    reinterpret_cast<uint16_t*>(p)[1] = static_cast<uint16_t>(v >> 16);
  } else {
    p[0] = static_cast<uint8_t>(v);
    p[1] = static_cast<uint8_t>(v >> 8);
    p[2] = static_cast<uint8_t>(v >> 16);
    p[3] = static_cast<uint8_t>(v >> 24);
  }
}

// Epoch kept on the device (see PushTargets): fix up the by-value copy of the kernel argument.
// Only scalars are written and every access to the pointer arrays uses a compile-time index
// (unrolled loops with a guard): rewriting the arrays, or indexing them with a run-time value,
// makes the compiler keep the whole struct in local memory, which cost the compress kernels a
// fifth of their bandwidth.  The counter is written by a kernel earlier in stream order.
__device__ __forceinline__ void resolve_epoch(PushTargets& t) {
  if (t.epoch_dev == nullptr) return;
  const uint32_t e = *t.epoch_dev;
  t.epoch = e;
  t.parity_off = (e & 1u) ? t.parity_stride : 0;
}
__device__ __forceinline__ void resolve_epoch(UnpackSources& s) {
  if (s.epoch_dev == nullptr) return;
  s.parity_off = (*s.epoch_dev & 1u) ? s.parity_stride : 0;
}

// NVLS multicast stores: one store, delivered by the NVLink switch to the same offset of every
// GPU bound to the multicast object (this GPU included).  Natural alignment required.
__device__ __forceinline__ void multimem_st_u32(uint8_t* p, uint32_t v) {
  asm volatile("multimem.st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void multimem_st_u128(uint8_t* p, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(__uint_as_float(v.x)),
               "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
               : "memory");
}

// The same 4 payload bytes to every destination.
__device__ __forceinline__ void push_u32(const PushTargets& t, int64_t byte_off, uint32_t v) {
  if (t.mc != nullptr && ((reinterpret_cast<uintptr_t>(t.mc) + t.parity_off + byte_off) & 3) == 0) {
    multimem_st_u32(t.mc + t.parity_off + byte_off, v);
    return;
  }
#pragma unroll
  for (int p = 0; p < kMaxWorld; ++p)
    if (p < t.world) store_u32_any(t.payload[p] + t.parity_off + byte_off, v);
}
__device__ __forceinline__ void push_u8(const PushTargets& t, int64_t byte_off, uint8_t v) {
#pragma unroll
  for (int p = 0; p < kMaxWorld; ++p)
    if (p < t.world) t.payload[p][t.parity_off + byte_off] = v;
}
// 16 payload bytes to every destination; byte_off and the destinations 16-byte aligned
// (push_aligned16).  Peer stores of this width cross NVLink as full 128-byte+ runs per warp
// instead of one 32-byte sector per warp and destination.
__device__ __forceinline__ void push_u128(const PushTargets& t, int64_t byte_off, uint4 v) {
  if (t.mc != nullptr) {   // same alignment as the destinations (push_aligned16 covers it)
    multimem_st_u128(t.mc + t.parity_off + byte_off, v);
    return;
  }
#pragma unroll
  for (int p = 0; p < kMaxWorld; ++p)
    if (p < t.world) *reinterpret_cast<uint4*>(t.payload[p] + t.parity_off + byte_off) = v;
}
// True when payload + data_off is 16-byte aligned in every destination.
__device__ __forceinline__ bool push_aligned16(const PushTargets& t, int64_t data_off) {
  uintptr_t bits = t.mc != nullptr ? reinterpret_cast<uintptr_t>(t.mc + t.parity_off + data_off) : 0;
#pragma unroll
  for (int p = 0; p < kMaxWorld; ++p)
    if (p < t.world) bits |= reinterpret_cast<uintptr_t>(t.payload[p] + t.parity_off + data_off);
  return (bits & 15) == 0;
}
// payload[j] (+ parity offset) for a run-time j: selects over compile-time indices, so that the
// kernel argument stays in parameter space (see resolve_epoch).
__device__ __forceinline__ uint8_t* select_dest(const PushTargets& t, int j) {
  uint8_t* d = t.payload[0];
#pragma unroll
  for (int p = 1; p < kMaxWorld; ++p)
    if (p == j) d = t.payload[p];
  return d + t.parity_off;
}
// True when an earlier kernel of the step recorded a failure (see PushTargets::guard).
__device__ __forceinline__ bool status_guarded(const int* guard) {
  return guard != nullptr && *reinterpret_cast<const volatile int*>(guard) != 0;
}
__device__ __forceinline__ bool push_guarded(const PushTargets& t) { return status_guarded(t.guard); }
// Elements of shard j when n elements are cut into shards of S.
__device__ __forceinline__ int64_t shard_len(int64_t n, int64_t S, int j) {
  const int64_t left = n - int64_t(j) * S;
  return left <= 0 ? 0 : (left < S ? left : S);
}

// Where the bytes of the tensor part being compressed go: every destination (all-gather form)
// or, in scatter mode, the one destination that owns the current shard.
struct PushCursor {
  uint8_t* one;  // scatter mode: payload of the current shard's owner; null otherwise
};
__device__ __forceinline__ void put_u128(const PushTargets& t, const PushCursor& c, int64_t off, uint4 v) {
  if (c.one) *reinterpret_cast<uint4*>(c.one + off) = v;
  else push_u128(t, off, v);
}
__device__ __forceinline__ void put_u32(const PushTargets& t, const PushCursor& c, int64_t off, uint32_t v);
__device__ __forceinline__ void put_u8(const PushTargets& t, const PushCursor& c, int64_t off, uint8_t v);

__device__ __forceinline__ void push_bytes(const PushTargets& t, int64_t byte_off,
                                           const uint8_t* src, int count) {
#pragma unroll
  for (int p = 0; p < kMaxWorld; ++p)
    if (p < t.world)
      for (int i = 0; i < count; ++i) t.payload[p][t.parity_off + byte_off + i] = src[i];
}

__device__ __forceinline__ void put_u32(const PushTargets& t, const PushCursor& c, int64_t off, uint32_t v) {
  if (c.one) store_u32_any(c.one + off, v);
  else push_u32(t, off, v);
}
__device__ __forceinline__ void put_u8(const PushTargets& t, const PushCursor& c, int64_t off, uint8_t v) {
  if (c.one) c.one[off] = v;
  else push_u8(t, off, v);
}
__device__ __forceinline__ void put_bytes(const PushTargets& t, const PushCursor& c, int64_t off,
                                          const uint8_t* src, int count) {
  if (c.one) {
    for (int i = 0; i < count; ++i) c.one[off + i] = src[i];
  } else {
    push_bytes(t, off, src, count);
  }
}

// Called by every thread at the end of a compressing kernel.  Elects the last
// CTA through `done` and lets it publish the epoch flag to every destination.
// Ordering: the CTA barrier orders all of the CTA's payload stores before
// thread 0's fence, and fences are cumulative, so one fence per CTA (not one per
// thread: a system-scope fence is expensive, more so while a host-to-device
// copy is in flight) makes the whole CTA's stores visible before the counter
// is bumped; the last CTA fences again after observing every other CTA's bump
// and only then releases the flags.  With a single local destination the
// consumer is on this GPU and device scope is enough.  The counter is left at
// zero for the next launch.
__device__ __forceinline__ void publish_when_grid_done(const PushTargets& t) {
  if (t.done == nullptr) return;
  __syncthreads();
  if (threadIdx.x == 0) {
    const bool remote = t.world > 1 || t.remote != 0;
    if (remote) __threadfence_system(); else __threadfence();
    const unsigned int total = gridDim.x * gridDim.y * gridDim.z;
    const unsigned int prev = atomicAdd(t.done, 1u);
    if (prev == total - 1) {
      if (remote) __threadfence_system(); else __threadfence();
      *t.done = 0u;
#pragma unroll
      for (int p = 0; p < kMaxWorld; ++p)
        if (p < t.world && t.flag[p] != nullptr) st_release_sys(t.flag[p], t.epoch);
    }
  }
}

// Combine one byte per lane into 32-bit words: lane 4k ends up with the bytes
// of lanes 4k..4k+3 (little-endian).  All 32 lanes must call.
__device__ __forceinline__ uint32_t gather4_bytes(uint32_t b) {
  uint32_t w = b & 0xffu;
  w |= (__shfl_down_sync(0xffffffffu, b, 1) & 0xffu) << 8;
  w |= (__shfl_down_sync(0xffffffffu, b, 2) & 0xffu) << 16;
  w |= (__shfl_down_sync(0xffffffffu, b, 3) & 0xffu) << 24;
  return w;
}
// Same for one 16-bit half-word per lane: lane 2k gets lanes 2k, 2k+1.
__device__ __forceinline__ uint32_t gather2_halves(uint32_t h) {
  return (h & 0xffffu) | ((__shfl_down_sync(0xffffffffu, h, 1) & 0xffffu) << 16);
}

__device__ __forceinline__ void sgd_update(const SgdApply& a, int64_t i, float g) {
  // plain fp32 maths; contraction allowed (not part of any payload)
  float p = a.param[i];
  g = g + a.weight_decay * p;
  float buf = a.first_step ? g : a.mu * a.momentum[i] + g;
  a.momentum[i] = buf;
  a.param[i] = p - a.lr * buf;
}

}  // namespace cuda
}  // namespace hipress
