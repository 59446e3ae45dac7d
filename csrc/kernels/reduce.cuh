// Grid-wide min/max (and abs-max) reduction without a host round-trip.
//
// Each CTA reduces its grid-stride share and writes one partial pair; the last
// CTA to finish (elected through a counter) folds the partials and calls a
// finaliser that turns the extremes into header bytes and scale factors on the
// device.  The reference does this with thrust::minmax_element, two 4-byte
// device-to-host copies and a stream synchronise per batch
// (terngrad_body.h:186-195).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace hipress {
namespace cuda {

constexpr int kReduceMaxBlocks = 1024;

struct MinMaxScratch {
  unsigned int counter;  // zero between launches
  unsigned int pad;
  float mn, mx;    // result
  float inv, gap;  // compress-side scale and decode-side step
  float partial_min[kReduceMaxBlocks];
  float partial_max[kReduceMaxBlocks];
};

__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide reduction of (mn, mx); result valid in thread 0.
template <int THREADS>
__device__ __forceinline__ void block_minmax(float& mn, float& mx) {
  __shared__ float smin[THREADS / 32];
  __shared__ float smax[THREADS / 32];
  mn = warp_min(mn);
  mx = warp_max(mx);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    smin[warp] = mn;
    smax[warp] = mx;
  }
  __syncthreads();
  if (warp == 0) {
    mn = lane < THREADS / 32 ? smin[lane] : smin[0];
    mx = lane < THREADS / 32 ? smax[lane] : smax[0];
    mn = warp_min(mn);
    mx = warp_max(mx);
  }
  __syncthreads();
}

// Returns true in every thread of exactly one CTA: the last to arrive.  Before
// returning true the partials of all CTAs are visible to the caller.
template <int THREADS>
__device__ __forceinline__ bool grid_minmax_last_block(MinMaxScratch* s, float mn, float mx,
                                                       float& out_mn, float& out_mx) {
  __shared__ bool is_last;
  block_minmax<THREADS>(mn, mx);
  if (threadIdx.x == 0) {
    s->partial_min[blockIdx.x] = mn;
    s->partial_max[blockIdx.x] = mx;
    __threadfence();
    const unsigned int prev = atomicAdd(&s->counter, 1u);
    is_last = (prev == gridDim.x - 1);
  }
  __syncthreads();
  if (!is_last) return false;
  __threadfence();
  float a = INFINITY, b = -INFINITY;
  for (int i = threadIdx.x; i < int(gridDim.x); i += THREADS) {
    a = fminf(a, reinterpret_cast<volatile float*>(s->partial_min)[i]);
    b = fmaxf(b, reinterpret_cast<volatile float*>(s->partial_max)[i]);
  }
  block_minmax<THREADS>(a, b);
  __shared__ float res[2];
  if (threadIdx.x == 0) {
    res[0] = a;
    res[1] = b;
    s->counter = 0u;
  }
  __syncthreads();
  out_mn = res[0];
  out_mx = res[1];
  return true;
}

}  // namespace cuda
}  // namespace hipress
