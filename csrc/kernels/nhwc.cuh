// Shared pieces of the streaming kernels over channels-last bf16 activations (batch norm,
// bias + ReLU): a [rows][channels] view of an NHWC tensor, a CTA owning a tile of up to 256
// channels and a contiguous range of rows, a thread owning 8 adjacent channels (16-byte
// accesses) for the whole kernel.
#pragma once
#include <cuda_bf16.h>

#include "kernels.h"

namespace hipress {
namespace cuda {
namespace {

constexpr int kBnThreads = 256;
constexpr int kBnVec = 8;  // channels per thread

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[kBnVec]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const float2 f = __bfloat1622float2(h[q]);
    v[2 * q] = f.x;
    v[2 * q + 1] = f.y;
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[kBnVec]) {
  uint4 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int q = 0; q < 4; ++q) h[q] = __floats2bfloat162_rn(v[2 * q], v[2 * q + 1]);
  *reinterpret_cast<uint4*>(p) = raw;
}

struct Geom {
  int tx;                  // threads along channels (power of two, <= 32)
  int tiles;               // channel tiles = C / (tx * 8)
  int row_blocks;          // CTAs along rows
  int64_t rows_per_block;
};

// Threads of a CTA: tx = t % g.tx (channel group), ty = t / g.tx (row lane), TY = 256 / g.tx.
struct Lane {
  int tx, ty, TY, c0;
  int64_t r_begin, r_end;
};
__device__ __forceinline__ Lane lane_of(int tx_count, int64_t M, int64_t rows_per_block) {
  Lane l;
  l.tx = threadIdx.x % tx_count;
  l.ty = threadIdx.x / tx_count;
  l.TY = kBnThreads / tx_count;
  l.c0 = (blockIdx.x * tx_count + l.tx) * kBnVec;
  l.r_begin = int64_t(blockIdx.y) * rows_per_block;
  l.r_end = l.r_begin + rows_per_block < M ? l.r_begin + rows_per_block : M;
  return l;
}

// Sums a[0..8) and b[0..8) of every thread over the row lanes of the CTA; on return thread t
// (t < tx_count*8) holds the CTA totals of channel t of the tile in (ra, rb).
__device__ __forceinline__ void reduce_rows(const float (&a)[kBnVec], const float (&b)[kBnVec], int tx_count,
                                            float* sh /* 2 * 256 * 8 floats */, float& ra, float& rb) {
  const int tx = threadIdx.x % tx_count, ty = threadIdx.x / tx_count;
  const int ct = tx_count * kBnVec, TY = kBnThreads / tx_count;
  float* sa = sh;
  float* sb = sh + kBnThreads * kBnVec;
#pragma unroll
  for (int k = 0; k < kBnVec; ++k) {
    sa[ty * ct + tx * kBnVec + k] = a[k];
    sb[ty * ct + tx * kBnVec + k] = b[k];
  }
  __syncthreads();
  ra = 0.f;
  rb = 0.f;
  if (int(threadIdx.x) < ct) {
    for (int y = 0; y < TY; ++y) {
      ra += sa[y * ct + threadIdx.x];
      rb += sb[y * ct + threadIdx.x];
    }
  }
}

// Launch geometry for `M` rows of `C` channels: C/8 must be a power of two up to 32 or a multiple of 32.
inline bool geometry(int64_t M, int C, Geom* g) {
  if (M < 1 || C < kBnVec || C % kBnVec) return false;
  const int groups = C / kBnVec;
  int tx = 1;
  while (tx < 32 && tx < groups) tx <<= 1;
  if (groups % tx) return false;  // C/8 must be a power of two up to 32, or a multiple of 32
  g->tx = tx;
  g->tiles = groups / tx;
  const int ty = kBnThreads / tx;
  // one wave: these kernels hold ~64 registers per thread, so 4 CTAs of 256 threads fit an SM
  int64_t want = (148 * 4 + g->tiles - 1) / g->tiles;
  const int64_t most = (M + int64_t(ty) * 4 - 1) / (int64_t(ty) * 4);  // >= 4 rows per thread
  if (want > most) want = most;
  if (want < 1) want = 1;
  if (want > kBnMaxRowBlocks) want = kBnMaxRowBlocks;
  g->rows_per_block = (M + want - 1) / want;
  g->row_blocks = int((M + g->rows_per_block - 1) / g->rows_per_block);
  return true;
}


}  // namespace
}  // namespace cuda
}  // namespace hipress
