// Convolution epilogues for channels-last bf16 activations: bias + ReLU, optionally followed by
// 2x2 / stride 2 max pooling, forward and backward.
//
// In the VGG-19 benchmark step the stock kernels spent 8 of 17 ms on this: a broadcasting bias
// add, a ReLU, a pooling kernel with 64-bit indices, an atomic-scatter pooling backward, a ReLU
// backward and a separate reduction for the bias gradient, each a full pass (or several) over
// activations of up to 411 MB.  Max pooling commutes with the monotonic bias + ReLU,
//     maxpool(relu(x + b)) = relu(maxpool(x) + b),
// so a pooled layer needs one read of the convolution output and one write of the quarter-size
// result (plus one index byte per output element); nothing of full size is written.
//
//   forward           y = relu(x + b)                                   1 read, 1 write
//   forward + pool    y = relu(max4(x) + b), idx = arg max (0..3)       1 read, 1/4 write
//   backward          dz = dy * (y > 0),  db = sum dz                   2 reads, 1 write
//   backward + pool   dz[arg max] = dy * (y > 0), 0 elsewhere, db       1/2 read, 1 write
//
// db: per-CTA column sums, then a small finalize kernel (fixed order, deterministic).
// Geometry as in nhwc.cuh.  The reference has no model code.
#include "kernels.h"
#include "nhwc.cuh"

namespace hipress {
namespace cuda {

namespace {

template <bool POOL>
__global__ void __launch_bounds__(kBnThreads)
bias_relu_fwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ bias,
                     __nv_bfloat16* __restrict__ y, uint8_t* __restrict__ idx, int64_t M, int C, int tx_count,
                     int64_t rows_per_block, int Ho, int Wo) {
  const Lane l = lane_of(tx_count, M, rows_per_block);
  float b[kBnVec];
#pragma unroll
  for (int k = 0; k < kBnVec; ++k) b[k] = bias ? bias[l.c0 + k] : 0.f;
  if (!POOL) {
    int64_t r = l.r_begin + l.ty;
    for (; r + 3 * l.TY < l.r_end; r += 4 * l.TY) {
      float v[4][kBnVec];
#pragma unroll
      for (int u = 0; u < 4; ++u) load8(x + (r + u * l.TY) * C + l.c0, v[u]);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
#pragma unroll
        for (int k = 0; k < kBnVec; ++k) v[u][k] = fmaxf(v[u][k] + b[k], 0.f);
        store8(y + (r + u * l.TY) * C + l.c0, v[u]);
      }
    }
    for (; r < l.r_end; r += l.TY) {
      float v[kBnVec];
      load8(x + r * C + l.c0, v);
#pragma unroll
      for (int k = 0; k < kBnVec; ++k) v[k] = fmaxf(v[k] + b[k], 0.f);
      store8(y + r * C + l.c0, v);
    }
  } else {
    const int W = 2 * Wo;
    for (int64_t r = l.r_begin + l.ty; r < l.r_end; r += l.TY) {
      const int wo = int(r % Wo);
      const int64_t q = r / Wo;       // n * Ho + ho
      const int64_t in0 = (2 * q * W + 2 * wo) * int64_t(C) + l.c0;   // row 2*ho of image n: (n*H + 2ho) = 2q
      float v[4][kBnVec];
      load8(x + in0, v[0]);
      load8(x + in0 + C, v[1]);
      load8(x + in0 + int64_t(W) * C, v[2]);
      load8(x + in0 + int64_t(W) * C + C, v[3]);
      float best[kBnVec];
      uint32_t where[kBnVec];
#pragma unroll
      for (int k = 0; k < kBnVec; ++k) {
        best[k] = v[0][k];
        where[k] = 0;
#pragma unroll
        for (int u = 1; u < 4; ++u)
          if (v[u][k] > best[k] || v[u][k] != v[u][k]) {
            best[k] = v[u][k];
            where[k] = u;
          }
        best[k] = fmaxf(best[k] + b[k], 0.f);
      }
      store8(y + r * C + l.c0, best);
      uint2 packed;
      packed.x = where[0] | (where[1] << 8) | (where[2] << 16) | (where[3] << 24);
      packed.y = where[4] | (where[5] << 8) | (where[6] << 16) | (where[7] << 24);
      *reinterpret_cast<uint2*>(idx + r * C + l.c0) = packed;
    }
  }
}

template <bool POOL>
__global__ void __launch_bounds__(kBnThreads)
bias_relu_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ y,
                     const uint8_t* __restrict__ idx, __nv_bfloat16* __restrict__ dz,
                     float* __restrict__ partial, int64_t M, int C, int tx_count, int64_t rows_per_block,
                     int Ho, int Wo) {
  __shared__ float sh[2 * kBnThreads * kBnVec];
  const Lane l = lane_of(tx_count, M, rows_per_block);
  float s[kBnVec], unused[kBnVec];
#pragma unroll
  for (int k = 0; k < kBnVec; ++k) s[k] = unused[k] = 0.f;
  if (!POOL) {
    int64_t r = l.r_begin + l.ty;
    for (; r + 1 * l.TY < l.r_end; r += 2 * l.TY) {
      float g[2][kBnVec], o[2][kBnVec];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        load8(dy + (r + u * l.TY) * C + l.c0, g[u]);
        load8(y + (r + u * l.TY) * C + l.c0, o[u]);
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
#pragma unroll
        for (int k = 0; k < kBnVec; ++k) {
          g[u][k] = o[u][k] > 0.f ? g[u][k] : 0.f;
          s[k] += g[u][k];
        }
        store8(dz + (r + u * l.TY) * C + l.c0, g[u]);
      }
    }
    for (; r < l.r_end; r += l.TY) {
      float g[kBnVec], o[kBnVec];
      load8(dy + r * C + l.c0, g);
      load8(y + r * C + l.c0, o);
#pragma unroll
      for (int k = 0; k < kBnVec; ++k) {
        g[k] = o[k] > 0.f ? g[k] : 0.f;
        s[k] += g[k];
      }
      store8(dz + r * C + l.c0, g);
    }
  } else {
    const int W = 2 * Wo;
    for (int64_t r = l.r_begin + l.ty; r < l.r_end; r += l.TY) {
      const int wo = int(r % Wo);
      const int64_t q = r / Wo;
      const int64_t in0 = (2 * q * W + 2 * wo) * int64_t(C) + l.c0;
      float g[kBnVec], o[kBnVec];
      load8(dy + r * C + l.c0, g);
      load8(y + r * C + l.c0, o);
      const uint2 packed = *reinterpret_cast<const uint2*>(idx + r * C + l.c0);
      uint32_t where[kBnVec];
#pragma unroll
      for (int k = 0; k < kBnVec; ++k) {
        g[k] = o[k] > 0.f ? g[k] : 0.f;
        s[k] += g[k];
        where[k] = ((k < 4 ? packed.x : packed.y) >> (8 * (k & 3))) & 255u;
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        float d[kBnVec];
#pragma unroll
        for (int k = 0; k < kBnVec; ++k) d[k] = where[k] == uint32_t(u) ? g[k] : 0.f;
        store8(dz + in0 + int64_t(u >> 1) * W * C + int64_t(u & 1) * C, d);
      }
    }
  }
  float S, ignored;
  reduce_rows(s, unused, tx_count, sh, S, ignored);
  const int ct = tx_count * kBnVec;
  if (int(threadIdx.x) < ct) partial[int64_t(blockIdx.y) * C + blockIdx.x * ct + threadIdx.x] = S;
}

// Column sums of a [rows][C] bf16 matrix (the bias gradient of a linear layer): per-CTA partial
// sums here, colsum_finalize_kernel after.
__global__ void __launch_bounds__(kBnThreads)
colsum_partial_kernel(const __nv_bfloat16* __restrict__ dy, float* __restrict__ partial, int64_t M, int C,
                      int tx_count, int64_t rows_per_block) {
  __shared__ float sh[2 * kBnThreads * kBnVec];
  const Lane l = lane_of(tx_count, M, rows_per_block);
  float s[kBnVec], unused[kBnVec];
#pragma unroll
  for (int k = 0; k < kBnVec; ++k) s[k] = unused[k] = 0.f;
  int64_t r = l.r_begin + l.ty;
  for (; r + 3 * l.TY < l.r_end; r += 4 * l.TY) {
    float g[4][kBnVec];
#pragma unroll
    for (int u = 0; u < 4; ++u) load8(dy + (r + u * l.TY) * C + l.c0, g[u]);
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int k = 0; k < kBnVec; ++k) s[k] += g[u][k];
  }
  for (; r < l.r_end; r += l.TY) {
    float g[kBnVec];
    load8(dy + r * C + l.c0, g);
#pragma unroll
    for (int k = 0; k < kBnVec; ++k) s[k] += g[k];
  }
  float S, ignored;
  reduce_rows(s, unused, tx_count, sh, S, ignored);
  const int ct = tx_count * kBnVec;
  if (int(threadIdx.x) < ct) partial[int64_t(blockIdx.y) * C + blockIdx.x * ct + threadIdx.x] = S;
}

constexpr int kSumThreads = 1024;
constexpr int kSumWarps = kSumThreads / 32;

// out[c] = sum over row blocks of partial[y][c]; grid = C / 32, lane = channel, warps stride over y.
__global__ void __launch_bounds__(kSumThreads)
colsum_finalize_kernel(const float* __restrict__ partial, int row_blocks, int C, float* __restrict__ out) {
  __shared__ float sh[kSumWarps][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  float t = 0.f;
  if (c < C) {
    for (int y0 = warp; y0 < row_blocks; y0 += kSumWarps * 8) {
      float p[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int y = y0 + j * kSumWarps;
        p[j] = y < row_blocks ? __ldcg(&partial[int64_t(y) * C + c]) : 0.f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) t += p[j];
    }
  }
  sh[warp][lane] = t;
  __syncthreads();
  if (warp != 0 || c >= C) return;
  for (int w = 1; w < kSumWarps; ++w) t += sh[w][lane];
  out[c] = t;
}

}  // namespace

bool bias_relu_supported(int64_t rows, int channels) {
  Geom g;
  return geometry(rows, channels, &g);
}

int64_t bias_relu_partial_elems(int64_t rows, int channels) {
  Geom g;
  if (!geometry(rows, channels, &g)) return 0;
  return int64_t(g.row_blocks) * channels;
}

cudaError_t colsum_bf16(const void* dy, float* out, float* partial, int64_t rows, int channels,
                        cudaStream_t stream) {
  Geom g;
  if (!dy || !out || !partial || !geometry(rows, channels, &g)) return cudaErrorInvalidValue;
  const dim3 grid(static_cast<unsigned>(g.tiles), static_cast<unsigned>(g.row_blocks), 1);
  colsum_partial_kernel<<<grid, kBnThreads, 0, stream>>>(static_cast<const __nv_bfloat16*>(dy), partial, rows,
                                                         channels, g.tx, g.rows_per_block);
  colsum_finalize_kernel<<<(channels + 31) / 32, kSumThreads, 0, stream>>>(partial, g.row_blocks, channels, out);
  return cudaGetLastError();
}

cudaError_t bias_relu_forward(const void* x, const float* bias, void* y, uint8_t* idx, int n, int h, int w,
                              int channels, int pool, cudaStream_t stream) {
  if (!x || !y || n < 1 || h < 1 || w < 1) return cudaErrorInvalidValue;
  if (pool && (!idx || (h & 1) || (w & 1))) return cudaErrorInvalidValue;
  const int ho = pool ? h / 2 : h, wo = pool ? w / 2 : w;
  const int64_t rows = int64_t(n) * ho * wo;
  Geom g;
  if (!geometry(rows, channels, &g)) return cudaErrorInvalidValue;
  const dim3 grid(static_cast<unsigned>(g.tiles), static_cast<unsigned>(g.row_blocks), 1);
  const auto* xb = static_cast<const __nv_bfloat16*>(x);
  auto* yb = static_cast<__nv_bfloat16*>(y);
  if (pool)
    bias_relu_fwd_kernel<true><<<grid, kBnThreads, 0, stream>>>(xb, bias, yb, idx, rows, channels, g.tx,
                                                                g.rows_per_block, ho, wo);
  else
    bias_relu_fwd_kernel<false><<<grid, kBnThreads, 0, stream>>>(xb, bias, yb, idx, rows, channels, g.tx,
                                                                 g.rows_per_block, ho, wo);
  return cudaGetLastError();
}

cudaError_t bias_relu_backward(const void* dy, const void* y, const uint8_t* idx, void* dz, float* dbias,
                               float* partial, int n, int h, int w, int channels, int pool,
                               cudaStream_t stream) {
  if (!dy || !y || !dz || !dbias || !partial || n < 1 || h < 1 || w < 1) return cudaErrorInvalidValue;
  if (pool && (!idx || (h & 1) || (w & 1))) return cudaErrorInvalidValue;
  const int ho = pool ? h / 2 : h, wo = pool ? w / 2 : w;
  const int64_t rows = int64_t(n) * ho * wo;
  Geom g;
  if (!geometry(rows, channels, &g)) return cudaErrorInvalidValue;
  const dim3 grid(static_cast<unsigned>(g.tiles), static_cast<unsigned>(g.row_blocks), 1);
  const auto* gb = static_cast<const __nv_bfloat16*>(dy);
  const auto* yb = static_cast<const __nv_bfloat16*>(y);
  auto* zb = static_cast<__nv_bfloat16*>(dz);
  if (pool)
    bias_relu_bwd_kernel<true><<<grid, kBnThreads, 0, stream>>>(gb, yb, idx, zb, partial, rows, channels, g.tx,
                                                                g.rows_per_block, ho, wo);
  else
    bias_relu_bwd_kernel<false><<<grid, kBnThreads, 0, stream>>>(gb, yb, idx, zb, partial, rows, channels, g.tx,
                                                                 g.rows_per_block, ho, wo);
  colsum_finalize_kernel<<<(channels + 31) / 32, kSumThreads, 0, stream>>>(partial, g.row_blocks, channels, dbias);
  return cudaGetLastError();
}

}  // namespace cuda
}  // namespace hipress
