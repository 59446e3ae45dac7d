// Residual add + LayerNorm over bf16 rows, forward and backward.
//
//   forward   z = bf16(x + delta);  y = (z - mean) * rstd * gamma + beta         (maths in fp32)
//   backward  g = dy * gamma;  dz = rstd * (g - mean(g) - xhat * mean(g * xhat))  (= dx = ddelta)
//             dgamma = sum_rows dy * xhat,  dbeta = sum_rows dy
//
// In the BERT-large benchmark step (4,096 tokens x 1,024 features per layer) the stock path ran
// the residual stream in fp32 because autocast pins LayerNorm to fp32: a cast, an fp32 add, an
// fp32 LayerNorm, a cast back, and in backward a separate (slow) gamma/beta reduction -- about
// a fifth of the step for tensors of 8 MB.  Here one warp owns a row (16-byte accesses, row
// held in registers, two-pass variance).  Backward is two light kernels: the input gradient row
// by row, and the gamma / beta sums column by column (a thread owns 8 columns and walks a range
// of rows, geometry of nhwc.cuh) finished by a small column-sum kernel in fixed order.  A first
// version did both in one kernel with per-lane gamma / beta accumulators: 196 registers, one
// CTA per SM, 0.34 of the copy bandwidth; it remains as the path for feature counts the column
// geometry does not cover.  The reference has no model code.
#include <cuda_bf16.h>

#include "kernels.h"
#include "nhwc.cuh"

namespace hipress {
namespace cuda {

namespace {

constexpr int kLnThreads = 256;
constexpr int kLnWarps = kLnThreads / 32;

__device__ __forceinline__ void ln_load8(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const float2 f = __bfloat1622float2(h[q]);
    v[2 * q] = f.x;
    v[2 * q + 1] = f.y;
  }
}
__device__ __forceinline__ uint4 ln_pack8(const float (&v)[8]) {
  uint4 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int q = 0; q < 4; ++q) h[q] = __floats2bfloat162_rn(v[2 * q], v[2 * q + 1]);
  return raw;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// CHUNKS: 8-element groups per lane; the row has H <= CHUNKS * 256 features, H % 8 == 0.
template <int CHUNKS, bool ADD>
__global__ void __launch_bounds__(kLnThreads)
add_ln_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ delta,
                  const float* __restrict__ gamma, const float* __restrict__ beta,
                  __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ z_out,
                  float* __restrict__ mean_out, float* __restrict__ rstd_out, int64_t rows, int H, float eps) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float inv_h = 1.0f / float(H);
  for (int64_t r = int64_t(blockIdx.x) * kLnWarps + warp; r < rows; r += int64_t(gridDim.x) * kLnWarps) {
    float z[CHUNKS][8];
    float s = 0.f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int col = (c * 32 + lane) * 8;
      if (col < H) {
        ln_load8(x + r * H + col, z[c]);
        if (ADD) {
          float d[8];
          ln_load8(delta + r * H + col, d);
#pragma unroll
          for (int k = 0; k < 8; ++k) z[c][k] += d[k];
          // the sum is what backward sees: round it to bf16 first, normalise the rounded values
          const uint4 packed = ln_pack8(z[c]);
          *reinterpret_cast<uint4*>(z_out + r * H + col) = packed;
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&packed);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float2 f = __bfloat1622float2(h[q]);
            z[c][2 * q] = f.x;
            z[c][2 * q + 1] = f.y;
          }
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) s += z[c][k];
      }
    }
    const float mean = warp_sum(s) * inv_h;
    float v = 0.f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int col = (c * 32 + lane) * 8;
      if (col < H) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float d = z[c][k] - mean;
          v += d * d;
        }
      }
    }
    const float rstd = rsqrtf(warp_sum(v) * inv_h + eps);
    if (lane == 0) {
      mean_out[r] = mean;
      rstd_out[r] = rstd;
    }
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int col = (c * 32 + lane) * 8;
      if (col < H) {
        const float4 g0 = *reinterpret_cast<const float4*>(gamma + col);
        const float4 g1 = *reinterpret_cast<const float4*>(gamma + col + 4);
        const float4 b0 = *reinterpret_cast<const float4*>(beta + col);
        const float4 b1 = *reinterpret_cast<const float4*>(beta + col + 4);
        const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
        const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
        float o[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = (z[c][k] - mean) * rstd * g[k] + b[k];
        *reinterpret_cast<uint4*>(y + r * H + col) = ln_pack8(o);
      }
    }
  }
}

template <int CHUNKS>
__global__ void __launch_bounds__(kLnThreads)
add_ln_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ z,
                  const float* __restrict__ mean, const float* __restrict__ rstd,
                  const float* __restrict__ gamma, __nv_bfloat16* __restrict__ dz,
                  float* __restrict__ partial /* [gridDim.x][2][H] */, int64_t rows, int H) {
  __shared__ float sh[kLnWarps][2][32 * 8 + 8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float inv_h = 1.0f / float(H);
  float dg[CHUNKS][8], db[CHUNKS][8], gam[CHUNKS][8];
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int col = (c * 32 + lane) * 8;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      dg[c][k] = db[c][k] = 0.f;
      gam[c][k] = col < H ? gamma[col + k] : 0.f;
    }
  }
  for (int64_t r = int64_t(blockIdx.x) * kLnWarps + warp; r < rows; r += int64_t(gridDim.x) * kLnWarps) {
    const float mu = mean[r], rs = rstd[r];
    float g[CHUNKS][8], xh[CHUNKS][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int col = (c * 32 + lane) * 8;
      if (col < H) {
        ln_load8(dy + r * H + col, g[c]);
        ln_load8(z + r * H + col, xh[c]);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          xh[c][k] = (xh[c][k] - mu) * rs;
          db[c][k] += g[c][k];
          dg[c][k] += g[c][k] * xh[c][k];
          g[c][k] *= gam[c][k];
          s1 += g[c][k];
          s2 += g[c][k] * xh[c][k];
        }
      }
    }
    const float c1 = warp_sum(s1) * inv_h, c2 = warp_sum(s2) * inv_h;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int col = (c * 32 + lane) * 8;
      if (col < H) {
        float o[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = rs * (g[c][k] - c1 - xh[c][k] * c2);
        *reinterpret_cast<uint4*>(dz + r * H + col) = ln_pack8(o);
      }
    }
  }
  // per-CTA sums of the gamma / beta gradients, one 256-column chunk at a time
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      sh[warp][0][lane * 8 + k] = dg[c][k];
      sh[warp][1][lane * 8 + k] = db[c][k];
    }
    __syncthreads();
    const int col = c * 256 + threadIdx.x;
    if (col < H) {
      float a = 0.f, b = 0.f;
#pragma unroll
      for (int w = 0; w < kLnWarps; ++w) {
        a += sh[w][0][threadIdx.x];
        b += sh[w][1][threadIdx.x];
      }
      partial[(int64_t(blockIdx.x) * 2 + 0) * H + col] = a;
      partial[(int64_t(blockIdx.x) * 2 + 1) * H + col] = b;
    }
    __syncthreads();
  }
}

// Input gradient only (no gamma / beta accumulators: a third of the registers of the combined
// kernel above, so several CTAs share an SM).  Used together with ln_wgrad_partial_kernel.
template <int CHUNKS>
__global__ void __launch_bounds__(kLnThreads)
add_ln_dz_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ z,
                 const float* __restrict__ mean, const float* __restrict__ rstd,
                 const float* __restrict__ gamma, __nv_bfloat16* __restrict__ dz, int64_t rows, int H) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float inv_h = 1.0f / float(H);
  for (int64_t r = int64_t(blockIdx.x) * kLnWarps + warp; r < rows; r += int64_t(gridDim.x) * kLnWarps) {
    const float mu = mean[r], rs = rstd[r];
    float g[CHUNKS][8], xh[CHUNKS][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int col = (c * 32 + lane) * 8;
      if (col < H) {
        ln_load8(dy + r * H + col, g[c]);
        ln_load8(z + r * H + col, xh[c]);
        const float4 g0 = *reinterpret_cast<const float4*>(gamma + col);
        const float4 g1 = *reinterpret_cast<const float4*>(gamma + col + 4);
        const float gam[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          xh[c][k] = (xh[c][k] - mu) * rs;
          g[c][k] *= gam[k];
          s1 += g[c][k];
          s2 += g[c][k] * xh[c][k];
        }
      }
    }
    const float c1 = warp_sum(s1) * inv_h, c2 = warp_sum(s2) * inv_h;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int col = (c * 32 + lane) * 8;
      if (col < H) {
        float o[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = rs * (g[c][k] - c1 - xh[c][k] * c2);
        *reinterpret_cast<uint4*>(dz + r * H + col) = ln_pack8(o);
      }
    }
  }
}

// Column sums for dgamma (dy * xhat) and dbeta (dy): a thread owns 8 columns and walks a range of
// rows (geometry of nhwc.cuh), per-CTA partials in the layout ln_colsum_kernel reads.
__global__ void __launch_bounds__(kBnThreads)
ln_wgrad_partial_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ z,
                        const float* __restrict__ mean, const float* __restrict__ rstd,
                        float* __restrict__ partial, int64_t rows, int H, int tx_count, int64_t rows_per_block) {
  __shared__ float sh[2 * kBnThreads * kBnVec];
  const Lane l = lane_of(tx_count, rows, rows_per_block);
  float dg[kBnVec], db[kBnVec];
#pragma unroll
  for (int k = 0; k < kBnVec; ++k) dg[k] = db[k] = 0.f;
  int64_t r = l.r_begin + l.ty;
  for (; r + l.TY < l.r_end; r += 2 * l.TY) {
    float g[2][kBnVec], v[2][kBnVec], mu[2], rs[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      load8(dy + (r + u * l.TY) * H + l.c0, g[u]);
      load8(z + (r + u * l.TY) * H + l.c0, v[u]);
      mu[u] = mean[r + u * l.TY];
      rs[u] = rstd[r + u * l.TY];
    }
#pragma unroll
    for (int u = 0; u < 2; ++u)
#pragma unroll
      for (int k = 0; k < kBnVec; ++k) {
        db[k] += g[u][k];
        dg[k] += g[u][k] * (v[u][k] - mu[u]) * rs[u];
      }
  }
  for (; r < l.r_end; r += l.TY) {
    float g[kBnVec], v[kBnVec];
    load8(dy + r * H + l.c0, g);
    load8(z + r * H + l.c0, v);
    const float mu = mean[r], rs = rstd[r];
#pragma unroll
    for (int k = 0; k < kBnVec; ++k) {
      db[k] += g[k];
      dg[k] += g[k] * (v[k] - mu) * rs;
    }
  }
  float DG, DB;
  reduce_rows(dg, db, tx_count, sh, DG, DB);
  const int ct = tx_count * kBnVec;
  if (int(threadIdx.x) < ct) {
    const int col = blockIdx.x * ct + threadIdx.x;
    partial[(int64_t(blockIdx.y) * 2 + 0) * H + col] = DG;
    partial[(int64_t(blockIdx.y) * 2 + 1) * H + col] = DB;
  }
}

constexpr int kLnSumThreads = 1024;
constexpr int kLnSumWarps = kLnSumThreads / 32;

// dgamma[c] / dbeta[c] = sum over CTAs of their partials; grid = (H / 32, 2), lane = column.
__global__ void __launch_bounds__(kLnSumThreads)
ln_colsum_kernel(const float* __restrict__ partial, int blocks, int H, float* __restrict__ dgamma,
                 float* __restrict__ dbeta) {
  __shared__ float sh[kLnSumWarps][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col = blockIdx.x * 32 + lane;
  const int which = blockIdx.y;
  float t = 0.f;
  if (col < H) {
    for (int y0 = warp; y0 < blocks; y0 += kLnSumWarps * 4) {
      float p[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int y = y0 + j * kLnSumWarps;
        p[j] = y < blocks ? __ldcg(&partial[(int64_t(y) * 2 + which) * H + col]) : 0.f;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) t += p[j];
    }
  }
  sh[warp][lane] = t;
  __syncthreads();
  if (warp != 0 || col >= H) return;
  for (int w = 1; w < kLnSumWarps; ++w) t += sh[w][lane];
  (which == 0 ? dgamma : dbeta)[col] = t;
}

int ln_grid(int64_t rows) {
  int64_t blocks = (rows + kLnWarps - 1) / kLnWarps;
  if (blocks > 148 * 2) blocks = 148 * 2;
  return int(blocks < 1 ? 1 : blocks);
}

}  // namespace

bool add_ln_supported(int64_t rows, int hidden) { return rows >= 1 && hidden >= 8 && hidden % 8 == 0 && hidden <= 2048; }

int64_t add_ln_partial_elems(int64_t rows, int hidden) {
  Geom g;
  const int64_t blocks = geometry(rows, hidden, &g) && g.row_blocks > ln_grid(rows) ? g.row_blocks : ln_grid(rows);
  return blocks * 2 * hidden;
}

cudaError_t add_ln_forward(const void* x, const void* delta, const float* gamma, const float* beta, void* y,
                           void* z, float* mean, float* rstd, int64_t rows, int hidden, float eps,
                           cudaStream_t stream) {
  if (!add_ln_supported(rows, hidden) || !x || !gamma || !beta || !y || !mean || !rstd || (delta && !z))
    return cudaErrorInvalidValue;
  const auto* xb = static_cast<const __nv_bfloat16*>(x);
  const auto* db = static_cast<const __nv_bfloat16*>(delta);
  auto* yb = static_cast<__nv_bfloat16*>(y);
  auto* zb = static_cast<__nv_bfloat16*>(z);
  const int grid = ln_grid(rows);
  const int chunks = (hidden + 255) / 256;
#define HP_LN_FWD(C)                                                                                          \
  do {                                                                                                        \
    if (db) add_ln_fwd_kernel<C, true><<<grid, kLnThreads, 0, stream>>>(xb, db, gamma, beta, yb, zb, mean, rstd, rows, hidden, eps); \
    else add_ln_fwd_kernel<C, false><<<grid, kLnThreads, 0, stream>>>(xb, db, gamma, beta, yb, zb, mean, rstd, rows, hidden, eps);   \
  } while (0)
  if (chunks <= 1) HP_LN_FWD(1);
  else if (chunks <= 2) HP_LN_FWD(2);
  else if (chunks <= 4) HP_LN_FWD(4);
  else HP_LN_FWD(8);
#undef HP_LN_FWD
  return cudaGetLastError();
}

cudaError_t add_ln_backward(const void* dy, const void* z, const float* mean, const float* rstd,
                            const float* gamma, void* dz, float* dgamma, float* dbeta, float* partial,
                            int64_t rows, int hidden, cudaStream_t stream) {
  if (!add_ln_supported(rows, hidden) || !dy || !z || !mean || !rstd || !gamma || !dz || !dgamma || !dbeta || !partial)
    return cudaErrorInvalidValue;
  const auto* gb = static_cast<const __nv_bfloat16*>(dy);
  const auto* zb = static_cast<const __nv_bfloat16*>(z);
  auto* ob = static_cast<__nv_bfloat16*>(dz);
  const int chunks = (hidden + 255) / 256;
  Geom g;
  if (geometry(rows, hidden, &g)) {
    // two light kernels: the input gradient row by row, the gamma / beta sums column by column
    int64_t dz_blocks = (rows + kLnWarps - 1) / kLnWarps;
    if (dz_blocks > 148 * 8) dz_blocks = 148 * 8;
    const int dz_grid = int(dz_blocks);
#define HP_LN_DZ(C) add_ln_dz_kernel<C><<<dz_grid, kLnThreads, 0, stream>>>(gb, zb, mean, rstd, gamma, ob, rows, hidden)
    if (chunks <= 1) HP_LN_DZ(1);
    else if (chunks <= 2) HP_LN_DZ(2);
    else if (chunks <= 4) HP_LN_DZ(4);
    else HP_LN_DZ(8);
#undef HP_LN_DZ
    ln_wgrad_partial_kernel<<<dim3(static_cast<unsigned>(g.tiles), static_cast<unsigned>(g.row_blocks), 1), kBnThreads, 0,
                              stream>>>(gb, zb, mean, rstd, partial, rows, hidden, g.tx, g.rows_per_block);
    ln_colsum_kernel<<<dim3(static_cast<unsigned>((hidden + 31) / 32), 2, 1), kLnSumThreads, 0, stream>>>(
        partial, g.row_blocks, hidden, dgamma, dbeta);
    return cudaGetLastError();
  }
  // feature counts the column geometry does not cover: one combined kernel
  const int grid = ln_grid(rows);
#define HP_LN_BWD(C) add_ln_bwd_kernel<C><<<grid, kLnThreads, 0, stream>>>(gb, zb, mean, rstd, gamma, ob, partial, rows, hidden)
  if (chunks <= 1) HP_LN_BWD(1);
  else if (chunks <= 2) HP_LN_BWD(2);
  else if (chunks <= 4) HP_LN_BWD(4);
  else HP_LN_BWD(8);
#undef HP_LN_BWD
  ln_colsum_kernel<<<dim3(static_cast<unsigned>((hidden + 31) / 32), 2, 1), kLnSumThreads, 0, stream>>>(
      partial, grid, hidden, dgamma, dbeta);
  return cudaGetLastError();
}

}  // namespace cuda
}  // namespace hipress
