// Training-mode batch normalisation for channels-last bf16 activations, fused with the ReLU
// and the residual add that follow it in a ResNet block.
//
// Why this is here: in the ResNet-50 data-parallel benchmark (64 images per GPU) the framework
// library's channels-last batch-norm kernels took 54 % of the device time of a training step,
// 5-15x off what one pass over the activations costs at HBM speed.  A batch-norm layer is pure
// streaming work:
//
//   forward   stats:  one read of x                      -> per-channel mean / inverse std
//             apply:  y = relu(x*a + b [+ residual])      one read (two with residual), one write
//   backward  reduce: sums of dy' and dy'*(x - mean), dy' = dy * (y > 0)
//             elemt:  dx = dy'*a + x*k2 + k3 [, dres = dy']
//
// Every kernel uses the same geometry: a CTA owns a tile of up to 256 channels and a contiguous
// range of rows (row = one pixel of one image, C contiguous bf16 values).  A thread owns 8
// adjacent channels (one 16-byte load per row) for the whole kernel, so per-channel constants
// sit in registers, and four rows are in flight per thread.  The two reductions store one
// partial result per CTA and channel; a small finalize kernel (32 channels per CTA, eight warps
// striding over the partials, merged in a fixed order, so results are deterministic) combines
// them -- the variance with Chan's parallel update, so no precision is lost to
// E[x^2] - E[x]^2 over the whole batch -- and writes the coefficients the elementwise kernel
// needs.  (A first version let the last CTA to finish combine all partials: one thread per
// channel walking ~1,200 partials in sequence took 6x longer than reading the activations.)
//
// The reference has no model code; this belongs to the model zoo built around its codecs.
#include <cuda_bf16.h>

#include "kernels.h"
#include "nhwc.cuh"

namespace hipress {
namespace cuda {

namespace {

// ---------------------------------------------------------------- forward: statistics
__global__ void __launch_bounds__(kBnThreads)
bn_stats_kernel(const __nv_bfloat16* __restrict__ x, int64_t M, int C, int tx_count, int64_t rows_per_block,
                float2* __restrict__ partial) {
  __shared__ float sh[2 * kBnThreads * kBnVec];
  const Lane l = lane_of(tx_count, M, rows_per_block);
  float s[kBnVec], q[kBnVec];
#pragma unroll
  for (int k = 0; k < kBnVec; ++k) s[k] = q[k] = 0.f;
  const __nv_bfloat16* base = x + l.c0;
  int64_t r = l.r_begin + l.ty;
  for (; r + 3 * l.TY < l.r_end; r += 4 * l.TY) {
    float v[4][kBnVec];
#pragma unroll
    for (int u = 0; u < 4; ++u) load8(base + (r + u * l.TY) * C, v[u]);
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int k = 0; k < kBnVec; ++k) {
        s[k] += v[u][k];
        q[k] += v[u][k] * v[u][k];
      }
  }
  for (; r < l.r_end; r += l.TY) {
    float v[kBnVec];
    load8(base + r * C, v);
#pragma unroll
    for (int k = 0; k < kBnVec; ++k) {
      s[k] += v[k];
      q[k] += v[k] * v[k];
    }
  }
  float S, Q;
  reduce_rows(s, q, tx_count, sh, S, Q);
  const int ct = tx_count * kBnVec;
  const int c = blockIdx.x * ct + threadIdx.x;
  if (int(threadIdx.x) < ct) {
    const float cnt = float(l.r_end - l.r_begin);
    const float mean_b = cnt > 0.f ? S / cnt : 0.f;
    partial[int64_t(blockIdx.y) * C + c] = make_float2(mean_b, fmaxf(Q - S * mean_b, 0.f));
  }
}

constexpr int kFinChannels = 32;  // channels per finalize CTA (one per lane)
constexpr int kFinThreads = 1024;
constexpr int kFinWarps = kFinThreads / 32;
constexpr int kFinBatch = 10;     // partials requested together: their load latencies overlap

// Chan et al.: merge (count, mean, M2) of two disjoint sets.
__device__ __forceinline__ void chan_merge(float& cnt, float& mean, float& m2, float nb, float mb, float m2b) {
  if (nb <= 0.f) return;
  const float tot = cnt + nb;
  const float delta = mb - mean;
  const float frac = __fdividef(nb, tot);  // weights of a mean: 2 ulp is plenty, an IEEE divide per step is not free
  mean += delta * frac;
  m2 += m2b + delta * delta * (cnt * frac);
  cnt = tot;
}

// grid = C / 32.  Lane = channel, warp w merges row blocks w, w+32, ... and the warp results are
// merged in warp order.  The walk over the partials is a chain of dependent updates fed by
// loads that miss L1; with one load per step it is pure latency (measured: 30 us per layer),
// so the loads of a few steps are issued together.
__global__ void __launch_bounds__(kFinThreads)
bn_stats_finalize_kernel(const float2* __restrict__ partial, int row_blocks, int64_t M, int C,
                         int64_t rows_per_block, const float* __restrict__ gamma,
                         const float* __restrict__ beta, float* running_mean, float* running_var,
                         long long* num_batches, float momentum, float eps, float* __restrict__ mean_out,
                         float* __restrict__ invstd_out, float2* __restrict__ ab_out) {
  __shared__ float sh[3][kFinWarps][kFinChannels];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = blockIdx.x * kFinChannels + lane;
  float cnt = 0.f, mean = 0.f, m2 = 0.f;
  // per-channel scalars of the epilogue, requested now so that they arrive during the merge
  float w_c = 1.f, b_c = 0.f, rm_c = 0.f, rv_c = 0.f;
  if (warp == 0 && c < C) {
    if (gamma) w_c = gamma[c];
    if (beta) b_c = beta[c];
    if (running_mean) {
      rm_c = running_mean[c];
      rv_c = running_var[c];
    }
  }
  if (c < C) {
    for (int y0 = warp; y0 < row_blocks; y0 += kFinWarps * kFinBatch) {
      float2 p[kFinBatch];
#pragma unroll
      for (int j = 0; j < kFinBatch; ++j) {
        const int y = y0 + j * kFinWarps;
        p[j] = y < row_blocks ? __ldcg(&partial[int64_t(y) * C + c]) : make_float2(0.f, 0.f);
      }
#pragma unroll
      for (int j = 0; j < kFinBatch; ++j) {
        const int y = y0 + j * kFinWarps;
        if (y >= row_blocks) break;
        const int64_t b0 = int64_t(y) * rows_per_block;
        const int64_t b1 = b0 + rows_per_block < M ? b0 + rows_per_block : M;
        chan_merge(cnt, mean, m2, float(b1 - b0), p[j].x, p[j].y);
      }
    }
  }
  sh[0][warp][lane] = cnt;
  sh[1][warp][lane] = mean;
  sh[2][warp][lane] = m2;
  __syncthreads();
  if (warp != 0 || c >= C) return;
  for (int w = 1; w < kFinWarps; ++w) chan_merge(cnt, mean, m2, sh[0][w][lane], sh[1][w][lane], sh[2][w][lane]);
  const float var = m2 / cnt;
  const float invstd = rsqrtf(var + eps);
  mean_out[c] = mean;
  invstd_out[c] = invstd;
  const float a = w_c * invstd;
  ab_out[c] = make_float2(a, b_c - mean * a);
  if (running_mean) {
    running_mean[c] = (1.f - momentum) * rm_c + momentum * mean;
    running_var[c] = (1.f - momentum) * rv_c + momentum * (cnt > 1.f ? m2 / (cnt - 1.f) : var);
  }
  if (num_batches && c == 0) *num_batches += 1;
}

// ---------------------------------------------------------------- forward: apply
template <bool RELU, bool ADD>
__global__ void __launch_bounds__(kBnThreads)
bn_apply_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                __nv_bfloat16* __restrict__ y, int64_t M, int C, int tx_count, int64_t rows_per_block,
                const float2* __restrict__ ab) {
  const Lane l = lane_of(tx_count, M, rows_per_block);
  float a[kBnVec], b[kBnVec];
#pragma unroll
  for (int k = 0; k < kBnVec; ++k) {
    const float2 t = ab[l.c0 + k];
    a[k] = t.x;
    b[k] = t.y;
  }
  int64_t r = l.r_begin + l.ty;
  for (; r + 3 * l.TY < l.r_end; r += 4 * l.TY) {
    float v[4][kBnVec], w[4][kBnVec];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      load8(x + (r + u * l.TY) * C + l.c0, v[u]);
      if (ADD) load8(res + (r + u * l.TY) * C + l.c0, w[u]);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
#pragma unroll
      for (int k = 0; k < kBnVec; ++k) {
        float o = fmaf(v[u][k], a[k], b[k]);
        if (ADD) o += w[u][k];
        v[u][k] = RELU ? fmaxf(o, 0.f) : o;
      }
      store8(y + (r + u * l.TY) * C + l.c0, v[u]);
    }
  }
  for (; r < l.r_end; r += l.TY) {
    float v[kBnVec], w[kBnVec];
    load8(x + r * C + l.c0, v);
    if (ADD) load8(res + r * C + l.c0, w);
#pragma unroll
    for (int k = 0; k < kBnVec; ++k) {
      float o = fmaf(v[k], a[k], b[k]);
      if (ADD) o += w[k];
      v[k] = RELU ? fmaxf(o, 0.f) : o;
    }
    store8(y + r * C + l.c0, v);
  }
}

// ---------------------------------------------------------------- backward: reductions
template <bool RELU>
__global__ void __launch_bounds__(kBnThreads)
bn_bwd_reduce_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                     const __nv_bfloat16* __restrict__ y, int64_t M, int C, int tx_count,
                     int64_t rows_per_block, const float* __restrict__ mean, float2* __restrict__ partial) {
  __shared__ float sh[2 * kBnThreads * kBnVec];
  const Lane l = lane_of(tx_count, M, rows_per_block);
  float mu[kBnVec], s1[kBnVec], s2[kBnVec];
#pragma unroll
  for (int k = 0; k < kBnVec; ++k) {
    mu[k] = mean[l.c0 + k];
    s1[k] = s2[k] = 0.f;
  }
  int64_t r = l.r_begin + l.ty;
  for (; r + 1 * l.TY < l.r_end; r += 2 * l.TY) {
    float g[2][kBnVec], v[2][kBnVec], o[2][kBnVec];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      load8(dy + (r + u * l.TY) * C + l.c0, g[u]);
      load8(x + (r + u * l.TY) * C + l.c0, v[u]);
      if (RELU) load8(y + (r + u * l.TY) * C + l.c0, o[u]);
    }
#pragma unroll
    for (int u = 0; u < 2; ++u)
#pragma unroll
      for (int k = 0; k < kBnVec; ++k) {
        const float d = (!RELU || o[u][k] > 0.f) ? g[u][k] : 0.f;
        s1[k] += d;
        s2[k] += d * (v[u][k] - mu[k]);
      }
  }
  for (; r < l.r_end; r += l.TY) {
    float g[kBnVec], v[kBnVec], o[kBnVec];
    load8(dy + r * C + l.c0, g);
    load8(x + r * C + l.c0, v);
    if (RELU) load8(y + r * C + l.c0, o);
#pragma unroll
    for (int k = 0; k < kBnVec; ++k) {
      const float d = (!RELU || o[k] > 0.f) ? g[k] : 0.f;
      s1[k] += d;
      s2[k] += d * (v[k] - mu[k]);
    }
  }
  float S1, S2;
  reduce_rows(s1, s2, tx_count, sh, S1, S2);
  const int ct = tx_count * kBnVec;
  const int c = blockIdx.x * ct + threadIdx.x;
  if (int(threadIdx.x) < ct) partial[int64_t(blockIdx.y) * C + c] = make_float2(S1, S2);
}

// grid = C / 32; same layout as bn_stats_finalize_kernel, plain sums.
__global__ void __launch_bounds__(kFinThreads)
bn_bwd_finalize_kernel(const float2* __restrict__ partial, int row_blocks, int64_t M, int C,
                       const float* __restrict__ mean, const float* __restrict__ invstd,
                       const float* __restrict__ gamma, float* __restrict__ dgamma,
                       float* __restrict__ dbeta, float4* __restrict__ coef) {
  __shared__ float sh[2][kFinWarps][kFinChannels];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = blockIdx.x * kFinChannels + lane;
  float t1 = 0.f, t2 = 0.f;
  float is = 0.f, m = 0.f, wgt = 1.f;  // requested now, used after the merge
  if (warp == 0 && c < C) {
    is = invstd[c];
    m = mean[c];
    if (gamma) wgt = gamma[c];
  }
  if (c < C) {
    for (int y0 = warp; y0 < row_blocks; y0 += kFinWarps * kFinBatch) {
      float2 p[kFinBatch];
#pragma unroll
      for (int j = 0; j < kFinBatch; ++j) {
        const int y = y0 + j * kFinWarps;
        p[j] = y < row_blocks ? __ldcg(&partial[int64_t(y) * C + c]) : make_float2(0.f, 0.f);
      }
#pragma unroll
      for (int j = 0; j < kFinBatch; ++j) {
        t1 += p[j].x;
        t2 += p[j].y;
      }
    }
  }
  sh[0][warp][lane] = t1;
  sh[1][warp][lane] = t2;
  __syncthreads();
  if (warp != 0 || c >= C) return;
  for (int w = 1; w < kFinWarps; ++w) {
    t1 += sh[0][w][lane];
    t2 += sh[1][w][lane];
  }
  if (dbeta) dbeta[c] = t1;
  if (dgamma) dgamma[c] = t2 * is;
  // dx = a*(dy' - mean(dy') - xhat*mean(dy'*xhat)),  xhat = (x - m)*is,  a = w*is
  const float a = wgt * is;
  const float inv_count = 1.f / float(M);
  const float k2 = -a * is * is * t2 * inv_count;
  const float k3 = -a * t1 * inv_count - m * k2;
  coef[c] = make_float4(a, k2, k3, 0.f);
}

// ---------------------------------------------------------------- backward: elementwise
template <bool RELU, bool ADD>
__global__ void __launch_bounds__(kBnThreads)
bn_bwd_elemt_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                    const __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ dx,
                    __nv_bfloat16* __restrict__ dres, int64_t M, int C, int tx_count,
                    int64_t rows_per_block, const float4* __restrict__ coef) {
  const Lane l = lane_of(tx_count, M, rows_per_block);
  float a[kBnVec], k2[kBnVec], k3[kBnVec];
#pragma unroll
  for (int k = 0; k < kBnVec; ++k) {
    const float4 t = coef[l.c0 + k];
    a[k] = t.x;
    k2[k] = t.y;
    k3[k] = t.z;
  }
  int64_t r = l.r_begin + l.ty;
  for (; r + 1 * l.TY < l.r_end; r += 2 * l.TY) {
    float g[2][kBnVec], v[2][kBnVec], o[2][kBnVec];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      load8(dy + (r + u * l.TY) * C + l.c0, g[u]);
      load8(x + (r + u * l.TY) * C + l.c0, v[u]);
      if (RELU) load8(y + (r + u * l.TY) * C + l.c0, o[u]);
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
#pragma unroll
      for (int k = 0; k < kBnVec; ++k) {
        const float d = (!RELU || o[u][k] > 0.f) ? g[u][k] : 0.f;
        g[u][k] = d;
        v[u][k] = fmaf(d, a[k], fmaf(v[u][k], k2[k], k3[k]));
      }
      store8(dx + (r + u * l.TY) * C + l.c0, v[u]);
      if (ADD) store8(dres + (r + u * l.TY) * C + l.c0, g[u]);
    }
  }
  for (; r < l.r_end; r += l.TY) {
    float g[kBnVec], v[kBnVec], o[kBnVec];
    load8(dy + r * C + l.c0, g);
    load8(x + r * C + l.c0, v);
    if (RELU) load8(y + r * C + l.c0, o);
#pragma unroll
    for (int k = 0; k < kBnVec; ++k) {
      const float d = (!RELU || o[k] > 0.f) ? g[k] : 0.f;
      g[k] = d;
      v[k] = fmaf(d, a[k], fmaf(v[k], k2[k], k3[k]));
    }
    store8(dx + r * C + l.c0, v);
    if (ADD) store8(dres + r * C + l.c0, g);
  }
}

}  // namespace

bool bn_supported(int64_t rows, int channels) {
  Geom g;
  return geometry(rows, channels, &g);
}

int64_t bn_partial_elems(int64_t rows, int channels) {
  Geom g;
  if (!geometry(rows, channels, &g)) return 0;
  return int64_t(g.row_blocks) * channels;
}

cudaError_t bn_forward(const void* x, const void* residual, void* y, int64_t rows, int channels,
                       const float* gamma, const float* beta, float* running_mean, float* running_var,
                       long long* num_batches, float momentum, float eps, int relu, float* mean,
                       float* invstd, float* ab, float* partial, cudaStream_t stream) {
  Geom g;
  if (!geometry(rows, channels, &g) || !x || !y || !mean || !invstd || !ab || !partial)
    return cudaErrorInvalidValue;
  const dim3 grid(static_cast<unsigned>(g.tiles), static_cast<unsigned>(g.row_blocks), 1);
  const int fin_grid = (channels + kFinChannels - 1) / kFinChannels;
  const auto* xb = static_cast<const __nv_bfloat16*>(x);
  const auto* rb = static_cast<const __nv_bfloat16*>(residual);
  auto* yb = static_cast<__nv_bfloat16*>(y);
  auto* part = reinterpret_cast<float2*>(partial);
  bn_stats_kernel<<<grid, kBnThreads, 0, stream>>>(xb, rows, channels, g.tx, g.rows_per_block, part);
  bn_stats_finalize_kernel<<<fin_grid, kFinThreads, 0, stream>>>(part, g.row_blocks, rows, channels, g.rows_per_block,
                                                                gamma, beta, running_mean, running_var, num_batches,
                                                                momentum, eps, mean, invstd,
                                                                reinterpret_cast<float2*>(ab));
  const float2* abp = reinterpret_cast<const float2*>(ab);
#define HP_BN_APPLY(R, A) \
  bn_apply_kernel<R, A><<<grid, kBnThreads, 0, stream>>>(xb, rb, yb, rows, channels, g.tx, g.rows_per_block, abp)
  if (relu && rb) HP_BN_APPLY(true, true);
  else if (relu) HP_BN_APPLY(true, false);
  else if (rb) HP_BN_APPLY(false, true);
  else HP_BN_APPLY(false, false);
#undef HP_BN_APPLY
  return cudaGetLastError();
}

cudaError_t bn_backward(const void* dy, const void* x, const void* y, void* dx, void* dres, int64_t rows,
                        int channels, const float* gamma, const float* mean, const float* invstd,
                        int relu, float* dgamma, float* dbeta, float* coef, float* partial,
                        cudaStream_t stream) {
  Geom g;
  if (!geometry(rows, channels, &g) || !dy || !x || !dx || !mean || !invstd || !coef || !partial ||
      (relu && !y))
    return cudaErrorInvalidValue;
  const dim3 grid(static_cast<unsigned>(g.tiles), static_cast<unsigned>(g.row_blocks), 1);
  const int fin_grid = (channels + kFinChannels - 1) / kFinChannels;
  const auto* gb = static_cast<const __nv_bfloat16*>(dy);
  const auto* xb = static_cast<const __nv_bfloat16*>(x);
  const auto* yb = static_cast<const __nv_bfloat16*>(y);
  auto* dxb = static_cast<__nv_bfloat16*>(dx);
  auto* drb = static_cast<__nv_bfloat16*>(dres);
  auto* part = reinterpret_cast<float2*>(partial);
  auto* cf = reinterpret_cast<float4*>(coef);
  if (relu)
    bn_bwd_reduce_kernel<true><<<grid, kBnThreads, 0, stream>>>(gb, xb, yb, rows, channels, g.tx, g.rows_per_block,
                                                                mean, part);
  else
    bn_bwd_reduce_kernel<false><<<grid, kBnThreads, 0, stream>>>(gb, xb, yb, rows, channels, g.tx, g.rows_per_block,
                                                                 mean, part);
  bn_bwd_finalize_kernel<<<fin_grid, kFinThreads, 0, stream>>>(part, g.row_blocks, rows, channels, mean, invstd, gamma,
                                                              dgamma, dbeta, cf);
#define HP_BN_ELEMT(R, A) \
  bn_bwd_elemt_kernel<R, A><<<grid, kBnThreads, 0, stream>>>(gb, xb, yb, dxb, drb, rows, channels, g.tx, g.rows_per_block, cf)
  if (relu && drb) HP_BN_ELEMT(true, true);
  else if (relu) HP_BN_ELEMT(true, false);
  else if (drb) HP_BN_ELEMT(false, true);
  else HP_BN_ELEMT(false, false);
#undef HP_BN_ELEMT
  return cudaGetLastError();
}

}  // namespace cuda
}  // namespace hipress
