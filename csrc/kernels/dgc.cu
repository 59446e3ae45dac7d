// Deep-gradient-compression pre/post-processing and the fused AdamW update.
//
// DGC (Lin et al.) wraps a top-k sparsifier with three things the reference
// does not contain (its dgc_body.h is only the selector):
//   * momentum correction   u = m*u + g ;  v = v + u ;  send sparse(v)
//   * momentum factor masking: u and v are cleared at the sent positions
//   * local gradient clipping: g is scaled by min(1, clip / |g|) per bucket
//     before it enters u (clip already divided by sqrt(world) by the caller)
// The selector itself is sparse_compress (sparse.cu) run on v.
#include "kernels.h"
#include "p2p.cuh"

namespace hipress {
namespace cuda {

namespace {

constexpr int kThreads = 256;

inline int grid_for(int64_t items, int max_blocks) {
  int64_t blocks = (items + kThreads - 1) / kThreads;
  if (blocks < 1) blocks = 1;
  if (blocks > max_blocks) blocks = max_blocks;
  return int(blocks);
}

__global__ void __launch_bounds__(kThreads)
sumsq_kernel(const float* __restrict__ g, int64_t n, float* __restrict__ out) {
  __shared__ float sh[kThreads / 32];
  float acc = 0.f;
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  const int64_t tid = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t nv = (reinterpret_cast<uintptr_t>(g) & 15) == 0 ? (n >> 2) : 0;  // 16-byte loads when aligned
  for (int64_t i = tid; i < nv; i += stride) {
    const float4 a = reinterpret_cast<const float4*>(g)[i];
    acc += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
  }
  for (int64_t i = (nv << 2) + tid; i < n; i += stride) acc += g[i] * g[i];
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    acc = threadIdx.x < kThreads / 32 ? sh[threadIdx.x] : 0.f;
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (threadIdx.x == 0) atomicAdd(out, acc);
  }
}

// u = m*u + s*g ; v += u, with s = min(1, clip/|g|) when clip > 0.
__global__ void __launch_bounds__(kThreads)
dgc_accumulate_kernel(const float* __restrict__ g, float* __restrict__ u, float* __restrict__ v,
                      int64_t n, float momentum, float clip, const float* __restrict__ sumsq) {
  float s = 1.0f;
  if (clip > 0.f) {
    const float norm = sqrtf(*sumsq);
    s = fminf(1.0f, clip / (norm + 1e-6f));
  }
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  const int64_t tid = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  const bool vec = ((reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(u) |
                     reinterpret_cast<uintptr_t>(v)) & 15) == 0;
  const int64_t nv = vec ? (n >> 2) : 0;
  for (int64_t i = tid; i < nv; i += stride) {
    const float4 g4 = reinterpret_cast<const float4*>(g)[i];
    float4 u4 = reinterpret_cast<float4*>(u)[i];
    float4 v4 = reinterpret_cast<float4*>(v)[i];
    u4.x = momentum * u4.x + s * g4.x;
    u4.y = momentum * u4.y + s * g4.y;
    u4.z = momentum * u4.z + s * g4.z;
    u4.w = momentum * u4.w + s * g4.w;
    v4.x += u4.x;
    v4.y += u4.y;
    v4.z += u4.z;
    v4.w += u4.w;
    reinterpret_cast<float4*>(u)[i] = u4;
    reinterpret_cast<float4*>(v)[i] = v4;
  }
  for (int64_t i = (nv << 2) + tid; i < n; i += stride) {
    const float uu = momentum * u[i] + s * g[i];
    u[i] = uu;
    v[i] += uu;
  }
}

// u[idx] = 0 for every index of a sparse payload; also clears the clip scratch.
__global__ void __launch_bounds__(kThreads)
dgc_mask_kernel(const uint8_t* __restrict__ payload, int64_t cap, float* __restrict__ u, int64_t n,
                float* __restrict__ sumsq, const uint32_t* epoch_dev, int64_t parity_stride) {
  if (epoch_dev != nullptr && (*epoch_dev & 1u)) payload += parity_stride;  // see PushTargets
  uint32_t total = 0;
  for (int k = 0; k < 4; ++k) total |= uint32_t(payload[k]) << (8 * k);
  if (blockIdx.x == 0 && threadIdx.x == 0 && sumsq != nullptr) *sumsq = 0.f;
  if (total < 4 || int64_t(total) > cap) return;
  const int64_t k = (int64_t(total) - 4) / 8;
  const uint32_t* idx = reinterpret_cast<const uint32_t*>(payload + 4);
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t x = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; x < k; x += stride) {
    const uint32_t i = idx[x];
    if (int64_t(i) < n) u[i] = 0.f;
  }
}

__device__ __forceinline__ void adamw_one(const AdamWApply& a, float bc1, float rsqrt_bc2, float g,
                                          float& p, float& m, float& v) {
  p -= a.lr * a.weight_decay * p;  // decoupled weight decay
  m = a.beta1 * m + (1.0f - a.beta1) * g;
  v = a.beta2 * v + (1.0f - a.beta2) * g * g;
  const float denom = sqrtf(v) * rsqrt_bc2 + a.eps;
  p -= (a.lr / bc1) * (m / denom);
}

// VEC: all four arrays 16-byte aligned; four elements per thread and iteration.
template <bool VEC>
__global__ void __launch_bounds__(kThreads)
adamw_kernel(float* __restrict__ grad, float scale, AdamWApply a, int64_t n) {
  // an earlier kernel of the step recorded a failure: leave parameters and moments untouched
  if (a.guard != nullptr && *reinterpret_cast<const volatile int*>(a.guard) != 0) return;
  const float step = float(a.step_dev != nullptr ? int(*a.step_dev) : a.step);
  const float bc1 = 1.0f - powf(a.beta1, step);
  const float rsqrt_bc2 = 1.0f / sqrtf(1.0f - powf(a.beta2, step));
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  const int64_t tid = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t nv = VEC ? (n >> 2) : 0;
  for (int64_t i = tid; i < nv; i += stride) {
    const float4 g4 = reinterpret_cast<const float4*>(grad)[i];
    const float4 p4 = reinterpret_cast<const float4*>(a.param)[i];
    const float4 m4 = reinterpret_cast<const float4*>(a.exp_avg)[i];
    const float4 v4 = reinterpret_cast<const float4*>(a.exp_avg_sq)[i];
    float g[4] = {g4.x, g4.y, g4.z, g4.w}, p[4] = {p4.x, p4.y, p4.z, p4.w};
    float m[4] = {m4.x, m4.y, m4.z, m4.w}, v[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) adamw_one(a, bc1, rsqrt_bc2, g[k] * scale, p[k], m[k], v[k]);
    reinterpret_cast<float4*>(a.exp_avg)[i] = make_float4(m[0], m[1], m[2], m[3]);
    reinterpret_cast<float4*>(a.exp_avg_sq)[i] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4*>(a.param)[i] = make_float4(p[0], p[1], p[2], p[3]);
    if (a.clear_grad) reinterpret_cast<float4*>(grad)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  for (int64_t i = (nv << 2) + tid; i < n; i += stride) {
    float p = a.param[i], m = a.exp_avg[i], v = a.exp_avg_sq[i];
    adamw_one(a, bc1, rsqrt_bc2, grad[i] * scale, p, m, v);
    a.exp_avg[i] = m;
    a.exp_avg_sq[i] = v;
    a.param[i] = p;
    if (a.clear_grad) grad[i] = 0.f;
  }
}

}  // namespace

cudaError_t dgc_sumsq(const float* g, int64_t n, float* out, cudaStream_t stream) {
  if (n <= 0 || g == nullptr || out == nullptr) return cudaErrorInvalidValue;
  sumsq_kernel<<<grid_for(n, 148 * 4), kThreads, 0, stream>>>(g, n, out);
  return cudaGetLastError();
}

cudaError_t dgc_accumulate(const float* grad, float* u, float* v, int64_t n, float momentum,
                           float clip, float* sumsq_scratch, cudaStream_t stream) {
  if (n <= 0) return cudaErrorInvalidValue;
  if (clip > 0.f) {
    if (sumsq_scratch == nullptr) return cudaErrorInvalidValue;
    sumsq_kernel<<<grid_for(n, 148 * 4), kThreads, 0, stream>>>(grad, n, sumsq_scratch);
  }
  dgc_accumulate_kernel<<<grid_for(n, 148 * 8), kThreads, 0, stream>>>(grad, u, v, n, momentum, clip,
                                                                       sumsq_scratch);
  return cudaGetLastError();
}

cudaError_t dgc_mask(const uint8_t* payload, int64_t payload_capacity, float* u, int64_t n,
                     float* sumsq_scratch, cudaStream_t stream, const uint32_t* epoch_dev,
                     int64_t parity_stride) {
  if (n <= 0 || (reinterpret_cast<uintptr_t>(payload) & 3)) return cudaErrorInvalidValue;
  const int64_t kmax = (payload_capacity - 4) / 8;
  dgc_mask_kernel<<<grid_for(kmax, 148 * 4), kThreads, 0, stream>>>(payload, payload_capacity, u, n,
                                                                    sumsq_scratch, epoch_dev, parity_stride);
  return cudaGetLastError();
}

cudaError_t adamw_apply_dense(float* grad, float scale, const AdamWApply& apply, int64_t n,
                              cudaStream_t stream) {
  if (n <= 0 || !apply.param || !apply.exp_avg || !apply.exp_avg_sq || apply.step < 1)
    return cudaErrorInvalidValue;
  const bool vec = ((reinterpret_cast<uintptr_t>(grad) | reinterpret_cast<uintptr_t>(apply.param) |
                     reinterpret_cast<uintptr_t>(apply.exp_avg) |
                     reinterpret_cast<uintptr_t>(apply.exp_avg_sq)) & 15) == 0;
  if (vec) adamw_kernel<true><<<grid_for((n + 3) >> 2, 148 * 8), kThreads, 0, stream>>>(grad, scale, apply, n);
  else adamw_kernel<false><<<grid_for(n, 148 * 8), kThreads, 0, stream>>>(grad, scale, apply, n);
  return cudaGetLastError();
}

}  // namespace cuda
}  // namespace hipress
