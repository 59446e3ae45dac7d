// Flag wait/signal kernels and small dense helpers.
#include "kernels.h"
#include "p2p.cuh"

namespace hipress {
namespace cuda {

namespace {

constexpr int kThreads = 256;

// One warp; lane r watches flag r.  Epochs only grow, so "reached" is >= with
// wrap-around handled by a signed difference.  The spin is bounded by wall
// time: on expiry the kernel records the failure and returns, the context
// stays usable and the host decides what to do.
__global__ void wait_flags_kernel(const uint32_t* flags, int world, uint32_t epoch,
                                  const uint32_t* epoch_dev, uint64_t timeout_ns, int* status,
                                  unsigned long long* wait_stats) {
  if (epoch_dev != nullptr) epoch = *epoch_dev;
  const int lane = threadIdx.x;
  bool ok = true;
  const uint64_t t0 = globaltimer_ns();
  if (lane < world) {
    ok = false;
    for (;;) {
      const uint32_t v = ld_acquire_sys(flags + lane);
      if (int32_t(v - epoch) >= 0) {
        ok = true;
        break;
      }
      if (globaltimer_ns() - t0 > timeout_ns) break;
      __nanosleep(200);
    }
  }
  const unsigned int all = __ballot_sync(0xffffffffu, ok);
  if (lane == 0 && all != 0xffffffffu && status != nullptr) atomicExch(status, int(kFlagTimeout));
  if (lane == 0 && wait_stats != nullptr) {
    const unsigned long long waited = globaltimer_ns() - t0;   // every lane is done after the ballot
    atomicAdd(wait_stats, waited);
    atomicMax(wait_stats + 1, waited);
    atomicAdd(wait_stats + 2, 1ull);
  }
}

__global__ void stamp_time_kernel(unsigned long long* slot) { *slot = globaltimer_ns(); }

__global__ void signal_flags_kernel(PushTargets dst) {
  resolve_epoch(dst);
  if (threadIdx.x < dst.world && dst.flag[threadIdx.x] != nullptr) {
    __threadfence_system();
    st_release_sys(dst.flag[threadIdx.x], dst.epoch);
  }
}

template <bool VEC>
__global__ void __launch_bounds__(kThreads)
sgd_dense_kernel(float* __restrict__ grad, float scale, SgdApply a, int64_t n) {
  // an earlier kernel of the step recorded a failure: leave parameters and momentum untouched
  if (a.guard != nullptr && *reinterpret_cast<const volatile int*>(a.guard) != 0) return;
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  const int64_t tid = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (VEC) {
    const int64_t nv = n >> 2;
    for (int64_t i = tid; i < nv; i += stride) {
      float4 g = reinterpret_cast<float4*>(grad)[i];
      float4 p = reinterpret_cast<float4*>(a.param)[i];
      float4 b = a.first_step ? make_float4(0, 0, 0, 0) : reinterpret_cast<float4*>(a.momentum)[i];
      float gg[4] = {g.x * scale, g.y * scale, g.z * scale, g.w * scale};
      float pp[4] = {p.x, p.y, p.z, p.w};
      float bb[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float d = gg[k] + a.weight_decay * pp[k];
        bb[k] = a.first_step ? d : a.mu * bb[k] + d;
        pp[k] -= a.lr * bb[k];
      }
      reinterpret_cast<float4*>(grad)[i] =
          a.clear_grad ? make_float4(0.f, 0.f, 0.f, 0.f) : make_float4(gg[0], gg[1], gg[2], gg[3]);
      reinterpret_cast<float4*>(a.momentum)[i] = make_float4(bb[0], bb[1], bb[2], bb[3]);
      reinterpret_cast<float4*>(a.param)[i] = make_float4(pp[0], pp[1], pp[2], pp[3]);
    }
    for (int64_t i = (nv << 2) + tid; i < n; i += stride) {
      const float g = grad[i] * scale;
      grad[i] = a.clear_grad ? 0.f : g;
      sgd_update(a, i, g);
    }
  } else {
    for (int64_t i = tid; i < n; i += stride) {
      const float g = grad[i] * scale;
      grad[i] = a.clear_grad ? 0.f : g;
      sgd_update(a, i, g);
    }
  }
}

__global__ void __launch_bounds__(kThreads)
add_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out,
           int64_t n) {
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    out[i] = a[i] + b[i];
}

struct SrcTable {
  const float* p[kMaxWorld];
};

// epoch_dev: when set, the sources given are the slots of even epochs and odd epochs read
// parity_elems floats further (slots are double-buffered by epoch parity, see PushTargets).
__global__ void __launch_bounds__(kThreads)
gather_sum_kernel(SrcTable srcs, int world, float* __restrict__ out, int64_t n, float post_scale,
                  const uint32_t* epoch_dev, int64_t parity_elems, const int* guard) {
  if (status_guarded(guard)) return;
  const int64_t shift = (epoch_dev != nullptr && (*epoch_dev & 1u)) ? parity_elems : 0;
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    float acc = srcs.p[0][shift + i];
#pragma unroll
    for (int r = 1; r < kMaxWorld; ++r)
      if (r < world) acc += srcs.p[r][shift + i];
    out[i] = acc * post_scale;
  }
}

// slot(parity of *epoch_dev) = src: the dense codec's staging copy when the epoch lives on the device.
__global__ void __launch_bounds__(kThreads)
dense_stage_kernel(const float* __restrict__ src, float* __restrict__ slot_even, int64_t parity_elems,
                   const uint32_t* epoch_dev, int64_t n) {
  float* dst = slot_even + ((*epoch_dev & 1u) ? parity_elems : 0);
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) dst[i] = src[i];
}

inline int grid_for(int64_t items, int max_blocks) {
  int64_t blocks = (items + kThreads - 1) / kThreads;
  if (blocks < 1) blocks = 1;
  if (blocks > max_blocks) blocks = max_blocks;
  return int(blocks);
}

}  // namespace

cudaError_t wait_flags(const uint32_t* flags, int world, uint32_t epoch, uint64_t timeout_ns,
                       int* status, cudaStream_t stream, const uint32_t* epoch_dev,
                       unsigned long long* wait_stats) {
  if (world < 1 || world > kMaxWorld) return cudaErrorInvalidValue;
  wait_flags_kernel<<<1, 32, 0, stream>>>(flags, world, epoch, epoch_dev, timeout_ns, status, wait_stats);
  return cudaGetLastError();
}

cudaError_t stamp_time(unsigned long long* slot, cudaStream_t stream) {
  if (slot == nullptr) return cudaErrorInvalidValue;
  stamp_time_kernel<<<1, 1, 0, stream>>>(slot);
  return cudaGetLastError();
}

namespace {
__global__ void bump_epoch_kernel(uint32_t* epoch_dev) { *epoch_dev += 1u; }
}  // namespace

cudaError_t bump_epoch(uint32_t* epoch_dev, cudaStream_t stream) {
  if (epoch_dev == nullptr) return cudaErrorInvalidValue;
  bump_epoch_kernel<<<1, 1, 0, stream>>>(epoch_dev);
  return cudaGetLastError();
}

cudaError_t signal_flags(const PushTargets& dst, cudaStream_t stream) {
  signal_flags_kernel<<<1, 32, 0, stream>>>(dst);
  return cudaGetLastError();
}

cudaError_t sgd_apply_dense(float* grad, float scale, const SgdApply& apply, int64_t n,
                            cudaStream_t stream) {
  if (n <= 0 || apply.param == nullptr || apply.momentum == nullptr) return cudaErrorInvalidValue;
  const bool vec = ((reinterpret_cast<uintptr_t>(grad) | reinterpret_cast<uintptr_t>(apply.param) |
                     reinterpret_cast<uintptr_t>(apply.momentum)) & 15) == 0;
  const int grid = grid_for((n + 3) >> 2, 148 * 8);
  if (vec) sgd_dense_kernel<true><<<grid, kThreads, 0, stream>>>(grad, scale, apply, n);
  else sgd_dense_kernel<false><<<grid, kThreads, 0, stream>>>(grad, scale, apply, n);
  return cudaGetLastError();
}

cudaError_t add_into(const float* a, const float* b, float* out, int64_t n, cudaStream_t stream) {
  if (n <= 0) return cudaErrorInvalidValue;
  add_kernel<<<grid_for(n, 148 * 8), kThreads, 0, stream>>>(a, b, out, n);
  return cudaGetLastError();
}

cudaError_t dense_gather_sum(const float* const* srcs, int world, float* out, int64_t n,
                             float post_scale, cudaStream_t stream, const uint32_t* epoch_dev,
                             int64_t parity_elems, const int* guard) {
  if (n <= 0 || world < 1 || world > kMaxWorld) return cudaErrorInvalidValue;
  SrcTable t{};
  for (int r = 0; r < world; ++r) t.p[r] = srcs[r];
  gather_sum_kernel<<<grid_for(n, 148 * 8), kThreads, 0, stream>>>(t, world, out, n, post_scale, epoch_dev,
                                                                   parity_elems, guard);
  return cudaGetLastError();
}

cudaError_t dense_stage(const float* src, float* slot_even, int64_t parity_elems, const uint32_t* epoch_dev,
                        int64_t n, cudaStream_t stream) {
  if (n <= 0 || epoch_dev == nullptr) return cudaErrorInvalidValue;
  dense_stage_kernel<<<grid_for(n, 148 * 8), kThreads, 0, stream>>>(src, slot_even, parity_elems, epoch_dev, n);
  return cudaGetLastError();
}

}  // namespace cuda
}  // namespace hipress
