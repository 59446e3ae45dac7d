// TBQ (threshold quantisation with residual feedback) for sm_100a.
//
// Compress: one pass that reads grad and residual with 16-byte loads, updates
// the residual, packs four 2-bit fields per byte, gathers the bytes of four
// lanes into one 32-bit word and stores that word into every destination
// (local buffer and/or NVLink peer slots).  The partial last byte is produced
// in the same kernel, so there is no host round-trip (the reference finishes
// the tail on the host: tbq_body.h:114-155).
//
// Unpack-accumulate: one pass over the dense tensor that decodes the payloads
// of all ranks in ascending rank order through a shared-memory byte table (the
// reference launches one full pass per peer payload: hp_cuda_kernel.cu:182-196),
// optionally scales the sum and applies a fused SGD-momentum update.
#include "../common/codec_math.h"
#include "kernels.h"
#include "p2p.cuh"
#include "unpack_lut.cuh"

namespace hipress {
namespace cuda {

namespace {

constexpr int kThreads = 256;

template <bool VEC>
__global__ void __launch_bounds__(kThreads)
tbq_compress_kernel(const float* __restrict__ grad, float* __restrict__ residual, int64_t n,
                    float thr, PushTargets dst) {
  resolve_epoch(dst);
  const int64_t nquads = n >> 2;                    // full bytes
  const int64_t nquads_padded = (nquads + 31) & ~int64_t(31);  // whole warps iterate together
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t q = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; q < nquads_padded; q += stride) {
    uint32_t byte = 0;
    if (q < nquads) {
      float g[4], r[4];
      if (VEC) {
        const float4 gv = __ldg(reinterpret_cast<const float4*>(grad) + q);
        const float4 rv = reinterpret_cast<const float4*>(residual)[q];
        g[0] = gv.x; g[1] = gv.y; g[2] = gv.z; g[3] = gv.w;
        r[0] = rv.x; r[1] = rv.y; r[2] = rv.z; r[3] = rv.w;
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          g[k] = grad[4 * q + k];
          r[k] = residual[4 * q + k];
        }
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) byte |= tbq_quant(r[k], g[k], thr) << (2 * k);
      if (VEC) {
        reinterpret_cast<float4*>(residual)[q] = make_float4(r[0], r[1], r[2], r[3]);
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) residual[4 * q + k] = r[k];
      }
    }
    const uint32_t word = gather4_bytes(byte);
    if ((threadIdx.x & 3) == 0 && q < nquads) {
      if (q + 3 < nquads) {
        push_u32(dst, q, word);
      } else {
        for (int64_t b = q; b < nquads; ++b) push_u8(dst, b, uint8_t(word >> (8 * (b - q))));
      }
    }
  }
  // partial last byte: unused fields stay "zero" (01)
  const int rem = int(n & 3);
  if (rem && blockIdx.x == 0 && threadIdx.x == 0) {
    uint32_t byte = kTbqEmptyByte;
    for (int k = 0; k < rem; ++k) {
      const int64_t j = (nquads << 2) + k;
      float r = residual[j];
      const uint32_t f = tbq_quant(r, grad[j], thr);
      residual[j] = r;
      byte = (byte & ~(3u << (2 * k))) | (f << (2 * k));
    }
    push_u8(dst, nquads, uint8_t(byte));
  }
  publish_when_grid_done(dst);
}

// Table-driven unpack (see unpack_lut.cuh): one 256 x 4 table shared by all ranks.
template <bool APPLY>
__global__ void __launch_bounds__(kUnpackThreads)
tbq_unpack_lut_kernel(UnpackSources src, float thr, float* __restrict__ out, int64_t n, int add,
                      float post_scale, SgdApply apply) {
  resolve_epoch(src);
  // nibble -> 2 decoded values; one 128-byte table shared by all ranks (see unpack_lut.cuh)
  __shared__ __align__(128) float lut[16 * 2];
  uint32_t first[kMaxWorld];
  unpack_nibble_prefetch<2>(src, 0, src.parity_off, n, first);
  if (threadIdx.x < 32) lut[threadIdx.x] = tbq_dequant((uint32_t(threadIdx.x) >> 1 >> (2 * (threadIdx.x & 1))) & 3u, thr);
  __syncthreads();
  if (unpack_coalesced_ok(src, out, APPLY, apply))
    unpack_nibble_body_coalesced2<APPLY, true>(lut, first, src, src.parity_off, out, n, add, post_scale, apply);
  else
    unpack_nibble_body<2, APPLY, true>(lut, first, src, src.parity_off, out, n, add, post_scale, apply);
}

inline int grid_for(int64_t items, int threads, int max_blocks) {
  int64_t blocks = (items + threads - 1) / threads;
  if (blocks < 1) blocks = 1;
  if (blocks > max_blocks) blocks = max_blocks;
  return int(blocks);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

cudaError_t tbq_compress(const float* grad, float* residual, int64_t n, float threshold,
                         const PushTargets& dst, cudaStream_t stream) {
  if (n <= 0) return cudaErrorInvalidValue;
  // 148 SMs x 8 resident CTAs of 256 threads
  const int grid = grid_for(n >> 2, kThreads, 148 * 8);
  if (aligned16(grad) && aligned16(residual))
    tbq_compress_kernel<true><<<grid, kThreads, 0, stream>>>(grad, residual, n, threshold, dst);
  else
    tbq_compress_kernel<false><<<grid, kThreads, 0, stream>>>(grad, residual, n, threshold, dst);
  return cudaGetLastError();
}

cudaError_t tbq_unpack_accum(const UnpackSources& src, float threshold, float* out, int64_t n,
                             int add, float post_scale, const SgdApply& apply,
                             cudaStream_t stream) {
  if (n <= 0 || src.world < 1 || src.world > kMaxWorld) return cudaErrorInvalidValue;
  // one thread decodes 16 elements per iteration
  const int grid = grid_for((n + 15) >> 4, kUnpackThreads, 148 * 4);
  if (apply.param != nullptr)
    tbq_unpack_lut_kernel<true><<<grid, kUnpackThreads, 0, stream>>>(src, threshold, out, n, add, post_scale, apply);
  else
    tbq_unpack_lut_kernel<false><<<grid, kUnpackThreads, 0, stream>>>(src, threshold, out, n, add, post_scale, apply);
  return cudaGetLastError();
}

}  // namespace cuda
}  // namespace hipress
