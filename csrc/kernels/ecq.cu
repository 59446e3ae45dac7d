// ECQ: error-compensated stochastic quantisation with a history tensor H, for
// sm_100a.  Payload layout follows the reference (ecq_body.h:266-276):
//   {i32 total = 10 + M, f32 max, u8 bitwidth, u8 unused_slots} + M data bytes.
// Semantics are the corrected ones implemented by the CPU codec
// (csrc/codec_cpu/codec_cpu.cpp): v = G + alpha*H keeps its sign, every data
// byte is produced, and the header is written on the device once the maximum
// is known (the reference reads the maximum on the host before the copy that
// delivers it has completed, ecq_body.h:203-214).
//
// Two kernels, no host synchronisation: abs-max grid reduction (+ header), then
// quantise / update H / pack / store to every destination / publish flag.
#include "../common/codec_math.h"
#include "kernels.h"
#include "p2p.cuh"
#include "reduce.cuh"

namespace hipress {
namespace cuda {

namespace {

constexpr int kThreads = 256;
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
inline int grid_for(int64_t items, int threads, int max_blocks) {
  int64_t blocks = (items + threads - 1) / threads;
  if (blocks < 1) blocks = 1;
  if (blocks > max_blocks) blocks = max_blocks;
  return int(blocks);
}

__global__ void __launch_bounds__(kThreads)
ecq_absmax_header_kernel(const float* __restrict__ grad, const float* __restrict__ hist, int64_t n,
                         float alpha, int bw, PushTargets dst, MinMaxScratch* scratch) {
  float mx = 0.0f, unused = 0.0f;
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    mx = fmaxf(mx, fabsf(ecq_compensated(grad[i], hist[i], alpha)));
  float gmn, gmx;
  if (!grid_minmax_last_block<kThreads>(scratch, unused, mx, gmn, gmx)) return;
  if (threadIdx.x == 0) {
    const bool zero = gmx < kEcqZeroCutoff;
    const float hmx = zero ? 0.0f : gmx;
    const float gap = zero ? 0.0f : ecq_gap(gmx, bw);
    scratch->mx = hmx;
    scratch->mn = zero ? 1.0f : 0.0f;  // "zero tensor" marker for kernel 2
    scratch->gap = gap;
    scratch->inv = zero ? 0.0f : ecq_gap_inverse(gap);
    const int dpb = 8 / bw;
    const int64_t M = (n + dpb - 1) / dpb;
    const uint32_t total = uint32_t(kEcqHeaderBytes + M);
    const uint32_t mb = __float_as_uint(hmx);
    uint8_t header[kEcqHeaderBytes];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      header[k] = uint8_t(total >> (8 * k));
      header[4 + k] = uint8_t(mb >> (8 * k));
    }
    header[8] = uint8_t(bw);
    header[9] = uint8_t(M * dpb - n);
    push_bytes(dst, 0, header, kEcqHeaderBytes);
  }
}

template <int BW>
__global__ void __launch_bounds__(kThreads)
ecq_quant_kernel(const float* __restrict__ grad, float* __restrict__ hist, int64_t n, float alpha,
                 float beta, uint64_t seed, PushTargets dst, const MinMaxScratch* scratch) {
  constexpr int DPB = 8 / BW;
  const float mx = scratch->mx, inv = scratch->inv, gap = scratch->gap;
  const bool zero = scratch->mn != 0.0f;
  const int64_t M = (n + DPB - 1) / DPB;
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t b = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; b < M; b += stride) {
    uint8_t q = 0;
    Lcg32 rng(tern_byte_seed(seed, b));
#pragma unroll
    for (int j = 0; j < DPB; ++j) {
      const int64_t e = b * DPB + j;
      if (e < n) {
        const float h = hist[e];
        const float v = ecq_compensated(grad[e], h, alpha);
        uint8_t t = 0;
        if (!zero) t = ecq_quant(v, mx, inv, rng.next_unit());
        q = uint8_t(q | (int(t) << (BW * j)));
        const uint32_t kept = uint32_t(t) & ((1u << BW) - 1u);
        hist[e] = ecq_history(h, beta, v, ecq_dequant(kept, gap, mx));
      }
    }
    push_u8(dst, kEcqHeaderBytes + b, q);
  }
  publish_when_grid_done(dst);
}

__global__ void __launch_bounds__(kThreads)
ecq_unpack_kernel(UnpackSources src, float* __restrict__ out, int64_t n, int add, float post_scale,
                  int* status) {
  __shared__ float s_mx[kMaxWorld], s_gap[kMaxWorld];
  __shared__ int s_bw[kMaxWorld];
  __shared__ int all_ok;
  if (threadIdx.x == 0) all_ok = 1;
  __syncthreads();
  if (threadIdx.x < src.world) {
    const uint8_t* p = src.payload[threadIdx.x];
    uint32_t total = 0, mb = 0;
    for (int k = 0; k < 4; ++k) {
      total |= uint32_t(p[k]) << (8 * k);
      mb |= uint32_t(p[4 + k]) << (8 * k);
    }
    const int bw = p[8], unused = p[9];
    bool ok = ecq_bitwidth_ok(bw) && int64_t(total) <= src.payload_bytes[threadIdx.x];
    if (ok) ok = (int64_t(total) - kEcqHeaderBytes) * (8 / bw) - unused == n;
    const float mx = __uint_as_float(mb);
    s_mx[threadIdx.x] = mx;
    s_bw[threadIdx.x] = bw;
    s_gap[threadIdx.x] = (ok && mx > 0.0f) ? ecq_gap(mx, bw) : 0.0f;
    if (!ok) all_ok = 0;
  }
  __syncthreads();
  if (!all_ok) {
    if (blockIdx.x == 0 && threadIdx.x == 0 && status) atomicExch(status, int(kBadHeader));
    return;
  }
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    float acc = add ? out[i] : 0.0f;
    for (int r = 0; r < src.world; ++r) {
      const int bw = s_bw[r], dpb = 8 / bw;
      const uint32_t byte = src.payload[r][kEcqHeaderBytes + i / dpb];
      const uint32_t q = (byte >> ((i % dpb) * bw)) & ((1u << bw) - 1u);
      const float v = ecq_dequant(q, s_gap[r], s_mx[r]);
      acc = (r == 0 && !add) ? v : hp_add(acc, v);
    }
    if (post_scale != 1.0f) acc = hp_mul(acc, post_scale);
    out[i] = acc;
  }
}

}  // namespace

cudaError_t ecq_compress(const float* grad, float* history, int64_t n, float alpha, float beta,
                         int bitwidth, uint64_t seed, const PushTargets& dst, void* scratch,
                         cudaStream_t stream) {
  if (n <= 0 || !ecq_bitwidth_ok(bitwidth) || scratch == nullptr) return cudaErrorInvalidValue;
  auto* s = static_cast<MinMaxScratch*>(scratch);
  PushTargets hdr_dst = dst;
  hdr_dst.done = nullptr;
  ecq_absmax_header_kernel<<<grid_for(n, kThreads, 148 * 4), kThreads, 0, stream>>>(
      grad, history, n, alpha, bitwidth, hdr_dst, s);
  const int dpb = 8 / bitwidth;
  const int grid = grid_for((n + dpb - 1) / dpb, kThreads, 148 * 8);
  switch (bitwidth) {
    case 2: ecq_quant_kernel<2><<<grid, kThreads, 0, stream>>>(grad, history, n, alpha, beta, seed, dst, s); break;
    case 4: ecq_quant_kernel<4><<<grid, kThreads, 0, stream>>>(grad, history, n, alpha, beta, seed, dst, s); break;
    default: ecq_quant_kernel<8><<<grid, kThreads, 0, stream>>>(grad, history, n, alpha, beta, seed, dst, s); break;
  }
  return cudaGetLastError();
}

cudaError_t ecq_unpack_accum(const UnpackSources& src, float* out, int64_t n, int add,
                             float post_scale, int* status, cudaStream_t stream) {
  if (n <= 0 || src.world < 1 || src.world > kMaxWorld) return cudaErrorInvalidValue;
  ecq_unpack_kernel<<<grid_for(n, kThreads, 148 * 8), kThreads, 0, stream>>>(src, out, n, add,
                                                                             post_scale, status);
  return cudaGetLastError();
}

}  // namespace cuda
}  // namespace hipress
