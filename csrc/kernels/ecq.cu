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
// quantise / update H / pack / store to every destination / publish flag.  Both read
// with 16-byte loads when the arrays are aligned, take the step's epoch (flag value, slot
// parity, rounding seed) from the device when asked to, and return at once when an earlier
// kernel of the step recorded a failure.
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

template <bool VEC>
__global__ void __launch_bounds__(kThreads)
ecq_absmax_header_kernel(const float* __restrict__ grad, const float* __restrict__ hist, int64_t n,
                         float alpha, int bw, PushTargets dst, MinMaxScratch* scratch) {
  if (push_guarded(dst)) return;
  resolve_epoch(dst);
  float mx = 0.0f, unused = 0.0f;
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  const int64_t tid = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t nv = VEC ? (n >> 2) : 0;  // 16-byte loads when both arrays are aligned
  for (int64_t i = tid; i < nv; i += stride) {
    const float4 g = __ldg(reinterpret_cast<const float4*>(grad) + i);
    const float4 h = __ldg(reinterpret_cast<const float4*>(hist) + i);
    mx = fmaxf(mx, fmaxf(fmaxf(fabsf(ecq_compensated(g.x, h.x, alpha)), fabsf(ecq_compensated(g.y, h.y, alpha))),
                         fmaxf(fabsf(ecq_compensated(g.z, h.z, alpha)), fabsf(ecq_compensated(g.w, h.w, alpha)))));
  }
  for (int64_t i = (nv << 2) + tid; i < n; i += stride)
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

// One thread quantises four consecutive elements (one 16-byte load of the gradient and of the
// history, one 16-byte store of the history) into BW/2 payload bytes; lanes then combine their
// bytes into 32-bit words, so that every destination gets word stores.  The random generator is
// seeded per payload byte, as in the CPU codec.
template <int BW, bool VEC>
__global__ void __launch_bounds__(kThreads)
ecq_quant_kernel(const float* __restrict__ grad, float* __restrict__ hist, int64_t n, float alpha,
                 float beta, uint64_t seed, PushTargets dst, const MinMaxScratch* scratch) {
  if (push_guarded(dst)) return;
  resolve_epoch(dst);
  if (dst.epoch_dev != nullptr) seed += uint64_t(dst.epoch) * kEpochSeedStride;
  constexpr int DPB = 8 / BW;
  constexpr int BPT = 4 / DPB;  // bytes per thread: 1, 2, 4
  const float mx = scratch->mx, inv = scratch->inv, gap = scratch->gap;
  const bool zero = scratch->mn != 0.0f;
  auto quant_byte = [&](const float* g, float* h, int count, int64_t byte_index) -> uint32_t {
    uint8_t q = 0;
    Lcg32 rng(tern_byte_seed(seed, byte_index));
#pragma unroll
    for (int j = 0; j < DPB; ++j) {
      if (j < count) {
        const float v = ecq_compensated(g[j], h[j], alpha);
        uint8_t t = 0;
        if (!zero) t = ecq_quant(v, mx, inv, rng.next_unit());
        q = uint8_t(q | (int(t) << (BW * j)));
        const uint32_t kept = uint32_t(t) & ((1u << BW) - 1u);
        h[j] = ecq_history(h[j], beta, v, ecq_dequant(kept, gap, mx));
      }
    }
    return q;
  };
  const int64_t units = n >> 2;
  const int64_t units_padded = (units + 31) & ~int64_t(31);
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t u = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; u < units_padded; u += stride) {
    uint32_t bytes = 0;
    if (u < units) {
      float g[4], h[4];
      if (VEC) {
        const float4 gv = __ldg(reinterpret_cast<const float4*>(grad) + u);
        const float4 hv = reinterpret_cast<const float4*>(hist)[u];
        g[0] = gv.x; g[1] = gv.y; g[2] = gv.z; g[3] = gv.w;
        h[0] = hv.x; h[1] = hv.y; h[2] = hv.z; h[3] = hv.w;
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          g[k] = grad[4 * u + k];
          h[k] = hist[4 * u + k];
        }
      }
#pragma unroll
      for (int b = 0; b < BPT; ++b)
        bytes |= quant_byte(g + b * DPB, h + b * DPB, DPB, u * BPT + b) << (8 * b);
      if (VEC) {
        reinterpret_cast<float4*>(hist)[u] = make_float4(h[0], h[1], h[2], h[3]);
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) hist[4 * u + k] = h[k];
      }
    }
    if (BPT == 1) {
      const uint32_t word = gather4_bytes(bytes);
      if ((threadIdx.x & 3) == 0 && u < units) {
        if (u + 3 < units) {
          push_u32(dst, kEcqHeaderBytes + u, word);
        } else {
          for (int64_t b = u; b < units; ++b) push_u8(dst, kEcqHeaderBytes + b, uint8_t(word >> (8 * (b - u))));
        }
      }
    } else if (BPT == 2) {
      const uint32_t word = gather2_halves(bytes);
      if ((threadIdx.x & 1) == 0 && u < units) {
        if (u + 1 < units) {
          push_u32(dst, kEcqHeaderBytes + 2 * u, word);
        } else {
          push_u8(dst, kEcqHeaderBytes + 2 * u, uint8_t(word));
          push_u8(dst, kEcqHeaderBytes + 2 * u + 1, uint8_t(word >> 8));
        }
      }
    } else {
      if (u < units) push_u32(dst, kEcqHeaderBytes + 4 * u, bytes);
    }
  }
  // fewer than four leftover elements
  const int64_t done = units << 2;
  if (done < n && blockIdx.x == 0 && threadIdx.x == 0) {
    int64_t byte_index = done / DPB;
    for (int64_t e = done; e < n; e += DPB, ++byte_index) {
      const int count = (n - e) >= DPB ? DPB : int(n - e);
      float g[DPB], h[DPB];
      for (int j = 0; j < count; ++j) {
        g[j] = grad[e + j];
        h[j] = hist[e + j];
      }
      push_u8(dst, kEcqHeaderBytes + byte_index, uint8_t(quant_byte(g, h, count, byte_index)));
      for (int j = 0; j < count; ++j) hist[e + j] = h[j];
    }
  }
  publish_when_grid_done(dst);
}

// One thread decodes one payload byte of every rank: DPB consecutive elements.
__global__ void __launch_bounds__(kThreads)
ecq_unpack_kernel(UnpackSources src, float* __restrict__ out, int64_t n, int add, float post_scale,
                  int* status) {
  if (status_guarded(src.guard)) return;
  resolve_epoch(src);
  __shared__ float s_mx[kMaxWorld], s_gap[kMaxWorld];
  __shared__ int s_bw[kMaxWorld];
  __shared__ int all_ok;
  if (threadIdx.x == 0) all_ok = 1;
  __syncthreads();
#pragma unroll
  for (int r = 0; r < kMaxWorld; ++r) {  // thread r reads header r; compile-time index into src
    if (int(threadIdx.x) == r && r < src.world) {
      const uint8_t* p = src.payload[r] + src.parity_off;
      uint32_t total = 0, mb = 0;
      for (int k = 0; k < 4; ++k) {
        total |= uint32_t(p[k]) << (8 * k);
        mb |= uint32_t(p[4 + k]) << (8 * k);
      }
      const int bw = p[8], unused = p[9];
      bool ok = ecq_bitwidth_ok(bw) && int64_t(total) <= src.payload_bytes[r];
      if (ok) ok = (int64_t(total) - kEcqHeaderBytes) * (8 / bw) - unused == n;
      const float mx = __uint_as_float(mb);
      s_mx[r] = mx;
      s_bw[r] = bw;
      s_gap[r] = (ok && mx > 0.0f) ? ecq_gap(mx, bw) : 0.0f;
      if (!ok || bw != int(src.payload[0][src.parity_off + 8])) all_ok = 0;
    }
  }
  __syncthreads();
  if (!all_ok) {
    if (blockIdx.x == 0 && threadIdx.x == 0 && status) atomicExch(status, int(kBadHeader));
    return;
  }
  const int bw = s_bw[0], dpb = 8 / bw;
  const uint32_t mask = (1u << bw) - 1u;
  const int64_t M = (n + dpb - 1) / dpb;
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t b = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; b < M; b += stride) {
    uint32_t byte[kMaxWorld];
#pragma unroll
    for (int r = 0; r < kMaxWorld; ++r)
      byte[r] = r < src.world ? uint32_t(src.payload[r][src.parity_off + kEcqHeaderBytes + b]) : 0u;
    for (int j = 0; j < dpb; ++j) {
      const int64_t i = b * dpb + j;
      if (i >= n) break;
      float acc = add ? out[i] : 0.0f;
#pragma unroll
      for (int r = 0; r < kMaxWorld; ++r) {
        if (r < src.world) {
          const float v = ecq_dequant((byte[r] >> (j * bw)) & mask, s_gap[r], s_mx[r]);
          acc = (r == 0 && !add) ? v : hp_add(acc, v);
        }
      }
      if (post_scale != 1.0f) acc = hp_mul(acc, post_scale);
      out[i] = acc;
    }
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
  const bool vec = aligned16(grad) && aligned16(history);
  const int hgrid = grid_for((n + 3) >> 2, kThreads, 148 * 4);
  if (vec) ecq_absmax_header_kernel<true><<<hgrid, kThreads, 0, stream>>>(grad, history, n, alpha, bitwidth, hdr_dst, s);
  else ecq_absmax_header_kernel<false><<<hgrid, kThreads, 0, stream>>>(grad, history, n, alpha, bitwidth, hdr_dst, s);
  const int grid = grid_for((n + 3) >> 2, kThreads, 148 * 8);
#define HP_ECQ(BW)                                                                                               \
  do {                                                                                                           \
    if (vec) ecq_quant_kernel<BW, true><<<grid, kThreads, 0, stream>>>(grad, history, n, alpha, beta, seed, dst, s);  \
    else ecq_quant_kernel<BW, false><<<grid, kThreads, 0, stream>>>(grad, history, n, alpha, beta, seed, dst, s);     \
  } while (0)
  switch (bitwidth) {
    case 2: HP_ECQ(2); break;
    case 4: HP_ECQ(4); break;
    default: HP_ECQ(8); break;
  }
#undef HP_ECQ
  return cudaGetLastError();
}

cudaError_t ecq_unpack_accum(const UnpackSources& src, float* out, int64_t n, int add,
                             float post_scale, int* status, cudaStream_t stream) {
  if (n <= 0 || src.world < 1 || src.world > kMaxWorld) return cudaErrorInvalidValue;
  // one thread per payload byte (at least two elements)
  ecq_unpack_kernel<<<grid_for((n + 1) >> 1, kThreads, 148 * 8), kThreads, 0, stream>>>(src, out, n, add,
                                                                                        post_scale, status);
  return cudaGetLastError();
}

}  // namespace cuda
}  // namespace hipress
