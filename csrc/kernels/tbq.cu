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

constexpr int kStageBytes = 512;  // payload bytes a warp gathers before it stores them

// wide: large tensors with 16-byte aligned destinations.  A warp then works on chunks of 512
// payload bytes (2,048 elements): in each of 16 sub-steps lane L quantises elements
// (j*32+L)*4 .. +3 of the chunk (coalesced 16-byte loads), the bytes are gathered in shared
// memory, and every lane stores 16 of them to each destination -- 512 contiguous bytes per warp
// and destination instead of 32, which is what NVLink peer stores need to run near link speed.
// The rest of the tensor (less than one chunk) takes the word path below.
template <bool VEC>
__global__ void __launch_bounds__(kThreads)
tbq_compress_kernel(const float* __restrict__ grad, float* __restrict__ residual, int64_t n,
                    float thr, PushTargets dst, int wide) {
  if (push_guarded(dst)) return;
  resolve_epoch(dst);
  const int64_t S = dst.shard_elems;
  PushCursor cur{nullptr};
  int64_t chunks = 0;
  constexpr int64_t CH = int64_t(kStageBytes) * 4;
  if (VEC && wide) {
    __shared__ __align__(16) uint8_t stage[kThreads / 32][kStageBytes];
    chunks = n / CH;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t warps = int64_t(gridDim.x) * (blockDim.x >> 5);
    for (int64_t c = int64_t(blockIdx.x) * (blockDim.x >> 5) + warp; c < chunks; c += warps) {
      const int64_t ebase = c * CH;
      int64_t bbase = ebase >> 2;  // first payload byte of the chunk, relative to its shard
      if (S > 0) {
        const int j = int(ebase / S);
        cur.one = select_dest(dst, j);
        bbase = (ebase - int64_t(j) * S) >> 2;
      }
#pragma unroll 1
      for (int j0 = 0; j0 < 16; j0 += 4) {
        float4 gv[4], rv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int64_t q = (ebase >> 2) + (j0 + u) * 32 + lane;
          gv[u] = __ldg(reinterpret_cast<const float4*>(grad) + q);
          rv[u] = reinterpret_cast<const float4*>(residual)[q];
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          float g[4] = {gv[u].x, gv[u].y, gv[u].z, gv[u].w};
          float r[4] = {rv[u].x, rv[u].y, rv[u].z, rv[u].w};
          uint32_t byte = 0;
#pragma unroll
          for (int k = 0; k < 4; ++k) byte |= tbq_quant(r[k], g[k], thr) << (2 * k);
          const int unit = (j0 + u) * 32 + lane;
          reinterpret_cast<float4*>(residual)[(ebase >> 2) + unit] = make_float4(r[0], r[1], r[2], r[3]);
          stage[warp][unit] = uint8_t(byte);
        }
      }
      __syncwarp();
      const uint4 v = reinterpret_cast<const uint4*>(stage[warp])[lane];
      put_u128(dst, cur, bbase + lane * 16, v);
      __syncwarp();
    }
  }

  // ---- the rest: one byte per thread, four lanes combine theirs into a 32-bit word
  const int64_t rest_begin = chunks * CH;
  int64_t shard_base = 0;  // first element of the shard holding the rest
  if (S > 0 && rest_begin < n) {
    const int j = int(rest_begin / S);
    cur.one = select_dest(dst, j);
    shard_base = int64_t(j) * S;
  }
  const int64_t q0 = rest_begin >> 2;               // first byte of the rest (tensor-relative)
  const int64_t qshift = shard_base >> 2;           // payload byte = tensor byte - qshift
  const int64_t nquads = n >> 2;                    // full bytes
  const int64_t span_padded = (nquads - q0 + 31) & ~int64_t(31);  // whole warps iterate together
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t k = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; k < span_padded; k += stride) {
    const int64_t q = q0 + k;
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
        for (int k2 = 0; k2 < 4; ++k2) {
          g[k2] = grad[4 * q + k2];
          r[k2] = residual[4 * q + k2];
        }
      }
#pragma unroll
      for (int k2 = 0; k2 < 4; ++k2) byte |= tbq_quant(r[k2], g[k2], thr) << (2 * k2);
      if (VEC) {
        reinterpret_cast<float4*>(residual)[q] = make_float4(r[0], r[1], r[2], r[3]);
      } else {
#pragma unroll
        for (int k2 = 0; k2 < 4; ++k2) residual[4 * q + k2] = r[k2];
      }
    }
    const uint32_t word = gather4_bytes(byte);
    if ((threadIdx.x & 3) == 0 && q < nquads) {
      if (q + 3 < nquads) {
        put_u32(dst, cur, q - qshift, word);
      } else {
        for (int64_t b = q; b < nquads; ++b) put_u8(dst, cur, b - qshift, uint8_t(word >> (8 * (b - q))));
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
    put_u8(dst, cur, nquads - qshift, uint8_t(byte));
  }
  publish_when_grid_done(dst);
}

// Table-driven unpack (see unpack_lut.cuh): one table shared by all ranks.  MODE is chosen by the
// launcher so that each form is its own kernel with its own register budget: kPair = pair table
// (aligned dense arrays), kConcat = concatenated shards, kGeneric = nibble table.
enum UnpackMode : int { kGeneric = 0, kPair = 1, kConcat = 2 };

template <bool APPLY, int MODE, int WORLD>
__global__ void __launch_bounds__(kUnpackThreads, MODE == kGeneric ? 1 : 4)
tbq_unpack_lut_kernel(UnpackSources src, float thr, float* __restrict__ out, int64_t n, int add,
                      float post_scale, SgdApply apply) {
  if (unpack_guarded(src)) return;
  resolve_epoch(src);
  // pair table [256][2] (2 KB): row (b << 4) | a = decode(a) + decode(b); otherwise the plain
  // nibble table [16][2]
  __shared__ __align__(128) float tab[MODE == kPair ? kPairRows * 2 : 32];
  uint32_t first[kMaxWorld];
  if constexpr (MODE != kConcat) unpack_nibble_prefetch<2>(src, 0, src.parity_off, n, first);
  if constexpr (MODE == kPair) {
    build_pair_tables<true>(tab, src.world, [&](int, int nibble, int which) {
      return tbq_dequant((uint32_t(nibble) >> (2 * which)) & 3u, thr);
    });
    __syncthreads();
    // a rank without a partner pairs with four "zero" fields, which decode to +0.0
    unpack_pair_body<APPLY, true, (WORLD > 0 ? WORLD : 1)>(tab, 0x55555555u, first, src, src.parity_off, out, n, add, post_scale, apply);
  } else {
    if (threadIdx.x < 32) tab[threadIdx.x] = tbq_dequant((uint32_t(threadIdx.x) >> 1 >> (2 * (threadIdx.x & 1))) & 3u, thr);
    __syncthreads();
    if constexpr (MODE == kConcat)
      unpack_concat_body<APPLY, true>(tab, src, src.parity_off, out, n, add, post_scale, apply);
    else
      unpack_nibble_body<2, APPLY, true>(tab, first, src, src.parity_off, out, n, add, post_scale, apply);
  }
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
  const bool vec = aligned16(grad) && aligned16(residual);
  const int64_t S = dst.shard_elems;
  bool dst16 = (dst.parity_stride & 15) == 0;
  for (int p = 0; p < dst.world; ++p) dst16 = dst16 && aligned16(dst.payload[p]);
  if (dst.mc != nullptr) dst16 = dst16 && aligned16(dst.mc);
  // scatter mode runs on the chunked path only (see tbq_compress_kernel)
  if (S > 0 && (!vec || !dst16 || S % 4096 != 0 || (n + S - 1) / S > dst.world)) return cudaErrorInvalidValue;
  // chunked path with 16-byte stores once there is a chunk per warp of a half-filled GPU
  const int64_t chunks = n / (int64_t(kStageBytes) * 4);
  const int wide = (vec && dst16 && (S > 0 || chunks >= 148 * 2)) ? 1 : 0;
  const int threads = wide ? 128 : kThreads;
  // word path: 148 SMs x 8 resident CTAs of 256 threads
  const int grid = wide ? grid_for(chunks * 32, threads, 148 * 16) : grid_for(n >> 2, kThreads, 148 * 8);
  if (vec)
    tbq_compress_kernel<true><<<grid, threads, 0, stream>>>(grad, residual, n, threshold, dst, wide);
  else
    tbq_compress_kernel<false><<<grid, threads, 0, stream>>>(grad, residual, n, threshold, dst, wide);
  return cudaGetLastError();
}

cudaError_t tbq_unpack_accum(const UnpackSources& src, float threshold, float* out, int64_t n,
                             int add, float post_scale, const SgdApply& apply,
                             cudaStream_t stream) {
  if (n <= 0 || src.world < 1 || src.world > kMaxWorld) return cudaErrorInvalidValue;
  if (src.shard_elems > 0) {
    // concatenated shards: 16-byte aligned dense arrays only
    bool ok = src.shard_elems % 2048 == 0 && aligned16(out) &&
              (n + src.shard_elems - 1) / src.shard_elems <= src.world;
    if (apply.param != nullptr) ok = ok && aligned16(apply.param) && aligned16(apply.momentum);
    if (!ok) return cudaErrorInvalidValue;
  }
  // one thread decodes 16 elements per iteration
  const int grid = grid_for((n + 15) >> 4, kUnpackThreads, 148 * 4);
  bool aligned = aligned16(out);
  if (apply.param != nullptr) aligned = aligned && aligned16(apply.param) && aligned16(apply.momentum);
  const int mode = src.shard_elems > 0 ? kConcat : (aligned ? kPair : kGeneric);
#define HP_LAUNCH(AP, MODE, W) \
  tbq_unpack_lut_kernel<AP, MODE, W><<<grid, kUnpackThreads, 0, stream>>>(src, threshold, out, n, add, post_scale, apply)
#define HP_PAIR(AP)                                                                                     \
  switch (src.world) {                                                                                  \
    case 1: HP_LAUNCH(AP, kPair, 1); break;  case 2: HP_LAUNCH(AP, kPair, 2); break;                    \
    case 3: HP_LAUNCH(AP, kPair, 3); break;  case 4: HP_LAUNCH(AP, kPair, 4); break;                    \
    case 5: HP_LAUNCH(AP, kPair, 5); break;  case 6: HP_LAUNCH(AP, kPair, 6); break;                    \
    case 7: HP_LAUNCH(AP, kPair, 7); break;  default: HP_LAUNCH(AP, kPair, 8); break;                   \
  }
  if (apply.param != nullptr) {
    if (mode == kConcat) HP_LAUNCH(true, kConcat, 0);
    else if (mode == kPair) { HP_PAIR(true) }
    else HP_LAUNCH(true, kGeneric, 0);
  } else {
    if (mode == kConcat) HP_LAUNCH(false, kConcat, 0);
    else if (mode == kPair) { HP_PAIR(false) }
    else HP_LAUNCH(false, kGeneric, 0);
  }
#undef HP_PAIR
#undef HP_LAUNCH
  return cudaGetLastError();
}

}  // namespace cuda
}  // namespace hipress
