// PowerSGD kernels for sm_100a.
//
// The two projections of a PowerSGD step,
//     P[n x r] = Mat[n x m] * Q[m x r]          (mode 0)
//     Q[m x r] = Mat^T      * P[n x r]          (mode 1)
// have r <= 16 and are bound by one read of Mat from HBM.  They run as
// tcgen05 tiles: Mat is streamed by TMA (128-byte swizzle) through a 6-stage
// shared-memory ring, one thread issues tcgen05.mma.kind::tf32 with a
// 128 x 16 fp32 accumulator in tensor memory, and four epilogue warps read the
// accumulator back with tcgen05.ld and reduce their rows into the *owner* of
// those rows with red.global.add.f32 -- the owner may be a peer GPU (NVLink
// peer memory), which makes the kernel a fused GEMM + reduce-scatter.  Mode 1
// consumes Mat through the MN-major operand form, so Mat is never transposed
// in memory.  A step's projections run as ONE grid over all matrices of the
// model (psgd_gemm_grouped: units of row tile x K range, largest first), because
// a launch per matrix costs more in ramp-up and drain than the small matrices
// take to stream.  The reference computes these with torch::mm (cuBLAS), one
// call per matrix, and leaves the all-reduce to its caller
// (ref powersgd_body.h:28, 49).
//
// Shapes TMA cannot describe (row pitch not a multiple of 16 bytes, unaligned
// base) take a plain SIMT kernel with the same interface.
//
// Also here: the hand-written Gram-Schmidt orthonormalisation (the reference
// uses geqrf + orgqr, powersgd_body.h:45-46) and the fused
// expand / residual kernel (ref powersgd_body.h:69-75).
#include <cuda.h>

#include <cstdlib>
#include <cstring>
#include <vector>
#include <algorithm>

#include "kernels.h"
#include "p2p.cuh"
#include "unpack_lut.cuh"

namespace hipress {
namespace cuda {

namespace {

constexpr int kBM = 128;     // accumulator rows per CTA (UMMA M)
constexpr int kBN = 16;      // padded rank (UMMA N)
constexpr int kBoxK = 32;    // fp32 elements along K of one TMA box = 128 bytes, the swizzle width
constexpr int kKPad = 64;    // the K extent of the operands is padded to a multiple of this
constexpr int kGemmThreads = 192;       // warp0 TMA, warp1 MMA, warps 2-5 epilogue
constexpr int kGemmGroup = 24;          // matrices per grouped launch (descriptors travel as kernel parameters)
constexpr uint64_t kWaitLimitNs = 2000000000ull;  // every barrier wait gives up after 2 s
constexpr int kTmemCols = 32;

// BK: fp32 elements along K per pipeline stage (32 or 64: one or two 128-byte boxes per matrix
// row, i.e. 128- or 256-byte runs in DRAM); STAGES: depth of the ring.
template <int BK, int STAGES>
struct GemmSmem {
  static constexpr int kStageA = kBM * BK * 4;
  static constexpr int kStageB = kBN * BK * 4;
  // 1024-byte aligned tiles first
  uint8_t a[STAGES][kStageA];
  uint8_t b[STAGES][kStageB];
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t accum;
  uint32_t tmem_base;
  int abort;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: false when the limit ran out or another role gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t i = 1;; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 63u) == 0u) {
      if (*abort) return false;
      if (globaltimer_ns() - t0 > kWaitLimitNs) break;
      __nanosleep(64);
    }
  }
  *abort = 1;
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar))
      : "memory");
}
// Shared-memory matrix descriptor, version 1.  layout: 2 = 128-byte swizzle of
// 16-byte units (K-major operands), 1 = 128-byte swizzle of 32-byte units, the
// only layout MN-major 32-bit (tf32) operands may use.
__device__ __forceinline__ uint64_t make_desc(uint32_t addr, uint32_t lbo, uint32_t sbo,
                                              uint32_t layout) {
  uint64_t d = 0;
  d |= uint64_t((addr >> 4) & 0x3fffu);
  d |= uint64_t((lbo >> 4) & 0x3fffu) << 16;
  d |= uint64_t((sbo >> 4) & 0x3fffu) << 32;
  d |= uint64_t(1) << 46;
  d |= uint64_t(layout & 7u) << 61;
  return d;
}
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}

struct OwnerTargets {
  int world;
  float* dst[kMaxWorld];
  int64_t rows_per_owner;
};

// MODE 0: out[n x r] += Mat * X,   A tile K-major  (rows of Mat x K along m)
// MODE 1: out[m x r] += Mat^T * X, A tile MN-major (columns of Mat x K along n)
// Xt is X transposed and zero-padded to [16][k_pad] (K-major B operand).
template <int MODE, int BK, int STAGES>
__device__ __forceinline__ void psgd_gemm_body(const CUtensorMap* map_a_p, const CUtensorMap* map_b_p,
                                               const float* __restrict__ Mat, int64_t n, int64_t m,
                                               int64_t out_rows, int r, int tile, int kb_begin, int nkb,
                                               const OwnerTargets& out, int* status) {
  using Smem = GemmSmem<BK, STAGES>;
  constexpr int kBK = BK, kStages = STAGES, kStageA = Smem::kStageA, kStageB = Smem::kStageB;
  constexpr int kBoxes = BK / kBoxK;   // 128-byte boxes along K per stage
  extern __shared__ uint8_t smem_raw[];
  Smem& s = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&s.full[i], 1);
      mbar_init(&s.empty[i], 1);
    }
    mbar_init(&s.accum, 1);
    s.abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&s.tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = s.tmem_base;
  volatile int* abort = &s.abort;

  if (nkb > 0) {
    if (warp == 0 && lane == 0) {
      // ---------------- TMA producer
      for (int i = 0; i < nkb; ++i) {
        const int st = i % kStages;
        const uint32_t round = uint32_t(i / kStages);
        if (round > 0 && !mbar_wait(&s.empty[st], (round - 1) & 1u, abort)) break;
        mbar_expect_tx(&s.full[st], kStageA + kStageB);
        const int k0 = (kb_begin + i) * kBK;
        if (MODE == 0) {
          // K-major A: one box of 128 rows x 128 bytes per 32 K elements, side by side in K
#pragma unroll
          for (int j = 0; j < kBoxes; ++j)
            tma_load_2d(s.a[st] + j * (kBM * 128), map_a_p, k0 + j * kBoxK, tile * kBM, &s.full[st]);
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            tma_load_2d(s.a[st] + j * (kBK * 128), map_a_p, tile * kBM + j * 32, k0, &s.full[st]);
        }
#pragma unroll
        for (int j = 0; j < kBoxes; ++j)
          tma_load_2d(s.b[st] + j * (kBN * 128), map_b_p, k0 + j * kBoxK, 0, &s.full[st]);
      }
    } else if (warp == 1 && lane == 0) {
      // ---------------- MMA issuer
      // instruction descriptor: fp32 accumulate, tf32 x tf32, N = 16, M = 128
      const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | (uint32_t(MODE == 1) << 15) |
                             (uint32_t(kBN >> 3) << 17) | (uint32_t(kBM >> 4) << 24);
      bool ok = true;
      for (int i = 0; i < nkb && ok; ++i) {
        const int st = i % kStages;
        const uint32_t round = uint32_t(i / kStages);
        ok = mbar_wait(&s.full[st], round & 1u, abort);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a0 = smem_u32(s.a[st]);
        const uint32_t b0 = smem_u32(s.b[st]);
#pragma unroll
        for (int k = 0; k < kBK / 8; ++k) {
          // K-major: 8 tf32 = 32 bytes further along the swizzled row; 8-row
          // groups are 1024 bytes apart.
          // MN-major: swizzle atoms are 4 K-rows x 128 bytes (512 bytes apart,
          // SBO); the four 32-column groups of the tile are one TMA box apart
          // (LBO); one MMA consumes 8 K-rows = 1024 bytes.
          // with two boxes per stage the K-major operands continue in the next box after four MMAs
          const uint64_t da = MODE == 0 ? make_desc(a0 + (k / 4) * (kBM * 128) + (k % 4) * 32, 16, 1024, 2)
                                        : make_desc(a0 + k * 1024, kBK * 128, 512, 1);
          const uint64_t db = make_desc(b0 + (k / 4) * (kBN * 128) + (k % 4) * 32, 16, 1024, 2);
          umma_tf32(tmem, da, db, idesc, (i > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&s.empty[st]);  // frees the stage once the MMAs have read it
      }
      if (ok) umma_commit(&s.accum);
    } else if (warp >= 2) {
      // ---------------- epilogue: TMEM -> registers -> owner's buffer
      if (mbar_wait(&s.accum, 0, abort)) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int quarter = warp & 3;  // TMEM lanes this warp may touch
        uint32_t v[16];
        const uint32_t taddr = tmem + (uint32_t(quarter * 32) << 16);
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, "
            "%12, %13, %14, %15}, [%16];"
            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
              "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
              "=r"(v[14]), "=r"(v[15])
            : "r"(taddr));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const int64_t row = int64_t(tile) * kBM + quarter * 32 + lane;
        if (row < out_rows) {
          int owner = int(row / out.rows_per_owner);
          if (owner >= out.world) owner = out.world - 1;
          float* dst = out.dst[owner] + row * r;
          if (r == 4 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
            // one 16-byte reduction per row: a remote owner sees a quarter of the NVLink
            // transactions of four scalar atomics
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(__uint_as_float(v[0])),
                         "f"(__uint_as_float(v[1])), "f"(__uint_as_float(v[2])), "f"(__uint_as_float(v[3]))
                         : "memory");
          } else if ((r & 1) == 0 && (reinterpret_cast<uintptr_t>(dst) & 7) == 0) {
#pragma unroll
            for (int c = 0; c < 16; c += 2)
              if (c < r)
                asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(dst + c), "f"(__uint_as_float(v[c])),
                             "f"(__uint_as_float(v[c + 1]))
                             : "memory");
          } else {
#pragma unroll
            for (int c = 0; c < 16; ++c)
              if (c < r) atomicAdd(dst + c, __uint_as_float(v[c]));
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (s.abort) {
    // give copies that may still be in flight time to land before the CTA's
    // shared memory is released
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    if (threadIdx.x == 0 && status != nullptr) atomicExch(status, int(kFlagTimeout));
  }
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols)
                 : "memory");
  }
}

// One matrix per launch: grid = (row tiles, K splits), a contiguous K range per CTA.  (Dealing
// the K blocks round-robin, so that the CTAs sharing a row tile would read neighbouring 128-byte
// pieces of the same rows at about the same time, was measured and is slower.)
template <int MODE, int BK, int STAGES>
__global__ void __launch_bounds__(kGemmThreads, 1)
psgd_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const float* __restrict__ Mat, int64_t n, int64_t m,
                 int64_t out_rows, int r, int total_kb, int kb_per_split, const __grid_constant__ OwnerTargets out,
                 int* status) {
  const int kb_begin = blockIdx.y * kb_per_split;
  const int kb_end = min(kb_begin + kb_per_split, total_kb);
  psgd_gemm_body<MODE, BK, STAGES>(&map_a, &map_b, Mat, n, m, out_rows, r, int(blockIdx.x), kb_begin,
                                          kb_end - kb_begin, out, status);
}

// All matrices of a step in one launch.  A kernel of this kind spends 7-8 us ramping up and
// draining whatever its size (a 9 MB convolution matrix streams in 1.5 us), so a model's tens of
// matrices are projected by ONE grid: CTA u works on unit u of a list that runs through the
// matrices (largest units first), a unit being one row tile x one K range of one matrix.
struct GroupedMat {
  alignas(64) CUtensorMap map_a;
  alignas(64) CUtensorMap map_b;
  const float* Mat;
  int64_t n, m, out_rows;
  OwnerTargets out;
  int unit_begin, tiles, kbps, total_kb;
};
struct GroupedGemm {
  int count;
  int r;
  GroupedMat mat[kGemmGroup];
};
template <int MODE, int BK, int STAGES>
__global__ void __launch_bounds__(kGemmThreads, 1)
psgd_gemm_grouped_kernel(const __grid_constant__ GroupedGemm g, int* status) {
  int u = int(blockIdx.x), i = 0;
  while (i + 1 < g.count && u >= g.mat[i + 1].unit_begin) ++i;
  const GroupedMat& M = g.mat[i];
  u -= M.unit_begin;
  const int tile = u % M.tiles, split = u / M.tiles;
  const int kb_begin = split * M.kbps;
  const int kb_end = min(kb_begin + M.kbps, M.total_kb);
  psgd_gemm_body<MODE, BK, STAGES>(&M.map_a, &M.map_b, M.Mat, M.n, M.m, M.out_rows, g.r, tile, kb_begin,
                                          kb_end - kb_begin, M.out, status);
}

// X[rows x r] row-major -> Xt[16][rows_pad], zero padded.
__global__ void transpose_pad_kernel(const float* __restrict__ X, int64_t rows, int r,
                                     float* __restrict__ Xt, int64_t rows_pad) {
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < rows_pad; i += stride) {
#pragma unroll
    for (int c = 0; c < kBN; ++c) Xt[c * rows_pad + i] = (i < rows && c < r) ? X[i * r + c] : 0.0f;
  }
}

// SIMT path, mode 0: one warp per output row.
__global__ void __launch_bounds__(256)
simt_gemm_p_kernel(const float* __restrict__ Mat, const float* __restrict__ Q, int64_t n, int64_t m,
                   int r, OwnerTargets out) {
  const int lane = threadIdx.x & 31;
  const int64_t row = int64_t(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (row >= n) return;
  float acc[16];
#pragma unroll
  for (int c = 0; c < 16; ++c) acc[c] = 0.f;
  for (int64_t k = lane; k < m; k += 32) {
    const float a = Mat[row * m + k];
#pragma unroll
    for (int c = 0; c < 16; ++c)
      if (c < r) acc[c] += a * Q[k * r + c];
  }
#pragma unroll
  for (int c = 0; c < 16; ++c) {
    if (c < r) {
      float v = acc[c];
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      acc[c] = v;
    }
  }
  if (lane == 0) {
    int owner = int(row / out.rows_per_owner);
    if (owner >= out.world) owner = out.world - 1;
    for (int c = 0; c < r; ++c) atomicAdd(out.dst[owner] + row * r + c, acc[c]);
  }
}

// SIMT path, mode 1: thread per Mat column, CTA per (column block, row chunk).
__global__ void __launch_bounds__(256)
simt_gemm_q_kernel(const float* __restrict__ Mat, const float* __restrict__ P, int64_t n, int64_t m,
                   int r, int64_t rows_per_cta, OwnerTargets out) {
  const int64_t col = int64_t(blockIdx.x) * 256 + threadIdx.x;
  const int64_t i0 = int64_t(blockIdx.y) * rows_per_cta;
  const int64_t i1 = min(i0 + rows_per_cta, n);
  if (col >= m) return;
  float acc[16];
#pragma unroll
  for (int c = 0; c < 16; ++c) acc[c] = 0.f;
  for (int64_t i = i0; i < i1; ++i) {
    const float a = Mat[i * m + col];
#pragma unroll
    for (int c = 0; c < 16; ++c)
      if (c < r) acc[c] += a * P[i * r + c];
  }
  int owner = int(col / out.rows_per_owner);
  if (owner >= out.world) owner = out.world - 1;
  for (int c = 0; c < r; ++c) atomicAdd(out.dst[owner] + col * r + c, acc[c]);
}

// ---------------------------------------------------------------- Gram-Schmidt
constexpr int kGsThreads = 1024;

__device__ __forceinline__ float block_sum(float v, float* sh) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  if (warp == 0) {
    v = lane < kGsThreads / 32 ? sh[lane] : 0.f;
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) sh[0] = v;
  }
  __syncthreads();
  return sh[0];
}

// One CTA orthonormalises one n x r matrix in place (modified Gram-Schmidt,
// columns left to right): col_j /= (|col_j| + eps); col_k -= <col_j, col_k> col_j.
__global__ void __launch_bounds__(kGsThreads)
gram_schmidt_kernel(float* __restrict__ P, int64_t n, int r, float eps) {
  __shared__ float sh[kGsThreads / 32];
  for (int j = 0; j < r; ++j) {
    float ss = 0.f;
    for (int64_t i = threadIdx.x; i < n; i += kGsThreads) {
      const float v = P[i * r + j];
      ss += v * v;
    }
    const float norm = sqrtf(block_sum(ss, sh));
    const float inv = 1.0f / (norm + eps);
    for (int64_t i = threadIdx.x; i < n; i += kGsThreads) P[i * r + j] *= inv;
    __syncthreads();
    for (int c = j + 1; c < r; ++c) {
      float dot = 0.f;
      for (int64_t i = threadIdx.x; i < n; i += kGsThreads) dot += P[i * r + j] * P[i * r + c];
      dot = block_sum(dot, sh);
      for (int64_t i = threadIdx.x; i < n; i += kGsThreads) P[i * r + c] -= dot * P[i * r + j];
      __syncthreads();
    }
  }
}

// ---------------------------------------------------------------- expand
// approx[i,k] = sum_c P[i,c] Q[k,c].
//   mode 0: Mat = approx; residual[:N] = grad - Mat[:N]; grad[:N] = Mat[:N]
//   mode 1: grad[:N] = scale * approx; Mat -= approx      (error feedback kept in Mat)
//   mode 2: Mat -= approx, and the parameters take a fused SGD-momentum step with
//           g = scale * approx (residual/grad unused)
template <int MODE>
__global__ void __launch_bounds__(256)
expand_kernel(const float* __restrict__ P, const float* __restrict__ Q, int64_t n, int64_t m, int r,
              float* __restrict__ Mat, float* __restrict__ residual, float* __restrict__ grad,
              int64_t N, float scale, SgdApply apply) {
  const int64_t total = n * m;
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; e < total; e += stride) {
    const int64_t i = e / m, k = e - i * m;
    float acc = 0.f;
    for (int c = 0; c < r; ++c) acc += P[i * r + c] * Q[k * r + c];
    if (MODE == 0) {
      Mat[e] = acc;
      if (e < N) {
        residual[e] = grad[e] - acc;
        grad[e] = acc;
      }
    } else if (MODE == 1) {
      Mat[e] -= acc;
      if (e < N) grad[e] = acc * scale;
    } else {
      Mat[e] -= acc;
      if (e < N) sgd_update(apply, e, acc * scale);
    }
  }
}

// Vectorised form of the expansion for 16-byte aligned matrices with m % 4 == 0: a CTA owns a
// 1024-column strip and walks down a band of rows; each thread keeps the Q rows of its four
// columns in registers, reads P rows as broadcasts, and touches Mat / grad / param / momentum
// with 16-byte accesses only (no per-element division).
template <int MODE, int R>
__device__ __forceinline__ void expand_rows_body(const float* __restrict__ P, const float* __restrict__ Q, int64_t n,
                                                 int64_t m, float* __restrict__ Mat, float* __restrict__ residual,
                                                 float* __restrict__ grad, int64_t N, float scale,
                                                 const SgdApply& apply, int rows_per_cta, int col_block,
                                                 int row_block) {
  const int64_t col = (int64_t(col_block) * 256 + threadIdx.x) * 4;
  if (col >= m) return;
  float q[4][R];
#pragma unroll
  for (int j = 0; j < 4; ++j)
#pragma unroll
    for (int c = 0; c < R; ++c) q[j][c] = Q[(col + j) * R + c];
  const int64_t r0 = int64_t(row_block) * rows_per_cta;
  const int64_t r1 = min(r0 + rows_per_cta, n);
  for (int64_t i = r0; i < r1; ++i) {
    float p[R];
#pragma unroll
    for (int c = 0; c < R; ++c) p[c] = __ldg(P + i * R + c);
    float a[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float acc = 0.f;
#pragma unroll
      for (int c = 0; c < R; ++c) acc += p[c] * q[j][c];
      a[j] = acc;
    }
    const int64_t e = i * m + col;
    float4* mp = reinterpret_cast<float4*>(Mat + e);
    if (MODE == 0) {
      *mp = make_float4(a[0], a[1], a[2], a[3]);
      if (e + 3 < N) {
        const float4 g = *reinterpret_cast<const float4*>(grad + e);
        *reinterpret_cast<float4*>(residual + e) = make_float4(g.x - a[0], g.y - a[1], g.z - a[2], g.w - a[3]);
        *reinterpret_cast<float4*>(grad + e) = make_float4(a[0], a[1], a[2], a[3]);
      } else {
        for (int j = 0; j < 4; ++j)
          if (e + j < N) {
            residual[e + j] = grad[e + j] - a[j];
            grad[e + j] = a[j];
          }
      }
    } else {
      const float4 mv = *mp;
      *mp = make_float4(mv.x - a[0], mv.y - a[1], mv.z - a[2], mv.w - a[3]);
      float g[4] = {a[0] * scale, a[1] * scale, a[2] * scale, a[3] * scale};
      if (MODE == 1) {
        if (e + 3 < N) {
          *reinterpret_cast<float4*>(grad + e) = make_float4(g[0], g[1], g[2], g[3]);
        } else {
          for (int j = 0; j < 4; ++j)
            if (e + j < N) grad[e + j] = g[j];
        }
      } else {
        if (e + 3 < N) {
          sgd_update4(apply, e, g);
        } else {
          for (int j = 0; j < 4; ++j)
            if (e + j < N) sgd_update(apply, e + j, g[j]);
        }
      }
    }
  }
}

template <int MODE, int R>
__global__ void __launch_bounds__(256)
expand_rows_kernel(const float* __restrict__ P, const float* __restrict__ Q, int64_t n, int64_t m,
                   float* __restrict__ Mat, float* __restrict__ residual, float* __restrict__ grad,
                   int64_t N, float scale, SgdApply apply, int rows_per_cta) {
  expand_rows_body<MODE, R>(P, Q, n, m, Mat, residual, grad, N, scale, apply, rows_per_cta, int(blockIdx.x),
                            int(blockIdx.y));
}

// The expand + SGD pass (mode 2) of every matrix of a step in one grid, for the same reason as the
// grouped projections: CTA u works on unit u (a 1024-column strip x a band of rows of one matrix).
constexpr int kExpandGroup = 32;
struct ExpandMat {
  const float* P;
  const float* Q;
  int64_t n, m, N;
  float* Mat;
  float* param;
  float* momentum;
  int unit_begin, col_blocks, rows_per;
};
struct GroupedExpand {
  int count;
  float scale;
  SgdApply apply;   // lr / momentum / weight decay / first_step shared; param and momentum per matrix
  ExpandMat mat[kExpandGroup];
};
template <int R>
__global__ void __launch_bounds__(256)
expand_rows_grouped_kernel(const __grid_constant__ GroupedExpand g) {
  int u = int(blockIdx.x), i = 0;
  while (i + 1 < g.count && u >= g.mat[i + 1].unit_begin) ++i;
  const ExpandMat& M = g.mat[i];
  u -= M.unit_begin;
  SgdApply apply = g.apply;
  apply.param = M.param;
  apply.momentum = M.momentum;
  expand_rows_body<2, R>(M.P, M.Q, M.n, M.m, M.Mat, nullptr, nullptr, M.N, g.scale, apply, M.rows_per,
                         u % M.col_blocks, u / M.col_blocks);
}

template <int MODE>
bool launch_expand_rows(const float* P, const float* Q, int64_t n, int64_t m, int r, float* Mat,
                        float* residual, float* grad, int64_t N, float scale, const SgdApply& apply,
                        cudaStream_t stream) {
  auto al = [](const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if ((m & 3) != 0 || !al(Mat) || !al(residual) || !al(grad) || !al(apply.param) || !al(apply.momentum))
    return false;
  const unsigned col_blocks = unsigned((m / 4 + 255) / 256);
  // enough CTAs for ~8 per SM, at least 8 rows each
  int64_t row_blocks = (148 * 8 + col_blocks - 1) / col_blocks;
  if (row_blocks > (n + 7) / 8) row_blocks = (n + 7) / 8;
  if (row_blocks < 1) row_blocks = 1;
  const int rows_per = int((n + row_blocks - 1) / row_blocks);
  const dim3 grid(col_blocks, unsigned((n + rows_per - 1) / rows_per), 1);
#define HP_EXPAND(RR) \
  expand_rows_kernel<MODE, RR><<<grid, 256, 0, stream>>>(P, Q, n, m, Mat, residual, grad, N, scale, apply, rows_per)
  switch (r) {
    case 1: HP_EXPAND(1); break;
    case 2: HP_EXPAND(2); break;
    case 4: HP_EXPAND(4); break;
    case 8: HP_EXPAND(8); break;
    default: return false;
  }
#undef HP_EXPAND
  return true;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// 2-D fp32 tensor map: `inner` contiguous elements per row, `outer` rows.
bool make_map(CUtensorMap* map, const float* base, int64_t inner, int64_t outer, int box_inner,
              int box_outer, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {cuuint64_t(inner), cuuint64_t(outer)};
  cuuint64_t strides[1] = {cuuint64_t(inner) * 4};
  cuuint32_t box[2] = {cuuint32_t(box_inner), cuuint32_t(box_outer)};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Pipeline shape of the tensor-core GEMM.  The default was chosen by measurement (see the
// kernel's profile); HIPRESS_PSGD_BK (32 | 64) and HIPRESS_PSGD_STAGES select another compiled
// shape for experiments.
struct GemmVariant {
  int bk, stages;
  size_t smem_bytes;
};
// Read on every call (two getenv look-ups per launch) so that a test or a probe can switch
// variants inside one process.
GemmVariant gemm_variant() {
  {
    int bk = 32, stages = 6;
    if (const char* e = std::getenv("HIPRESS_PSGD_BK")) bk = std::atoi(e);
    if (const char* e = std::getenv("HIPRESS_PSGD_STAGES")) stages = std::atoi(e);
    if (bk == 32 && stages == 6) return GemmVariant{32, 6, sizeof(GemmSmem<32, 6>)};
    if (bk == 32 && stages == 4) return GemmVariant{32, 4, sizeof(GemmSmem<32, 4>)};
    if (bk == 64 && stages == 3) return GemmVariant{64, 3, sizeof(GemmSmem<64, 3>)};
    if (bk == 64 && stages == 4) return GemmVariant{64, 4, sizeof(GemmSmem<64, 4>)};
    return GemmVariant{64, 6, sizeof(GemmSmem<64, 6>)};
  }
}

OwnerTargets owners_of(const ReduceTargets& red, int64_t rows) {
  OwnerTargets o{};
  o.world = red.world;
  for (int p = 0; p < red.world; ++p) o.dst[p] = red.dst[p];
  o.rows_per_owner = (rows + red.world - 1) / red.world;
  if (o.rows_per_owner < 1) o.rows_per_owner = 1;
  return o;
}

}  // namespace

int64_t psgd_kpad(int64_t k) { return (k + kKPad - 1) / kKPad * kKPad; }

bool psgd_tensor_core_eligible(const float* Mat, int64_t n, int64_t m) {
  return (reinterpret_cast<uintptr_t>(Mat) & 15) == 0 && (m % 4) == 0 && n >= 1 && m >= 1 &&
         encode_fn() != nullptr;
}

cudaError_t psgd_transpose_pad(const float* X, int64_t rows, int r, float* Xt, int64_t rows_pad,
                               cudaStream_t stream) {
  if (r < 1 || r > kBN || rows_pad < rows) return cudaErrorInvalidValue;
  int64_t blocks = (rows_pad + 255) / 256;
  if (blocks > 148 * 4) blocks = 148 * 4;
  transpose_pad_kernel<<<int(blocks), 256, 0, stream>>>(X, rows, r, Xt, rows_pad);
  return cudaGetLastError();
}

cudaError_t psgd_gemm(int mode, const float* Mat, int64_t n, int64_t m, const float* X,
                      const float* Xt, int r, const ReduceTargets& red, int force_simt, int* status,
                      cudaStream_t stream) {
  if (r < 1 || r > kBN || red.world < 1 || red.world > kMaxWorld || n < 1 || m < 1)
    return cudaErrorInvalidValue;
  const int64_t out_rows = mode == 0 ? n : m;
  const int64_t K = mode == 0 ? m : n;
  const OwnerTargets out = owners_of(red, out_rows);
  if (force_simt || Xt == nullptr || !psgd_tensor_core_eligible(Mat, n, m)) {
    if (mode == 0) {
      simt_gemm_p_kernel<<<unsigned((n + 7) / 8), 256, 0, stream>>>(Mat, X, n, m, r, out);
    } else {
      const int64_t col_blocks = (m + 255) / 256;
      int64_t chunks = (148 * 4 + col_blocks - 1) / col_blocks;
      if (chunks > (n + 15) / 16) chunks = (n + 15) / 16;
      if (chunks < 1) chunks = 1;
      const int64_t rows_per = (n + chunks - 1) / chunks;
      dim3 grid(unsigned(col_blocks), unsigned((n + rows_per - 1) / rows_per));
      simt_gemm_q_kernel<<<grid, 256, 0, stream>>>(Mat, X, n, m, r, rows_per, out);
    }
    return cudaGetLastError();
  }
  const int64_t k_pad = psgd_kpad(K);
  const GemmVariant var = gemm_variant();
  const int bk = var.bk;
  CUtensorMap map_a, map_b;
  const bool ok_a = mode == 0
                        ? make_map(&map_a, Mat, m, n, kBoxK, kBM, CU_TENSOR_MAP_SWIZZLE_128B)
                        : make_map(&map_a, Mat, m, n, 32, bk, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
  const bool ok_b = make_map(&map_b, Xt, k_pad, kBN, kBoxK, kBN, CU_TENSOR_MAP_SWIZZLE_128B);
  if (!ok_a || !ok_b) return cudaErrorInvalidValue;
  const int tiles = int((out_rows + kBM - 1) / kBM);
  const int total_kb = int(k_pad / bk);
  const size_t smem = var.smem_bytes + 1024;
  // As many CTAs as fit on the SMs at once (by shared memory): aim for one full wave, never
  // more, so that no partial second wave runs at low occupancy.
  int per_sm = int((227 * 1024) / smem);
  if (per_sm < 1) per_sm = 1;
  if (per_sm > 4) per_sm = 4;
  const int resident = 148 * per_sm;
  int splits = resident / tiles;
  const int max_splits = total_kb / 4 > 0 ? total_kb / 4 : 1;
  if (splits > max_splits) splits = max_splits;
  if (splits < 1) splits = 1;
  int kbps = (total_kb + splits - 1) / splits;
  splits = (total_kb + kbps - 1) / kbps;
  const dim3 grid(static_cast<unsigned>(tiles), static_cast<unsigned>(splits), 1);
#define HP_GEMM(MODE, BK, ST)                                                                                        \
  do {                                                                                                               \
    cudaError_t e = cudaFuncSetAttribute(psgd_gemm_kernel<MODE, BK, ST>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                         int(smem));                                                                 \
    if (e != cudaSuccess) return e;                                                                                  \
    psgd_gemm_kernel<MODE, BK, ST><<<grid, kGemmThreads, smem, stream>>>(map_a, map_b, Mat, n, m, out_rows, r,        \
                                                                         total_kb, kbps, out, status);               \
  } while (0)
#define HP_GEMM_MODE(BK, ST)           \
  do {                                 \
    if (mode == 0) HP_GEMM(0, BK, ST); \
    else HP_GEMM(1, BK, ST);           \
  } while (0)
  if (var.bk == 32 && var.stages == 6) HP_GEMM_MODE(32, 6);
  else if (var.bk == 32 && var.stages == 4) HP_GEMM_MODE(32, 4);
  else if (var.bk == 64 && var.stages == 3) HP_GEMM_MODE(64, 3);
  else if (var.bk == 64 && var.stages == 4) HP_GEMM_MODE(64, 4);
  else HP_GEMM_MODE(64, 6);
#undef HP_GEMM_MODE
#undef HP_GEMM
  return cudaGetLastError();
}

cudaError_t psgd_gemm_grouped(int mode, const PsgdGemmItem* items, int count, int r, int* status,
                              int* launches, cudaStream_t stream) {
  if (r < 1 || r > kBN || count < 0) return cudaErrorInvalidValue;
  const GemmVariant var = gemm_variant();
  const size_t smem = var.smem_bytes + 1024;
  int per_sm = int((227 * 1024) / smem);
  per_sm = per_sm < 1 ? 1 : (per_sm > 4 ? 4 : per_sm);
  const int resident = 148 * per_sm;

  struct Plan {
    int item;
    int tiles, total_kb, kbps, splits;
    double unit_bytes;
  };
  std::vector<Plan> plans;
  double total_bytes = 0;
  for (int i = 0; i < count; ++i) {
    const PsgdGemmItem& it = items[i];
    if (it.red.world < 1 || it.red.world > kMaxWorld || it.n < 1 || it.m < 1) return cudaErrorInvalidValue;
    if (it.Xt == nullptr || !psgd_tensor_core_eligible(it.Mat, it.n, it.m)) {
      const cudaError_t e = psgd_gemm(mode, it.Mat, it.n, it.m, it.X, it.Xt, r, it.red, 1, status, stream);
      if (e != cudaSuccess) return e;
      if (launches) ++*launches;
      continue;
    }
    const int64_t out_rows = mode == 0 ? it.n : it.m;
    const int64_t K = mode == 0 ? it.m : it.n;
    Plan pl{};
    pl.item = i;
    pl.tiles = int((out_rows + kBM - 1) / kBM);
    pl.total_kb = int(psgd_kpad(K) / var.bk);
    plans.push_back(pl);
    total_bytes += double(it.n) * double(it.m) * 4.0;
  }
  if (plans.empty()) return cudaSuccess;
  // Units of about equal size, one wave of resident CTAs in total where the row tiles allow it.
  const double target = total_bytes / double(resident);
  for (Plan& pl : plans) {
    const PsgdGemmItem& it = items[pl.item];
    const double bytes = double(it.n) * double(it.m) * 4.0;
    int64_t units = int64_t(bytes / target + 0.5);
    int splits = int(units / pl.tiles);
    const int max_splits = pl.total_kb / 4 > 0 ? pl.total_kb / 4 : 1;
    splits = splits < 1 ? 1 : (splits > max_splits ? max_splits : splits);
    pl.kbps = (pl.total_kb + splits - 1) / splits;
    pl.splits = (pl.total_kb + pl.kbps - 1) / pl.kbps;
    pl.unit_bytes = bytes / double(pl.tiles) / double(pl.splits);
  }
  // largest units first: the small ones fill the tail of the grid
  std::stable_sort(plans.begin(), plans.end(), [](const Plan& a, const Plan& b) { return a.unit_bytes > b.unit_bytes; });

  for (size_t base = 0; base < plans.size(); base += kGemmGroup) {
    GroupedGemm g{};
    g.count = int(std::min<size_t>(kGemmGroup, plans.size() - base));
    g.r = r;
    int units = 0;
    for (int j = 0; j < g.count; ++j) {
      const Plan& pl = plans[base + size_t(j)];
      const PsgdGemmItem& it = items[pl.item];
      GroupedMat& gm = g.mat[j];
      const int64_t out_rows = mode == 0 ? it.n : it.m;
      const int64_t K = mode == 0 ? it.m : it.n;
      const bool ok_a = mode == 0 ? make_map(&gm.map_a, it.Mat, it.m, it.n, kBoxK, kBM, CU_TENSOR_MAP_SWIZZLE_128B)
                                  : make_map(&gm.map_a, it.Mat, it.m, it.n, 32, var.bk,
                                             CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
      const bool ok_b = make_map(&gm.map_b, it.Xt, psgd_kpad(K), kBN, kBoxK, kBN, CU_TENSOR_MAP_SWIZZLE_128B);
      if (!ok_a || !ok_b) return cudaErrorInvalidValue;
      gm.Mat = it.Mat;
      gm.n = it.n;
      gm.m = it.m;
      gm.out_rows = out_rows;
      gm.out = owners_of(it.red, out_rows);
      gm.unit_begin = units;
      gm.tiles = pl.tiles;
      gm.kbps = pl.kbps;
      gm.total_kb = pl.total_kb;
      units += pl.tiles * pl.splits;
    }
#define HP_GROUPED(MODE, BK, ST)                                                                        \
  do {                                                                                                  \
    cudaError_t e = cudaFuncSetAttribute(psgd_gemm_grouped_kernel<MODE, BK, ST>,                        \
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));      \
    if (e != cudaSuccess) return e;                                                                     \
    psgd_gemm_grouped_kernel<MODE, BK, ST><<<unsigned(units), kGemmThreads, smem, stream>>>(g, status); \
  } while (0)
#define HP_GROUPED_MODE(BK, ST)           \
  do {                                    \
    if (mode == 0) HP_GROUPED(0, BK, ST); \
    else HP_GROUPED(1, BK, ST);           \
  } while (0)
    if (var.bk == 32 && var.stages == 6) HP_GROUPED_MODE(32, 6);
    else if (var.bk == 32 && var.stages == 4) HP_GROUPED_MODE(32, 4);
    else if (var.bk == 64 && var.stages == 3) HP_GROUPED_MODE(64, 3);
    else if (var.bk == 64 && var.stages == 4) HP_GROUPED_MODE(64, 4);
    else HP_GROUPED_MODE(64, 6);
#undef HP_GROUPED_MODE
#undef HP_GROUPED
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    if (launches) ++*launches;
  }
  return cudaSuccess;
}

// ---------------------------------------------------------------- batched small kernels
// A model has tens of matrices and each needs the same handful of tiny kernels per step
// (operand transposes, factor gathers, orthonormalisation).  Launched one by one they cost a
// few microseconds each with the device idle in between; here one launch covers up to
// kPsgdBatch matrices, their descriptors travelling in the kernel's parameter space.
namespace {

struct TransposeBatch {
  int count;
  PsgdTransposeItem item[kPsgdBatch];
};
__global__ void __launch_bounds__(256)
transpose_pad_batched_kernel(TransposeBatch b) {
  const PsgdTransposeItem it = b.item[blockIdx.y];
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < it.rows_pad; i += stride) {
#pragma unroll
    for (int c = 0; c < kBN; ++c)
      it.Xt[c * it.rows_pad + i] = (i < it.rows && c < it.r) ? it.X[i * it.r + c] : 0.0f;
  }
}

struct GatherBatch {
  int count, world;
  float scale;
  PsgdGatherItem item[kPsgdBatch];
};
__global__ void __launch_bounds__(256)
owner_gather_batched_kernel(GatherBatch b) {
  const PsgdGatherItem& it = b.item[blockIdx.y];
  const int64_t total = it.rows * it.r;
  int64_t rpo = (it.rows + b.world - 1) / b.world;
  if (rpo < 1) rpo = 1;
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; e < total; e += stride) {
    int owner = int((e / it.r) / rpo);
    if (owner >= b.world) owner = b.world - 1;
    it.out[e] = it.src[owner][e] * b.scale;
  }
}

struct GsBatch {
  int count;
  float eps;
  PsgdGsItem item[kPsgdBatch];
};
__global__ void __launch_bounds__(kGsThreads)
gram_schmidt_batched_kernel(GsBatch b) {
  __shared__ float sh[kGsThreads / 32];
  const PsgdGsItem it = b.item[blockIdx.x];
  float* P = it.P;
  const int64_t n = it.n;
  const int r = it.r;
  for (int j = 0; j < r; ++j) {
    float ss = 0.f;
    for (int64_t i = threadIdx.x; i < n; i += kGsThreads) {
      const float v = P[i * r + j];
      ss += v * v;
    }
    const float inv = 1.0f / (sqrtf(block_sum(ss, sh)) + b.eps);
    for (int64_t i = threadIdx.x; i < n; i += kGsThreads) P[i * r + j] *= inv;
    __syncthreads();
    for (int c = j + 1; c < r; ++c) {
      float dot = 0.f;
      for (int64_t i = threadIdx.x; i < n; i += kGsThreads) dot += P[i * r + j] * P[i * r + c];
      dot = block_sum(dot, sh);
      for (int64_t i = threadIdx.x; i < n; i += kGsThreads) P[i * r + c] -= dot * P[i * r + j];
      __syncthreads();
    }
  }
}

}  // namespace

cudaError_t psgd_transpose_pad_batched(const PsgdTransposeItem* items, int count, cudaStream_t stream) {
  for (int base = 0; base < count; base += kPsgdBatch) {
    TransposeBatch b{};
    b.count = count - base < kPsgdBatch ? count - base : kPsgdBatch;
    int64_t max_rows = 1;
    for (int i = 0; i < b.count; ++i) {
      b.item[i] = items[base + i];
      if (b.item[i].r < 1 || b.item[i].r > kBN || b.item[i].rows_pad < b.item[i].rows) return cudaErrorInvalidValue;
      if (b.item[i].rows_pad > max_rows) max_rows = b.item[i].rows_pad;
    }
    int64_t gx = (max_rows + 255) / 256;
    if (gx > 148) gx = 148;
    transpose_pad_batched_kernel<<<dim3(unsigned(gx), unsigned(b.count), 1), 256, 0, stream>>>(b);
  }
  return cudaGetLastError();
}

cudaError_t psgd_owner_gather_batched(const PsgdGatherItem* items, int count, int world, float scale,
                                      cudaStream_t stream) {
  if (world < 1 || world > kMaxWorld) return cudaErrorInvalidValue;
  for (int base = 0; base < count; base += kPsgdBatch) {
    GatherBatch b{};
    b.count = count - base < kPsgdBatch ? count - base : kPsgdBatch;
    b.world = world;
    b.scale = scale;
    int64_t max_total = 1;
    for (int i = 0; i < b.count; ++i) {
      b.item[i] = items[base + i];
      const int64_t t = b.item[i].rows * b.item[i].r;
      if (t > max_total) max_total = t;
    }
    int64_t gx = (max_total + 255) / 256;
    if (gx > 148) gx = 148;
    owner_gather_batched_kernel<<<dim3(unsigned(gx), unsigned(b.count), 1), 256, 0, stream>>>(b);
  }
  return cudaGetLastError();
}

cudaError_t gram_schmidt_batched(const PsgdGsItem* items, int count, float eps, cudaStream_t stream) {
  for (int base = 0; base < count; base += kPsgdBatch) {
    GsBatch b{};
    b.count = count - base < kPsgdBatch ? count - base : kPsgdBatch;
    b.eps = eps;
    for (int i = 0; i < b.count; ++i) {
      b.item[i] = items[base + i];
      if (b.item[i].n < 1 || b.item[i].r < 1 || b.item[i].r > kBN) return cudaErrorInvalidValue;
    }
    gram_schmidt_batched_kernel<<<b.count, kGsThreads, 0, stream>>>(b);
  }
  return cudaGetLastError();
}

cudaError_t gram_schmidt(float* P, int64_t n, int r, float eps, cudaStream_t stream) {
  if (n < 1 || r < 1 || r > kBN) return cudaErrorInvalidValue;
  gram_schmidt_kernel<<<1, kGsThreads, 0, stream>>>(P, n, r, eps);
  return cudaGetLastError();
}

cudaError_t psgd_expand_residual(const float* P, const float* Q, int64_t n, int64_t m, int r,
                                 float* Mat, float* residual, float* grad, int64_t N, int mode,
                                 float post_scale, cudaStream_t stream) {
  if (n < 1 || m < 1 || r < 1 || r > kBN || N > n * m) return cudaErrorInvalidValue;
  if (mode == 0 ? launch_expand_rows<0>(P, Q, n, m, r, Mat, residual, grad, N, post_scale, SgdApply{}, stream)
                : launch_expand_rows<1>(P, Q, n, m, r, Mat, residual, grad, N, post_scale, SgdApply{}, stream))
    return cudaGetLastError();
  int64_t blocks = (n * m + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (mode == 0)
    expand_kernel<0><<<int(blocks), 256, 0, stream>>>(P, Q, n, m, r, Mat, residual, grad, N, post_scale, SgdApply{});
  else
    expand_kernel<1><<<int(blocks), 256, 0, stream>>>(P, Q, n, m, r, Mat, residual, grad, N, post_scale, SgdApply{});
  return cudaGetLastError();
}

cudaError_t psgd_expand_sgd(const float* P, const float* Q, int64_t n, int64_t m, int r, float* Mat,
                            int64_t N, float post_scale, const SgdApply& apply, cudaStream_t stream) {
  if (n < 1 || m < 1 || r < 1 || r > kBN || N > n * m || apply.param == nullptr ||
      apply.momentum == nullptr)
    return cudaErrorInvalidValue;
  if (launch_expand_rows<2>(P, Q, n, m, r, Mat, nullptr, nullptr, N, post_scale, apply, stream))
    return cudaGetLastError();
  int64_t blocks = (n * m + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  expand_kernel<2><<<int(blocks), 256, 0, stream>>>(P, Q, n, m, r, Mat, nullptr, nullptr, N, post_scale, apply);
  return cudaGetLastError();
}

cudaError_t psgd_expand_sgd_grouped(const PsgdExpandItem* items, int count, int r, float post_scale,
                                    const SgdApply& common, int* launches, cudaStream_t stream) {
  if (count < 0 || r < 1 || r > kBN) return cudaErrorInvalidValue;
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  struct Plan {
    int item, col_blocks, rows_per, row_blocks;
    double unit_elems;
  };
  std::vector<Plan> plans;
  double total = 0;
  for (int i = 0; i < count; ++i) {
    const PsgdExpandItem& it = items[i];
    if (it.n < 1 || it.m < 1 || it.N > it.n * it.m || it.param == nullptr || it.momentum == nullptr)
      return cudaErrorInvalidValue;
    const bool rows_form = (it.m & 3) == 0 && al(it.Mat) && al(it.param) && al(it.momentum) &&
                           (r == 1 || r == 2 || r == 4 || r == 8);
    if (!rows_form) {
      SgdApply a = common;
      a.param = it.param;
      a.momentum = it.momentum;
      const cudaError_t e = psgd_expand_sgd(it.P, it.Q, it.n, it.m, r, it.Mat, it.N, post_scale, a, stream);
      if (e != cudaSuccess) return e;
      if (launches) ++*launches;
      continue;
    }
    Plan pl{};
    pl.item = i;
    pl.col_blocks = int((it.m / 4 + 255) / 256);
    plans.push_back(pl);
    total += double(it.n) * double(it.m);
  }
  if (plans.empty()) return cudaSuccess;
  const double target_ctas = 148.0 * 8.0;
  for (Plan& pl : plans) {
    const PsgdExpandItem& it = items[pl.item];
    const double share = double(it.n) * double(it.m) / total * target_ctas;
    int64_t row_blocks = int64_t(share / double(pl.col_blocks) + 0.5);
    const int64_t most = (it.n + 7) / 8;
    row_blocks = row_blocks < 1 ? 1 : (row_blocks > most ? most : row_blocks);
    pl.rows_per = int((it.n + row_blocks - 1) / row_blocks);
    pl.row_blocks = int((it.n + pl.rows_per - 1) / pl.rows_per);
    pl.unit_elems = double(pl.rows_per) * double(it.m < 1024 ? it.m : 1024);
  }
  std::stable_sort(plans.begin(), plans.end(), [](const Plan& a, const Plan& b) { return a.unit_elems > b.unit_elems; });
  for (size_t base = 0; base < plans.size(); base += kExpandGroup) {
    GroupedExpand g{};
    g.count = int(std::min<size_t>(kExpandGroup, plans.size() - base));
    g.scale = post_scale;
    g.apply = common;
    int units = 0;
    for (int j = 0; j < g.count; ++j) {
      const Plan& pl = plans[base + size_t(j)];
      const PsgdExpandItem& it = items[pl.item];
      ExpandMat& em = g.mat[j];
      em.P = it.P;
      em.Q = it.Q;
      em.n = it.n;
      em.m = it.m;
      em.N = it.N;
      em.Mat = it.Mat;
      em.param = it.param;
      em.momentum = it.momentum;
      em.unit_begin = units;
      em.col_blocks = pl.col_blocks;
      em.rows_per = pl.rows_per;
      units += pl.col_blocks * pl.row_blocks;
    }
    switch (r) {
      case 1: expand_rows_grouped_kernel<1><<<unsigned(units), 256, 0, stream>>>(g); break;
      case 2: expand_rows_grouped_kernel<2><<<unsigned(units), 256, 0, stream>>>(g); break;
      case 4: expand_rows_grouped_kernel<4><<<unsigned(units), 256, 0, stream>>>(g); break;
      default: expand_rows_grouped_kernel<8><<<unsigned(units), 256, 0, stream>>>(g); break;
    }
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    if (launches) ++*launches;
  }
  return cudaSuccess;
}

namespace {
struct GatherSrc {
  const float* p[kMaxWorld];
};
// out[row] = scale * (owner of row)'s accumulator[row]: the all-gather half of
// the factor all-reduce; owners may be peer GPUs (plain peer loads).
__global__ void __launch_bounds__(256)
owner_gather_kernel(GatherSrc src, int world, int64_t rows, int r, int64_t rows_per_owner,
                    float* __restrict__ out, float scale) {
  const int64_t total = rows * r;
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; e < total; e += stride) {
    int owner = int((e / r) / rows_per_owner);
    if (owner >= world) owner = world - 1;
    out[e] = src.p[owner][e] * scale;
  }
}
}  // namespace

cudaError_t psgd_owner_gather(const ReduceTargets& owners, int64_t rows, int r, float* out,
                              float scale, cudaStream_t stream) {
  if (owners.world < 1 || owners.world > kMaxWorld || rows < 1 || r < 1) return cudaErrorInvalidValue;
  GatherSrc src{};
  for (int p = 0; p < owners.world; ++p) src.p[p] = owners.dst[p];
  int64_t rpo = (rows + owners.world - 1) / owners.world;
  if (rpo < 1) rpo = 1;
  int64_t blocks = (rows * r + 255) / 256;
  if (blocks > 148 * 4) blocks = 148 * 4;
  owner_gather_kernel<<<int(blocks), 256, 0, stream>>>(src, owners.world, rows, r, rpo, out, scale);
  return cudaGetLastError();
}

}  // namespace cuda
}  // namespace hipress
