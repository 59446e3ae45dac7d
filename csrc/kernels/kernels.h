// Launch API of the sm_100a kernels.  Plain C++ over raw device pointers and a
// stream: no torch types here, so the .cu files compile in seconds and the
// same launchers serve the torch bindings, the task runtime and the C ABI.
//
// Every compressing kernel can deliver its payload to up to kMaxWorld
// destinations at once (`PushTargets`): the local output buffer and/or the
// receive slots of peer GPUs mapped into this process (NVLink peer memory).
// After the last CTA has stored its bytes, one thread publishes an epoch-valued
// flag to every destination with a system-scope release store.  Receivers wait
// on those flags with `wait_flags` (bounded) and then decode all ranks'
// payloads in a single pass over the dense tensor (`*_unpack_accum`).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace hipress {
namespace cuda {

constexpr int kMaxWorld = 8;

// Where a compressing kernel stores its payload.
//   payload[p]  start of the payload in destination p (local or peer memory)
//   flag[p]     flag word of destination p to publish `epoch` to; may be null
//   done        device counter used to elect the last CTA; must be zero on
//               entry, is reset to zero by the kernel
//
// Steps replayed from a CUDA graph cannot change kernel arguments, so the step's epoch may live
// on the device instead: when epoch_dev is set, the kernel reads the epoch from it, `payload`
// holds the addresses for even epochs and odd epochs use the slots parity_stride bytes further
// (slots are double-buffered by epoch parity), and codecs with a rounding seed add
// epoch * kEpochSeedStride to it.
struct PushTargets {
  int world = 0;
  uint8_t* payload[kMaxWorld] = {};
  uint32_t* flag[kMaxWorld] = {};
  uint32_t epoch = 0;
  unsigned int* done = nullptr;
  const uint32_t* epoch_dev = nullptr;
  int64_t parity_stride = 0;
  int64_t parity_off = 0;  // set on the device by resolve_epoch(): 0 or parity_stride
  // A single destination is normally this GPU's own slot (device-scope fences are enough);
  // set when the single destination is a peer, so that the payload is fenced at system scope.
  int remote = 0;
  // Scatter mode (sharded exchange, > 0): the tensor is cut into shards of shard_elems elements
  // (a multiple of 2048); shard j is compressed as a payload of its own -- own header, byte
  // indices and rounding seed (seed + j * kShardSeedStride) -- and stored into payload[j] only.
  // Flags of all `world` destinations are published once the whole grid is done.
  int64_t shard_elems = 0;
  // Device status word: when set and non-zero on entry (an earlier wait of this step timed out
  // or a payload was malformed) the kernel returns without storing or publishing anything.
  const int* guard = nullptr;
  // NVLS: multicast address of the payload (the same offset of every destination's buffer).
  // When set, aligned 4- and 16-byte payload stores are issued once with multimem.st instead of
  // once per destination; smaller stores and the flags stay unicast.
  uint8_t* mc = nullptr;
};
constexpr uint64_t kEpochSeedStride = 0x9E3779B97F4A7C15ull;
constexpr uint64_t kShardSeedStride = 0xD6E8FEB86659FD93ull;

// Payloads of all ranks as seen by the receiver, in canonical (ascending rank)
// accumulation order.
struct UnpackSources {
  int world = 0;
  const uint8_t* payload[kMaxWorld] = {};
  int64_t payload_bytes[kMaxWorld] = {};  // capacity of each slot (bounds checks)
  const uint32_t* epoch_dev = nullptr;    // see PushTargets
  int64_t parity_stride = 0;
  int64_t parity_off = 0;                 // set on the device by resolve_epoch()
  // Concatenation mode (sharded exchange, > 0; a multiple of 2048): the dense tensor is the
  // concatenation of `world` shards of shard_elems elements and payload[j] encodes shard j
  // alone, so every element is decoded from exactly one payload (nothing is summed).
  int64_t shard_elems = 0;
  // Device status word: when set and non-zero on entry the kernel returns without writing (a
  // wait earlier in the step timed out, or a payload was malformed: the slots may hold stale or
  // partial bytes, and parameters, momentum and residuals must stay as they are).
  const int* guard = nullptr;
};

// Optional fused SGD-with-momentum update applied to the decoded, averaged
// gradient g:  g += wd * p;  buf = mu * buf + g;  p -= lr * buf.
struct SgdApply {
  float* param = nullptr;  // null -> no update, only the dense gradient is written
  float* momentum = nullptr;
  float lr = 0.f, mu = 0.f, weight_decay = 0.f;
  int first_step = 0;  // buf = g on the first step (torch.optim.SGD semantics)
  // The caller does not keep the dense gradient: the kernel that applies the update writes
  // zeros where it would have written the gradient, which leaves the buffer ready for the next
  // backward pass and saves the separate clearing pass.
  int clear_grad = 0;
  const int* guard = nullptr;  // see UnpackSources::guard (checked by sgd_apply_dense)
};

// Error codes written to a device status word by bounded waits / bounds checks.
enum Status : int {
  kOk = 0,
  kFlagTimeout = 1,    // a peer's flag did not reach the epoch in time
  kPayloadBounds = 2,  // a header describes more bytes / elements than the slot holds
  kBadHeader = 3,
};

// ---------------------------------------------------------------- TBQ
// grad and residual hold n floats; each payload destination ceil(n/4) bytes.
cudaError_t tbq_compress(const float* grad, float* residual, int64_t n, float threshold,
                         const PushTargets& dst, cudaStream_t stream);
// out[i] = sum_r decode(payload_r)[i] (+ out[i] if add), times post_scale when != 1.
cudaError_t tbq_unpack_accum(const UnpackSources& src, float threshold, float* out, int64_t n,
                             int add, float post_scale, const SgdApply& apply,
                             cudaStream_t stream);

// ---------------------------------------------------------------- TernGrad
// Scratch needed by terngrad_compress / ecq_compress (bytes).
size_t minmax_scratch_bytes();
// residual may be null.  With a residual, the tensor quantised is grad+residual
// and residual receives the quantisation error.  scratch must be zero before
// its first use and is left ready for the next call.
cudaError_t terngrad_compress(const float* grad, float* residual, int64_t n, int bitwidth,
                              int enable_random, uint64_t seed, const PushTargets& dst,
                              void* scratch, cudaStream_t stream);
// Element count per payload is taken from its header and must equal n; all
// payloads must carry the same bitwidth (kBadHeader otherwise).  bitwidth_hint
// (0 = unknown) lets the launcher size the decode table for that bitwidth; a
// payload with another bitwidth is then rejected.
cudaError_t terngrad_unpack_accum(const UnpackSources& src, float* out, int64_t n, int add,
                                  float post_scale, const SgdApply& apply, int* status,
                                  cudaStream_t stream, int bitwidth_hint = 0);

// ---------------------------------------------------------------- ECQ
cudaError_t ecq_compress(const float* grad, float* history, int64_t n, float alpha, float beta,
                         int bitwidth, uint64_t seed, const PushTargets& dst, void* scratch,
                         cudaStream_t stream);
cudaError_t ecq_unpack_accum(const UnpackSources& src, float* out, int64_t n, int add,
                             float post_scale, int* status, cudaStream_t stream);

// ---------------------------------------------------------------- sparse top-k
size_t sparse_scratch_bytes(int64_t n);
// accumulate != 0: R += grad first (GradDrop); else grad is ignored (DGC).
// Each destination needs 4 + 8*ceil(n*keep_fraction) bytes.
cudaError_t sparse_compress(const float* grad, float* R, int64_t n, double sample_rate,
                            double keep_fraction, uint64_t seed, int accumulate,
                            const PushTargets& dst, void* scratch, cudaStream_t stream);
// The same compressor with the codec's state update fused into its one pass over the tensor.
//   mode 0  plain: select from R as it is (DGC without momentum correction)
//   mode 1  GradDrop: R += grad, then select from R
//   mode 2  DGC with momentum correction: u = momentum*u + s*grad; R (the velocity v) += u; select
//           from v; u and v are cleared at the sent positions (momentum factor masking).  s clips
//           the bucket's gradient to norm `clip` (> 0; sumsq: one float of scratch, zero on entry,
//           left zero).  zero_grad leaves zeros in grad: the dense gradient is rebuilt from the
//           payloads afterwards, which saves the separate clearing pass.
// For keep fractions up to 1 % the tensor is read once ("list form", see sparse.cu); otherwise,
// or when the scratch cannot hold the expected candidates, the multi-pass scan form runs.
// scratch: sparse_scratch_bytes(n) bytes, zero before its first use.
struct SparseFuse {
  int mode = 0;
  const float* grad = nullptr;
  float* u = nullptr;
  float momentum = 0.f, clip = 0.f;
  const float* sumsq = nullptr;
  int zero_grad = 0;
};
cudaError_t sparse_compress_fused(const SparseFuse& fuse, float* R, int64_t n, double sample_rate,
                                  double keep_fraction, uint64_t seed, const PushTargets& dst, void* scratch,
                                  cudaStream_t stream);
// {elements emitted, candidates over the sampled threshold (list form), threshold as float bits,
// candidates dropped so far for lack of pool space} of the last call on `scratch`; asynchronous
// copies to host4 on `stream`.
cudaError_t sparse_read_stats(const void* scratch, unsigned int* host4, cudaStream_t stream);
// add == 0 zero-fills out first.  Payloads are applied one after another in
// rank order so that the fp32 sum is reproducible on every replica.
cudaError_t sparse_unpack_accum(const UnpackSources& src, float* out, int64_t n, int add,
                                float post_scale, int* status, cudaStream_t stream);

// out[idx] = 0 for every index of every payload (one launch): after the optimizer has consumed a
// dense gradient that only held scattered payload entries, this leaves it all zero again
// without a pass over the whole buffer.
cudaError_t sparse_clear(const UnpackSources& src, float* out, int64_t n, cudaStream_t stream);

// ---------------------------------------------------------------- flags
// Spins (one warp) until flag[r] >= epoch for all r < world, or timeout_ns
// passes; on timeout writes kFlagTimeout to *status and returns normally.
// wait_stats (optional): three 64-bit device counters the kernel adds to -- {nanoseconds spent
// waiting, longest single wait in ns, number of waits} -- so that time lost to slower peers can
// be told apart from time spent computing, also when the step is replayed from a CUDA graph.
cudaError_t wait_flags(const uint32_t* flags, int world, uint32_t epoch, uint64_t timeout_ns,
                       int* status, cudaStream_t stream, const uint32_t* epoch_dev = nullptr,
                       unsigned long long* wait_stats = nullptr);
// *slot = device wall clock (globaltimer, ns): a one-thread kernel that marks a point of a stream.
cudaError_t stamp_time(unsigned long long* slot, cudaStream_t stream);
// *epoch_dev += 1: first kernel of a step whose epoch lives on the device (see PushTargets).
cudaError_t bump_epoch(uint32_t* epoch_dev, cudaStream_t stream);
// Publishes `epoch` to flag[p] of every destination (release, system scope).
cudaError_t signal_flags(const PushTargets& dst, cudaStream_t stream);

// ---------------------------------------------------------------- dense helpers
// Fused SGD-momentum over flat buffers (used for 1-D parameters and for the
// uncompressed baseline path).
cudaError_t sgd_apply_dense(float* grad, float scale, const SgdApply& apply, int64_t n,
                            cudaStream_t stream);
// out = a + b (fp32), n elements.
cudaError_t add_into(const float* a, const float* b, float* out, int64_t n, cudaStream_t stream);
// Sum of W dense fp32 buffers (peer pointers) into out: the P2P dense
// all-reduce used for small PowerSGD factors and 1-D parameters.
// With epoch_dev the sources are the slots of even epochs; odd epochs read parity_elems floats
// further.  guard: see UnpackSources::guard.
cudaError_t dense_gather_sum(const float* const* srcs, int world, float* out, int64_t n,
                             float post_scale, cudaStream_t stream, const uint32_t* epoch_dev = nullptr,
                             int64_t parity_elems = 0, const int* guard = nullptr);
// slot_even + (epoch odd ? parity_elems : 0) = src: staging copy of the dense codec when the
// step's epoch lives on the device (a captured step cannot change a copy's destination).
cudaError_t dense_stage(const float* src, float* slot_even, int64_t parity_elems, const uint32_t* epoch_dev,
                        int64_t n, cudaStream_t stream);

// ---------------------------------------------------------------- DGC / AdamW
// Momentum correction: u = momentum*u + s*grad; v += u, where s clips the
// bucket's gradient to norm `clip` (no clipping when clip <= 0).
// sumsq_scratch: one float, zero on entry when clip > 0; cleared by dgc_mask.
cudaError_t dgc_accumulate(const float* grad, float* u, float* v, int64_t n, float momentum,
                           float clip, float* sumsq_scratch, cudaStream_t stream);
// out += sum of g[i]^2 (out: one float, not cleared here).
cudaError_t dgc_sumsq(const float* g, int64_t n, float* out, cudaStream_t stream);
// Momentum factor masking: u[idx] = 0 for every index in the sparse payload.
cudaError_t dgc_mask(const uint8_t* payload, int64_t payload_capacity, float* u, int64_t n,
                     float* sumsq_scratch, cudaStream_t stream, const uint32_t* epoch_dev = nullptr,
                     int64_t parity_stride = 0);
struct AdamWApply {
  float* param = nullptr;
  float* exp_avg = nullptr;
  float* exp_avg_sq = nullptr;
  float lr = 0.f, beta1 = 0.9f, beta2 = 0.999f, eps = 1e-8f, weight_decay = 0.f;
  int step = 1;  // 1-based
  int clear_grad = 0;  // write zeros over grad after reading it (see SgdApply::clear_grad)
  const uint32_t* step_dev = nullptr;  // when set, the step count is read from the device (graph replays)
  const int* guard = nullptr;          // see UnpackSources::guard
};
// Fused AdamW (decoupled weight decay, bias correction) on g = scale*grad.
cudaError_t adamw_apply_dense(float* grad, float scale, const AdamWApply& apply, int64_t n,
                              cudaStream_t stream);

// ---------------------------------------------------------------- batch normalisation
// Training-mode batch norm over channels-last bf16 activations ([rows][channels], rows =
// batch x height x width), fused with an optional residual add and ReLU.  channels/8 must be a
// power of two up to 32 or a multiple of 32 (bn_supported).  Scratch owned by the caller:
// partial = 2*bn_partial_elems floats.
constexpr int kBnMaxRowBlocks = 1184;
bool bn_supported(int64_t rows, int channels);
int64_t bn_partial_elems(int64_t rows, int channels);
// y = act(bn(x) [+ residual]); writes mean, invstd, ab = (gamma*invstd, beta - mean*gamma*invstd)
// per channel and updates the running statistics (unbiased variance) when given.
cudaError_t bn_forward(const void* x, const void* residual, void* y, int64_t rows, int channels,
                       const float* gamma, const float* beta, float* running_mean, float* running_var,
                       long long* num_batches, float momentum, float eps, int relu, float* mean,
                       float* invstd, float* ab, float* partial, cudaStream_t stream);
// dy' = relu ? dy*(y > 0) : dy.  dx = d loss / d x; dres (optional) = dy'; dgamma, dbeta fp32;
// coef = 4*channels floats of scratch.
cudaError_t bn_backward(const void* dy, const void* x, const void* y, void* dx, void* dres, int64_t rows,
                        int channels, const float* gamma, const float* mean, const float* invstd,
                        int relu, float* dgamma, float* dbeta, float* coef, float* partial,
                        cudaStream_t stream);

// ---------------------------------------------------------------- bias + ReLU (+ 2x2 max pool)
// Convolution epilogue over channels-last bf16 [n][h][w][c]; c as for batch norm.  With pool,
// h and w must be even, y is [n][h/2][w/2][c] and idx holds the arg max (0..3 = 2*row + column)
// per output element.  partial = bias_relu_partial_elems(output rows, c) floats of scratch.
bool bias_relu_supported(int64_t rows, int channels);
int64_t bias_relu_partial_elems(int64_t rows, int channels);
cudaError_t bias_relu_forward(const void* x, const float* bias, void* y, uint8_t* idx, int n, int h, int w,
                              int channels, int pool, cudaStream_t stream);
// out[c] = sum over rows of dy[row][c] (bf16 in, fp32 out): the bias gradient of a linear layer.
// partial = bias_relu_partial_elems(rows, c) floats of scratch.
cudaError_t colsum_bf16(const void* dy, float* out, float* partial, int64_t rows, int channels,
                        cudaStream_t stream);
// dz [n][h][w][c] = gradient w.r.t. the convolution output, dbias [c] fp32.
cudaError_t bias_relu_backward(const void* dy, const void* y, const uint8_t* idx, void* dz, float* dbias,
                               float* partial, int n, int h, int w, int channels, int pool,
                               cudaStream_t stream);

// ---------------------------------------------------------------- residual add + LayerNorm
// Rows of `hidden` bf16 features (hidden % 8 == 0, <= 2048), gamma / beta fp32.
//   forward:  z = bf16(x + delta) (written when delta is given; otherwise z = x), y = LN(z);
//             mean / rstd: one fp32 value per row, for backward.
//   backward: dz (= gradient of x and of delta), dgamma, dbeta; partial = add_ln_partial_elems floats.
bool add_ln_supported(int64_t rows, int hidden);
int64_t add_ln_partial_elems(int64_t rows, int hidden);
cudaError_t add_ln_forward(const void* x, const void* delta, const float* gamma, const float* beta, void* y,
                           void* z, float* mean, float* rstd, int64_t rows, int hidden, float eps,
                           cudaStream_t stream);
cudaError_t add_ln_backward(const void* dy, const void* z, const float* mean, const float* rstd,
                            const float* gamma, void* dz, float* dgamma, float* dbeta, float* partial,
                            int64_t rows, int hidden, cudaStream_t stream);

// ---------------------------------------------------------------- max pooling
// 3x3, stride 2, padding 1 over channels-last bf16 [n][h][w][c] (c a multiple of 8).  The forward
// writes y [n][ho][wo][c] (ho = (h-1)/2 + 1) and one byte per output element: the winning window
// position kh*3 + kw.  The backward gathers, without atomics.
cudaError_t maxpool3x3s2_forward(const void* x, void* y, uint8_t* idx, int n, int h, int w, int c,
                                 cudaStream_t stream);
cudaError_t maxpool3x3s2_backward(const void* dy, const uint8_t* idx, void* dx, int n, int h, int w, int c,
                                  cudaStream_t stream);

// ---------------------------------------------------------------- PowerSGD
// All matrices row-major fp32.  Mat is n x m, P is n x r, Q is m x r, r <= 16.
// Output rows are split evenly over `world` owners; each row of the product is
// *added* into its owner's buffer (which has the full output shape and must be
// zero beforehand).  world == 1 means plain local accumulation.
struct ReduceTargets {
  int world = 1;
  float* dst[kMaxWorld] = {};
};
// K extent rounded up to the GEMM's K tile.
int64_t psgd_kpad(int64_t k);
// True when Mat can be described by a TMA tensor map (16-byte aligned base and
// row pitch) so that the tcgen05 path applies.
bool psgd_tensor_core_eligible(const float* Mat, int64_t n, int64_t m);
// X[rows x r] -> Xt[16][rows_pad] (transposed, zero padded): the K-major B
// operand of the tensor-core GEMM.  rows_pad = psgd_kpad(rows).
cudaError_t psgd_transpose_pad(const float* X, int64_t rows, int r, float* Xt, int64_t rows_pad,
                               cudaStream_t stream);
// mode 0: out[n x r] += Mat * X (X = Q, m x r);  mode 1: out[m x r] += Mat^T * X (X = P, n x r).
// Xt is psgd_transpose_pad(X); when it is null, force_simt is set, or Mat is
// not TMA-eligible the SIMT kernel runs instead of tcgen05.
cudaError_t psgd_gemm(int mode, const float* Mat, int64_t n, int64_t m, const float* X,
                      const float* Xt, int r, const ReduceTargets& red, int force_simt, int* status,
                      cudaStream_t stream);
// The same projection for a list of matrices in as few launches as possible (one per 24
// tensor-core-eligible matrices; the others fall back to psgd_gemm one by one).
struct PsgdGemmItem {
  const float* Mat = nullptr;
  int64_t n = 0, m = 0;
  const float* X = nullptr;    // [K x r]
  const float* Xt = nullptr;   // [16 x psgd_kpad(K)], or null: SIMT fallback
  ReduceTargets red;
};
cudaError_t psgd_gemm_grouped(int mode, const PsgdGemmItem* items, int count, int r, int* status,
                              int* launches, cudaStream_t stream);
// In-place modified Gram-Schmidt of the n x r matrix P (r <= 16).
cudaError_t gram_schmidt(float* P, int64_t n, int r, float eps, cudaStream_t stream);
// approx = P Q^T.  mode 0 (API parity): Mat = approx; residual = grad - Mat[:N]; grad = Mat[:N].
// mode 1 (error feedback in place): grad[:N] = post_scale * approx; Mat -= approx.
cudaError_t psgd_expand_residual(const float* P, const float* Q, int64_t n, int64_t m, int r,
                                 float* Mat, float* residual, float* grad, int64_t N, int mode,
                                 float post_scale, cudaStream_t stream);

// psgd_expand_sgd for a list of matrices in as few launches as possible (one grid per 32 matrices
// that take the vectorised form; the others one by one).  `common` carries lr / momentum / weight
// decay / first_step; param and momentum come from the items.
struct PsgdExpandItem {
  const float* P = nullptr;
  const float* Q = nullptr;
  int64_t n = 0, m = 0, N = 0;
  float* Mat = nullptr;
  float* param = nullptr;
  float* momentum = nullptr;
};
cudaError_t psgd_expand_sgd_grouped(const PsgdExpandItem* items, int count, int r, float post_scale,
                                    const SgdApply& common, int* launches, cudaStream_t stream);

// Batched forms of the small per-matrix kernels: one launch per kPsgdBatch matrices.
constexpr int kPsgdBatch = 32;
struct PsgdTransposeItem {
  const float* X;    // rows x r
  float* Xt;         // 16 x rows_pad
  int64_t rows, rows_pad;
  int r;
};
struct PsgdGatherItem {
  const float* src[kMaxWorld];  // every owner's accumulator (full output shape)
  float* out;                   // rows x r
  int64_t rows;
  int r;
};
struct PsgdGsItem {
  float* P;  // n x r, orthonormalised in place
  int64_t n;
  int r;
};
cudaError_t psgd_transpose_pad_batched(const PsgdTransposeItem* items, int count, cudaStream_t stream);
cudaError_t psgd_owner_gather_batched(const PsgdGatherItem* items, int count, int world, float scale,
                                      cudaStream_t stream);
cudaError_t gram_schmidt_batched(const PsgdGsItem* items, int count, float eps, cudaStream_t stream);

// Same expansion with the optimizer fused: Mat -= approx and the parameters take
// an SGD-momentum step with g = post_scale * approx (no dense gradient is written).
cudaError_t psgd_expand_sgd(const float* P, const float* Q, int64_t n, int64_t m, int r, float* Mat,
                            int64_t N, float post_scale, const SgdApply& apply, cudaStream_t stream);
// out[rows x r] = scale * (accumulator of each row's owner); owners[p] has the
// full output shape and may be peer memory.  Row ownership as in psgd_gemm.
cudaError_t psgd_owner_gather(const ReduceTargets& owners, int64_t rows, int r, float* out,
                              float scale, cudaStream_t stream);

}  // namespace cuda
}  // namespace hipress
