// Tensor-level codec operations: the per-algorithm compress / decompress
// entrypoints of the extension.  Each accepts CUDA tensors (sm_100a kernels on
// the current stream, no host synchronisation) or CPU tensors (the CPU codec),
// so the same call is both the product path and its oracle.
//
// They correspond to the reference's nine hp_cuda_* entrypoints
// (ref hp_cuda.cpp:18-102, hp_cuda_kernel.cu:30-301), with two differences:
// decompression takes the payloads of *all* ranks and makes one pass, and
// stochastic rounding / sampling take an explicit seed instead of the clock.
#pragma once
#include <torch/extension.h>

#include <vector>

namespace hipress {
namespace ops {

// Payload sizes (bytes) for n fp32 elements.
int64_t tbq_payload_bytes(int64_t n);
int64_t terngrad_payload_bytes(int64_t n, int64_t bitwidth);
int64_t sparse_payload_bytes(int64_t n, double keep_fraction);
int64_t ecq_payload_bytes(int64_t n, int64_t bitwidth);

void tbq_compress(const torch::Tensor& grad, torch::Tensor residual, torch::Tensor out,
                  double threshold);
// payloads: one uint8 tensor per rank, accumulated in list order.
void tbq_decompress(const std::vector<torch::Tensor>& payloads, torch::Tensor out, double threshold,
                    bool add, double post_scale);

void terngrad_compress(const torch::Tensor& grad, torch::Tensor out, int64_t bitwidth,
                       bool enable_random, int64_t seed, c10::optional<torch::Tensor> residual);
// bitwidth: 0 = read it from the payload headers on the device; a known bitwidth selects a kernel
// compiled for it (payloads with another bitwidth are then rejected through the status word).
void terngrad_decompress(const std::vector<torch::Tensor>& payloads, torch::Tensor out, bool add,
                         double post_scale, int64_t bitwidth);

// accumulate: R += grad first (GradDrop).  Otherwise grad may be undefined (DGC).
void sparse_compress(const c10::optional<torch::Tensor>& grad, torch::Tensor R, torch::Tensor out,
                     double sample_rate, double keep_fraction, int64_t seed, bool accumulate);
// DGC with momentum correction in one fused pipeline (CUDA): u = momentum*u + s*grad, v += u,
// top-k of v into `out`, u and v cleared at the sent positions; s clips grad to norm `clip`
// (<= 0: off); zero_grad leaves zeros in grad.
void dgc_momentum_compress(torch::Tensor grad, torch::Tensor u, torch::Tensor v, torch::Tensor out,
                           double sample_rate, double keep_fraction, int64_t seed, double momentum,
                           double clip, bool zero_grad);
void sparse_decompress(const std::vector<torch::Tensor>& payloads, torch::Tensor out, bool add,
                       double post_scale);

void ecq_compress(const torch::Tensor& grad, torch::Tensor history, torch::Tensor out, double alpha,
                  double beta, int64_t bitwidth, int64_t seed);
void ecq_decompress(const std::vector<torch::Tensor>& payloads, torch::Tensor out, bool add,
                    double post_scale);

// PowerSGD stages (intended maths of ref powersgd_body.h:10-78; the shipped
// code copies every result into a temporary and so computes nothing).
//   encode1: M[:N] = grad + residual;  P = M Q
//   encode2: P = orthonormalise(P);    Q = M^T P
//   decode : M = P Q^T; residual = grad - M[:N]; grad = M[:N]
// CUDA tensors run the tcgen05 GEMMs (TF32 inputs, fp32 accumulation).
void powersgd_encode1(const torch::Tensor& grad, const torch::Tensor& residual,
                      const torch::Tensor& Q, torch::Tensor M, torch::Tensor P);
void powersgd_encode2(torch::Tensor P, const torch::Tensor& M, torch::Tensor Q);
void powersgd_decode(const torch::Tensor& P, const torch::Tensor& Q, torch::Tensor M,
                     torch::Tensor residual, torch::Tensor grad);
// Building blocks of the data-parallel PowerSGD compressor.
// out (+)= M X  (mode 0, out is n x r, X is m x r)  or  M^T X  (mode 1, out is m x r, X is n x r).
// `owners`: one tensor per rank with out's shape; each output row is added into
// the tensor of the rank that owns it (even row split).  zero_first clears the
// local tensor before accumulating.  simt forces the non-tensor-core kernel.
void psgd_project(int64_t mode, const torch::Tensor& M, const torch::Tensor& X,
                  const std::vector<torch::Tensor>& owners, bool simt);
// outs[i] += Ms[i] Xs[i] (mode 0) or Ms[i]^T Xs[i] (mode 1) for a list of CUDA matrices, all tensor-core
// eligible ones in one grid.
void psgd_project_grouped(int64_t mode, const std::vector<torch::Tensor>& Ms, const std::vector<torch::Tensor>& Xs,
                          const std::vector<torch::Tensor>& outs);
void gram_schmidt(torch::Tensor P, double eps);
// grad_out[:N] = post_scale * P Q^T ; M -= P Q^T   (error feedback stays in M)
void psgd_expand_feedback(const torch::Tensor& P, const torch::Tensor& Q, torch::Tensor M,
                          torch::Tensor grad_out, double post_scale);

// out = scale * (each row taken from its owner's accumulator); owners as in psgd_project.
void psgd_owner_gather(const std::vector<torch::Tensor>& owners, torch::Tensor out, double scale);
// M -= P Q^T and a fused SGD-momentum step of `param` with g = post_scale * P Q^T.
void psgd_expand_sgd(const torch::Tensor& P, const torch::Tensor& Q, torch::Tensor M,
                     torch::Tensor param, torch::Tensor momentum, double post_scale, double lr,
                     double mu, double weight_decay, bool first_step);

// The same for a list of matrices of one rank, all matrices that take the vectorised form in one grid.
void psgd_expand_sgd_grouped(const std::vector<torch::Tensor>& Ps, const std::vector<torch::Tensor>& Qs,
                             const std::vector<torch::Tensor>& Ms, const std::vector<torch::Tensor>& params,
                             const std::vector<torch::Tensor>& momenta, double post_scale, double lr, double mu,
                             double weight_decay, bool first_step);

// Device status word of the last bounds / header failure seen by kernels
// launched through these ops on the tensor's device (0 = none); reading it
// synchronises the current stream.
int64_t read_status(const torch::Tensor& like, bool reset);
// Zero-initialised per-(device, stream) scratch used by kernels that need it.
void* scratch_for(const torch::Tensor& like, size_t bytes);
// Fused training-mode batch norm (+ residual add, + ReLU) for channels-last bf16 activations.
// bn_forward returns {y, stats}; stats = [4][C] floats (mean, invstd, scale/shift pairs) and is
// what bn_backward needs.  bn_backward returns {dx, dweight, dbias [, dresidual]}.
bool bn_supported(const torch::Tensor& x);
std::vector<torch::Tensor> bn_forward(const torch::Tensor& x, const c10::optional<torch::Tensor>& residual,
                                      const c10::optional<torch::Tensor>& weight,
                                      const c10::optional<torch::Tensor>& bias,
                                      c10::optional<torch::Tensor> running_mean,
                                      c10::optional<torch::Tensor> running_var,
                                      c10::optional<torch::Tensor> num_batches, double momentum, double eps,
                                      bool relu);
std::vector<torch::Tensor> bn_backward(const torch::Tensor& dy, const torch::Tensor& x,
                                       const c10::optional<torch::Tensor>& y,
                                       const c10::optional<torch::Tensor>& weight, const torch::Tensor& stats,
                                       bool relu, bool want_dres);

// 3x3 / stride 2 / padding 1 max pooling of channels-last bf16 activations: {y, idx} forward
// (idx: winning window position per output element, one byte), gather backward.
bool maxpool_supported(const torch::Tensor& x);
std::vector<torch::Tensor> maxpool3x3s2_forward(const torch::Tensor& x);
torch::Tensor maxpool3x3s2_backward(const torch::Tensor& dy, const torch::Tensor& idx, int64_t h, int64_t w);

// Convolution epilogue: y = relu(x + bias), optionally followed by 2x2 / stride 2 max pooling,
// over channels-last bf16 activations.  forward -> {y [, idx]}; backward -> {dz, dbias}.
bool bias_relu_supported(const torch::Tensor& x, bool pool);
std::vector<torch::Tensor> bias_relu_forward(const torch::Tensor& x, const torch::Tensor& bias, bool pool);
std::vector<torch::Tensor> bias_relu_backward(const torch::Tensor& dy, const torch::Tensor& y,
                                              const c10::optional<torch::Tensor>& idx, bool pool);

// Sum over all leading dimensions of a contiguous bf16 tensor -> fp32 [last dim] (bias gradients).
// {dW [out, in] fp32, db [out] fp32} of a linear layer from dy [tokens, out] and x [tokens, in] (bf16), the
// bias gradient taken by the GEMM's epilogue; an empty list when the library has no such algorithm for the
// shape (the caller then uses its separate GEMM and column sum).
std::vector<torch::Tensor> linear_wgrad_bgrad(const torch::Tensor& dy, const torch::Tensor& x);
bool colsum_supported(const torch::Tensor& dy);
torch::Tensor colsum(const torch::Tensor& dy);

// y = LayerNorm(x + delta) over the last dimension of contiguous bf16 tensors (delta optional).
// forward -> {y, z = bf16(x + delta) (x itself without delta), stats}; backward -> {dz, dweight, dbias}.
bool add_ln_supported(const torch::Tensor& x);
std::vector<torch::Tensor> add_ln_forward(const torch::Tensor& x, const c10::optional<torch::Tensor>& delta,
                                          const torch::Tensor& weight, const torch::Tensor& bias, double eps);
std::vector<torch::Tensor> add_ln_backward(const torch::Tensor& dy, const torch::Tensor& z, const torch::Tensor& stats,
                                           const torch::Tensor& weight);

int* status_word_for(const torch::Tensor& like);

}  // namespace ops
}  // namespace hipress
