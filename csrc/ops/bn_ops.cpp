// Tensor-level entry points of the fused batch-norm kernels (csrc/kernels/bn.cu).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "../kernels/kernels.h"
#include "ops.h"

namespace hipress {
namespace ops {

namespace {

#define HP_BN_CHECK(e)                                                                        \
  do {                                                                                        \
    cudaError_t _e = (e);                                                                     \
    TORCH_CHECK(_e == cudaSuccess, "hipress batch-norm launch failed: ", cudaGetErrorString(_e)); \
  } while (0)

struct Shape {
  int64_t rows;
  int channels;
};

Shape check_activation(const torch::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kBFloat16, name, " must be a bf16 CUDA tensor");
  TORCH_CHECK(t.dim() == 4 && t.is_contiguous(at::MemoryFormat::ChannelsLast), name,
              " must be a 4-D channels-last tensor");
  return {t.size(0) * t.size(2) * t.size(3), int(t.size(1))};
}

const float* opt_f32(const c10::optional<torch::Tensor>& t, int channels, const char* name) {
  if (!t || !t->defined()) return nullptr;
  TORCH_CHECK(t->is_cuda() && t->scalar_type() == torch::kFloat32 && t->is_contiguous() &&
                  t->numel() == channels, name, " must be a contiguous float32 CUDA tensor with one value per channel");
  return t->data_ptr<float>();
}

}  // namespace

bool bn_supported(const torch::Tensor& x) {
  if (!x.is_cuda() || x.scalar_type() != torch::kBFloat16 || x.dim() != 4 ||
      !x.is_contiguous(at::MemoryFormat::ChannelsLast))
    return false;
  return cuda::bn_supported(x.size(0) * x.size(2) * x.size(3), int(x.size(1)));
}

std::vector<torch::Tensor> bn_forward(const torch::Tensor& x, const c10::optional<torch::Tensor>& residual,
                                      const c10::optional<torch::Tensor>& weight,
                                      const c10::optional<torch::Tensor>& bias,
                                      c10::optional<torch::Tensor> running_mean,
                                      c10::optional<torch::Tensor> running_var,
                                      c10::optional<torch::Tensor> num_batches, double momentum, double eps,
                                      bool relu) {
  const Shape s = check_activation(x, "x");
  TORCH_CHECK(cuda::bn_supported(s.rows, s.channels), "unsupported channel count ", s.channels);
  const void* res = nullptr;
  if (residual && residual->defined()) {
    const Shape r = check_activation(*residual, "residual");
    TORCH_CHECK(r.rows == s.rows && r.channels == s.channels, "residual must have x's shape");
    res = residual->data_ptr();
  }
  c10::cuda::CUDAGuard guard(x.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  auto y = torch::empty_like(x, x.options(), at::MemoryFormat::ChannelsLast);
  auto f32 = x.options().dtype(torch::kFloat32);
  auto stats = torch::empty({4, s.channels}, f32);  // mean, invstd, (a, b) interleaved
  auto partial = torch::empty({2 * cuda::bn_partial_elems(s.rows, s.channels)}, f32);
  long long* nb = nullptr;
  if (num_batches && num_batches->defined()) {
    TORCH_CHECK(num_batches->is_cuda() && num_batches->scalar_type() == torch::kInt64, "num_batches must be int64");
    nb = reinterpret_cast<long long*>(num_batches->data_ptr<int64_t>());
  }
  float* rm = const_cast<float*>(opt_f32(running_mean, s.channels, "running_mean"));
  float* rv = const_cast<float*>(opt_f32(running_var, s.channels, "running_var"));
  TORCH_CHECK((rm == nullptr) == (rv == nullptr), "running_mean and running_var go together");
  float* st = stats.data_ptr<float>();
  HP_BN_CHECK(cuda::bn_forward(x.data_ptr(), res, y.data_ptr(), s.rows, s.channels,
                               opt_f32(weight, s.channels, "weight"), opt_f32(bias, s.channels, "bias"), rm, rv,
                               nb, float(momentum), float(eps), relu ? 1 : 0, st, st + s.channels,
                               st + 2 * s.channels, partial.data_ptr<float>(), stream));
  return {y, stats};
}

std::vector<torch::Tensor> bn_backward(const torch::Tensor& dy, const torch::Tensor& x,
                                       const c10::optional<torch::Tensor>& y,
                                       const c10::optional<torch::Tensor>& weight, const torch::Tensor& stats,
                                       bool relu, bool want_dres) {
  const Shape s = check_activation(x, "x");
  const Shape g = check_activation(dy, "dy");
  TORCH_CHECK(g.rows == s.rows && g.channels == s.channels, "dy must have x's shape");
  const void* yp = nullptr;
  if (relu) {
    TORCH_CHECK(y && y->defined(), "the fused ReLU needs the forward output");
    const Shape o = check_activation(*y, "y");
    TORCH_CHECK(o.rows == s.rows && o.channels == s.channels, "y must have x's shape");
    yp = y->data_ptr();
  }
  TORCH_CHECK(stats.is_cuda() && stats.scalar_type() == torch::kFloat32 && stats.is_contiguous() &&
                  stats.numel() == 4 * s.channels, "stats must be the tensor returned by bn_forward");
  c10::cuda::CUDAGuard guard(x.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  auto dx = torch::empty_like(x, x.options(), at::MemoryFormat::ChannelsLast);
  torch::Tensor dres;
  if (want_dres) dres = torch::empty_like(x, x.options(), at::MemoryFormat::ChannelsLast);
  auto f32 = x.options().dtype(torch::kFloat32);
  auto dwb = torch::empty({2, s.channels}, f32);
  auto scratch = torch::empty({4 * s.channels + 2 * cuda::bn_partial_elems(s.rows, s.channels)}, f32);
  const float* st = stats.data_ptr<float>();
  float* sc = scratch.data_ptr<float>();
  HP_BN_CHECK(cuda::bn_backward(dy.data_ptr(), x.data_ptr(), yp, dx.data_ptr(), want_dres ? dres.data_ptr() : nullptr,
                                s.rows, s.channels, opt_f32(weight, s.channels, "weight"), st, st + s.channels,
                                relu ? 1 : 0, dwb.data_ptr<float>(), dwb.data_ptr<float>() + s.channels, sc,
                                sc + 4 * s.channels, stream));
  std::vector<torch::Tensor> out{dx, dwb[0], dwb[1]};
  if (want_dres) out.push_back(dres);
  return out;
}

// ---------------------------------------------------------------- 3x3 / stride 2 max pooling
bool maxpool_supported(const torch::Tensor& x) {
  return x.is_cuda() && x.scalar_type() == torch::kBFloat16 && x.dim() == 4 &&
         x.is_contiguous(at::MemoryFormat::ChannelsLast) && x.size(1) >= 8 && x.size(1) % 8 == 0 &&
         x.numel() > 0;
}

std::vector<torch::Tensor> maxpool3x3s2_forward(const torch::Tensor& x) {
  TORCH_CHECK(maxpool_supported(x), "maxpool3x3s2 needs a channels-last bf16 CUDA tensor with channels % 8 == 0");
  const int n = int(x.size(0)), c = int(x.size(1)), h = int(x.size(2)), w = int(x.size(3));
  const int ho = (h - 1) / 2 + 1, wo = (w - 1) / 2 + 1;
  c10::cuda::CUDAGuard guard(x.device());
  auto y = torch::empty({n, c, ho, wo}, x.options(), at::MemoryFormat::ChannelsLast);
  auto idx = torch::empty({n, c, ho, wo}, x.options().dtype(torch::kUInt8), at::MemoryFormat::ChannelsLast);
  HP_BN_CHECK(cuda::maxpool3x3s2_forward(x.data_ptr(), y.data_ptr(), idx.data_ptr<uint8_t>(), n, h, w, c,
                                         at::cuda::getCurrentCUDAStream()));
  return {y, idx};
}

torch::Tensor maxpool3x3s2_backward(const torch::Tensor& dy, const torch::Tensor& idx, int64_t h, int64_t w) {
  check_activation(dy, "dy");
  TORCH_CHECK(idx.is_cuda() && idx.scalar_type() == torch::kUInt8 && idx.sizes() == dy.sizes() &&
                  idx.is_contiguous(at::MemoryFormat::ChannelsLast), "idx must be the forward's index tensor");
  const int n = int(dy.size(0)), c = int(dy.size(1));
  TORCH_CHECK(dy.size(2) == (h - 1) / 2 + 1 && dy.size(3) == (w - 1) / 2 + 1, "dy does not match the input size");
  c10::cuda::CUDAGuard guard(dy.device());
  auto dx = torch::empty({n, c, h, w}, dy.options(), at::MemoryFormat::ChannelsLast);
  HP_BN_CHECK(cuda::maxpool3x3s2_backward(dy.data_ptr(), idx.data_ptr<uint8_t>(), dx.data_ptr(), n, int(h), int(w), c,
                                          at::cuda::getCurrentCUDAStream()));
  return dx;
}

// ---------------------------------------------------------------- bias + ReLU (+ 2x2 max pool)
bool bias_relu_supported(const torch::Tensor& x, bool pool) {
  if (!x.is_cuda() || x.scalar_type() != torch::kBFloat16 || x.dim() != 4 || x.numel() == 0 ||
      !x.is_contiguous(at::MemoryFormat::ChannelsLast))
    return false;
  if (pool && ((x.size(2) & 1) || (x.size(3) & 1))) return false;
  const int64_t rows = x.size(0) * (pool ? x.size(2) / 2 : x.size(2)) * (pool ? x.size(3) / 2 : x.size(3));
  return cuda::bias_relu_supported(rows, int(x.size(1)));
}

std::vector<torch::Tensor> bias_relu_forward(const torch::Tensor& x, const torch::Tensor& bias, bool pool) {
  TORCH_CHECK(bias_relu_supported(x, pool), "bias_relu: unsupported activation tensor");
  const int n = int(x.size(0)), c = int(x.size(1)), h = int(x.size(2)), w = int(x.size(3));
  const int ho = pool ? h / 2 : h, wo = pool ? w / 2 : w;
  c10::cuda::CUDAGuard guard(x.device());
  auto y = torch::empty({n, c, ho, wo}, x.options(), at::MemoryFormat::ChannelsLast);
  torch::Tensor idx;
  if (pool) idx = torch::empty({n, c, ho, wo}, x.options().dtype(torch::kUInt8), at::MemoryFormat::ChannelsLast);
  HP_BN_CHECK(cuda::bias_relu_forward(x.data_ptr(), opt_f32(bias, c, "bias"), y.data_ptr(),
                                      pool ? idx.data_ptr<uint8_t>() : nullptr, n, h, w, c, pool ? 1 : 0,
                                      at::cuda::getCurrentCUDAStream()));
  if (pool) return {y, idx};
  return {y};
}

std::vector<torch::Tensor> bias_relu_backward(const torch::Tensor& dy, const torch::Tensor& y,
                                              const c10::optional<torch::Tensor>& idx, bool pool) {
  const Shape s = check_activation(y, "y");
  const Shape g = check_activation(dy, "dy");
  TORCH_CHECK(g.rows == s.rows && g.channels == s.channels && dy.sizes() == y.sizes(), "dy must have y's shape");
  const int n = int(y.size(0)), c = int(y.size(1));
  const int h = int(y.size(2)) * (pool ? 2 : 1), w = int(y.size(3)) * (pool ? 2 : 1);
  const uint8_t* ip = nullptr;
  if (pool) {
    TORCH_CHECK(idx && idx->defined() && idx->is_cuda() && idx->scalar_type() == torch::kUInt8 &&
                    idx->sizes() == y.sizes() && idx->is_contiguous(at::MemoryFormat::ChannelsLast),
                "idx must be the forward's index tensor");
    ip = idx->data_ptr<uint8_t>();
  }
  c10::cuda::CUDAGuard guard(y.device());
  auto dz = torch::empty({n, c, h, w}, y.options(), at::MemoryFormat::ChannelsLast);
  auto f32 = y.options().dtype(torch::kFloat32);
  auto db = torch::empty({c}, f32);
  auto partial = torch::empty({cuda::bias_relu_partial_elems(s.rows, c)}, f32);
  HP_BN_CHECK(cuda::bias_relu_backward(dy.data_ptr(), y.data_ptr(), ip, dz.data_ptr(), db.data_ptr<float>(),
                                       partial.data_ptr<float>(), n, h, w, c, pool ? 1 : 0,
                                       at::cuda::getCurrentCUDAStream()));
  return {dz, db};
}

// ---------------------------------------------------------------- column sums (bias gradients)
bool colsum_supported(const torch::Tensor& dy) {
  return dy.is_cuda() && dy.scalar_type() == torch::kBFloat16 && dy.is_contiguous() && dy.dim() >= 2 &&
         dy.numel() > 0 && cuda::bias_relu_supported(dy.numel() / dy.size(-1), int(dy.size(-1)));
}

torch::Tensor colsum(const torch::Tensor& dy) {
  TORCH_CHECK(colsum_supported(dy), "colsum: needs a contiguous bf16 CUDA tensor whose last dimension / 8 is a power of two up to 32 or a multiple of 32");
  const int64_t rows = dy.numel() / dy.size(-1);
  const int c = int(dy.size(-1));
  c10::cuda::CUDAGuard guard(dy.device());
  auto f32 = dy.options().dtype(torch::kFloat32);
  auto out = torch::empty({c}, f32);
  auto partial = torch::empty({cuda::bias_relu_partial_elems(rows, c)}, f32);
  HP_BN_CHECK(cuda::colsum_bf16(dy.data_ptr(), out.data_ptr<float>(), partial.data_ptr<float>(), rows, c,
                                at::cuda::getCurrentCUDAStream()));
  return out;
}

// ---------------------------------------------------------------- residual add + LayerNorm
namespace {
int64_t ln_rows(const torch::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kBFloat16 && t.is_contiguous() && t.dim() >= 1, name,
              " must be a contiguous bf16 CUDA tensor");
  return t.numel() / t.size(-1);
}
}  // namespace

bool add_ln_supported(const torch::Tensor& x) {
  return x.is_cuda() && x.scalar_type() == torch::kBFloat16 && x.is_contiguous() && x.dim() >= 1 &&
         x.numel() > 0 && cuda::add_ln_supported(x.numel() / x.size(-1), int(x.size(-1)));
}

std::vector<torch::Tensor> add_ln_forward(const torch::Tensor& x, const c10::optional<torch::Tensor>& delta,
                                          const torch::Tensor& weight, const torch::Tensor& bias, double eps) {
  TORCH_CHECK(add_ln_supported(x), "add_layer_norm: unsupported input");
  const int64_t rows = ln_rows(x, "x");
  const int hidden = int(x.size(-1));
  const bool add = delta && delta->defined();
  if (add) TORCH_CHECK(ln_rows(*delta, "delta") == rows && delta->sizes() == x.sizes(), "delta must have x's shape");
  c10::cuda::CUDAGuard guard(x.device());
  auto y = torch::empty_like(x);
  torch::Tensor z = add ? torch::empty_like(x) : x;
  auto stats = torch::empty({2, rows}, x.options().dtype(torch::kFloat32));
  HP_BN_CHECK(cuda::add_ln_forward(x.data_ptr(), add ? delta->data_ptr() : nullptr, opt_f32(weight, hidden, "weight"),
                                   opt_f32(bias, hidden, "bias"), y.data_ptr(), add ? z.data_ptr() : nullptr,
                                   stats.data_ptr<float>(), stats.data_ptr<float>() + rows, rows, hidden, float(eps),
                                   at::cuda::getCurrentCUDAStream()));
  return {y, z, stats};
}

std::vector<torch::Tensor> add_ln_backward(const torch::Tensor& dy, const torch::Tensor& z, const torch::Tensor& stats,
                                           const torch::Tensor& weight) {
  const int64_t rows = ln_rows(z, "z");
  const int hidden = int(z.size(-1));
  TORCH_CHECK(ln_rows(dy, "dy") == rows && dy.sizes() == z.sizes(), "dy must have z's shape");
  TORCH_CHECK(stats.is_cuda() && stats.scalar_type() == torch::kFloat32 && stats.is_contiguous() &&
                  stats.numel() == 2 * rows, "stats must be the tensor returned by add_ln_forward");
  c10::cuda::CUDAGuard guard(z.device());
  auto dz = torch::empty_like(z);
  auto f32 = z.options().dtype(torch::kFloat32);
  auto dwb = torch::empty({2, hidden}, f32);
  auto partial = torch::empty({cuda::add_ln_partial_elems(rows, hidden)}, f32);
  HP_BN_CHECK(cuda::add_ln_backward(dy.data_ptr(), z.data_ptr(), stats.data_ptr<float>(),
                                    stats.data_ptr<float>() + rows, opt_f32(weight, hidden, "weight"), dz.data_ptr(),
                                    dwb.data_ptr<float>(), dwb.data_ptr<float>() + hidden, partial.data_ptr<float>(),
                                    rows, hidden, at::cuda::getCurrentCUDAStream()));
  return {dz, dwb[0], dwb[1]};
}

}  // namespace ops
}  // namespace hipress
