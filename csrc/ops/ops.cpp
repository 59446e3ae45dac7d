#include "ops.h"

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <map>
#include <mutex>

#include "../codec_cpu/codec_cpu.h"
#include "../common/codec_math.h"
#include "../kernels/kernels.h"

namespace hipress {
namespace ops {

namespace {

#define HP_CHECK_CUDA(e)                                                              \
  do {                                                                                \
    cudaError_t _e = (e);                                                             \
    TORCH_CHECK(_e == cudaSuccess, "hipress kernel launch failed: ", cudaGetErrorString(_e)); \
  } while (0)

void check_f32(const torch::Tensor& t, const char* name) {
  TORCH_CHECK(t.defined(), name, " is undefined");
  TORCH_CHECK(t.scalar_type() == torch::kFloat32, name, " must be float32");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}
void check_u8(const torch::Tensor& t, const char* name) {
  TORCH_CHECK(t.defined(), name, " is undefined");
  TORCH_CHECK(t.scalar_type() == torch::kUInt8, name, " must be uint8");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}
void check_same_device(const torch::Tensor& a, const torch::Tensor& b) {
  TORCH_CHECK(a.device() == b.device(), "tensors must be on the same device");
}

cuda::PushTargets local_target(torch::Tensor& out) {
  cuda::PushTargets t;
  t.world = 1;
  t.payload[0] = out.data_ptr<uint8_t>();
  return t;
}

cuda::UnpackSources sources_of(const std::vector<torch::Tensor>& payloads, const torch::Tensor& out) {
  TORCH_CHECK(!payloads.empty() && payloads.size() <= size_t(cuda::kMaxWorld),
              "between 1 and ", cuda::kMaxWorld, " payloads expected");
  cuda::UnpackSources s;
  s.world = int(payloads.size());
  for (size_t r = 0; r < payloads.size(); ++r) {
    check_u8(payloads[r], "payload");
    check_same_device(payloads[r], out);
    s.payload[r] = payloads[r].data_ptr<uint8_t>();
    s.payload_bytes[r] = payloads[r].numel();
  }
  return s;
}

// CPU form of the one-pass unpack + accumulate: the decoded payloads are summed per element in
// the canonical order (tree_sum in codec_math.h), `decoded + out` is applied to the finished
// sum when accumulating, and the result is scaled.  decode(r, dst, add_to) decodes payload r.
template <typename Decode>
void cpu_accumulate(size_t world, int64_t n, float* out, bool add, double post_scale, Decode decode) {
  if (world == 1) {
    decode(0, out, add);
  } else {
    std::vector<std::vector<float>> tmp(world, std::vector<float>(size_t(n)));
    for (size_t r = 0; r < world; ++r) decode(r, tmp[r].data(), false);
    for (int64_t i = 0; i < n; ++i) {
      float v[cuda::kMaxWorld];
      for (size_t r = 0; r < world; ++r) v[r] = tmp[r][size_t(i)];
      const float s = tree_sum(v, int(world));
      out[i] = add ? hp_add(s, out[i]) : s;
    }
  }
  if (post_scale != 1.0)
    for (int64_t i = 0; i < n; ++i) out[i] = hp_mul(out[i], float(post_scale));
}

struct DeviceState {
  std::map<std::pair<int, cudaStream_t>, torch::Tensor> scratch;
  std::map<int, torch::Tensor> status;
  std::mutex mu;
};
DeviceState& state() {
  static DeviceState* s = new DeviceState();  // leaked on purpose: outlives static destruction order
  return *s;
}

}  // namespace

void* scratch_for(const torch::Tensor& like, size_t bytes) {
  auto& st = state();
  const int dev = like.get_device();
  const cudaStream_t stream = at::cuda::getCurrentCUDAStream(dev).stream();
  std::lock_guard<std::mutex> lk(st.mu);
  auto key = std::make_pair(dev, stream);
  auto it = st.scratch.find(key);
  if (bytes < 256 * 1024) bytes = 256 * 1024;  // one size for all users: never reallocated in flight
  if (it == st.scratch.end() || size_t(it->second.numel()) < bytes) {
    auto t = torch::zeros({int64_t(bytes)}, torch::dtype(torch::kUInt8).device(like.device()));
    it = st.scratch.insert_or_assign(key, t).first;
  }
  return it->second.data_ptr();
}

int* status_word_for(const torch::Tensor& like) {
  auto& st = state();
  const int dev = like.get_device();
  std::lock_guard<std::mutex> lk(st.mu);
  auto it = st.status.find(dev);
  if (it == st.status.end())
    it = st.status.emplace(dev, torch::zeros({4}, torch::dtype(torch::kInt32).device(like.device()))).first;
  return it->second.data_ptr<int>();
}

int64_t read_status(const torch::Tensor& like, bool reset) {
  if (!like.is_cuda()) return 0;
  status_word_for(like);
  torch::Tensor t;
  {
    std::lock_guard<std::mutex> lk(state().mu);
    t = state().status.at(like.get_device());
  }
  const int64_t v = t[0].item<int64_t>();
  if (reset && v != 0) t.zero_();
  return v;
}

int64_t tbq_payload_bytes(int64_t n) { return hipress::tbq_payload_bytes(n); }
int64_t terngrad_payload_bytes(int64_t n, int64_t bw) {
  TORCH_CHECK(tern_bitwidth_ok(int(bw)), "bitwidth must be 1, 2, 4 or 8");
  return hipress::tern_payload_bytes(n, int(bw));
}
int64_t sparse_payload_bytes(int64_t n, double keep_fraction) {
  return hipress::sparse_payload_bytes(std::min<int64_t>(n, sparse_expected_k(n, keep_fraction)));
}
int64_t ecq_payload_bytes(int64_t n, int64_t bw) {
  TORCH_CHECK(ecq_bitwidth_ok(int(bw)), "bitwidth must be 2, 4 or 8");
  return hipress::ecq_payload_bytes(n, int(bw));
}

// ------------------------------------------------------------------ TBQ
void tbq_compress(const torch::Tensor& grad, torch::Tensor residual, torch::Tensor out,
                  double threshold) {
  check_f32(grad, "grad");
  check_f32(residual, "residual");
  check_u8(out, "out");
  const int64_t n = grad.numel();
  TORCH_CHECK(residual.numel() == n, "residual must have as many elements as grad");
  TORCH_CHECK(out.numel() >= tbq_payload_bytes(n), "out needs ", tbq_payload_bytes(n), " bytes");
  check_same_device(grad, residual);
  check_same_device(grad, out);
  if (n == 0) return;
  if (grad.is_cuda()) {
    c10::cuda::CUDAGuard guard(grad.device());
    HP_CHECK_CUDA(cuda::tbq_compress(grad.data_ptr<float>(), residual.data_ptr<float>(), n,
                                     float(threshold), local_target(out),
                                     at::cuda::getCurrentCUDAStream()));
  } else {
    cpu::tbq_compress(grad.data_ptr<float>(), residual.data_ptr<float>(), n, float(threshold),
                      out.data_ptr<uint8_t>());
  }
}

void tbq_decompress(const std::vector<torch::Tensor>& payloads, torch::Tensor out, double threshold,
                    bool add, double post_scale) {
  check_f32(out, "out");
  const int64_t n = out.numel();
  if (n == 0) return;
  for (auto& p : payloads) {
    check_u8(p, "payload");
    TORCH_CHECK(p.numel() >= tbq_payload_bytes(n), "payload too small for out");
  }
  if (out.is_cuda()) {
    c10::cuda::CUDAGuard guard(out.device());
    HP_CHECK_CUDA(cuda::tbq_unpack_accum(sources_of(payloads, out), float(threshold),
                                         out.data_ptr<float>(), n, add ? 1 : 0, float(post_scale),
                                         cuda::SgdApply{}, at::cuda::getCurrentCUDAStream()));
  } else {
    TORCH_CHECK(!payloads.empty() && payloads.size() <= size_t(cuda::kMaxWorld),
                "between 1 and ", cuda::kMaxWorld, " payloads expected");
    cpu_accumulate(payloads.size(), n, out.data_ptr<float>(), add, post_scale,
                   [&](size_t r, float* dst, bool add_to) {
                     cpu::tbq_decompress(payloads[r].data_ptr<uint8_t>(), n, float(threshold), dst,
                                         add_to ? 1 : 0);
                   });
  }
}

// ------------------------------------------------------------------ TernGrad
void terngrad_compress(const torch::Tensor& grad, torch::Tensor out, int64_t bitwidth,
                       bool enable_random, int64_t seed, c10::optional<torch::Tensor> residual) {
  check_f32(grad, "grad");
  check_u8(out, "out");
  check_same_device(grad, out);
  TORCH_CHECK(tern_bitwidth_ok(int(bitwidth)), "bitwidth must be 1, 2, 4 or 8");
  const int64_t n = grad.numel();
  TORCH_CHECK(n > 0, "empty tensor");
  TORCH_CHECK(out.numel() == tern_payload_bytes(n, int(bitwidth)),
              "out must have exactly 10 + ceil(n/dpb) = ", tern_payload_bytes(n, int(bitwidth)), " bytes");
  float* res = nullptr;
  if (residual.has_value() && residual->defined()) {
    check_f32(*residual, "residual");
    check_same_device(grad, *residual);
    TORCH_CHECK(residual->numel() == n, "residual must have as many elements as grad");
    res = residual->data_ptr<float>();
  }
  if (grad.is_cuda()) {
    c10::cuda::CUDAGuard guard(grad.device());
    void* scratch = scratch_for(grad, cuda::minmax_scratch_bytes());
    HP_CHECK_CUDA(cuda::terngrad_compress(grad.data_ptr<float>(), res, n, int(bitwidth),
                                          enable_random ? 1 : 0, uint64_t(seed), local_target(out),
                                          scratch, at::cuda::getCurrentCUDAStream()));
  } else {
    const int rc = cpu::terngrad_compress(grad.data_ptr<float>(), n, int(bitwidth),
                                          enable_random ? 1 : 0, uint64_t(seed),
                                          out.data_ptr<uint8_t>(), out.numel(), res);
    TORCH_CHECK(rc == 0, "terngrad_compress failed");
  }
}

void terngrad_decompress(const std::vector<torch::Tensor>& payloads, torch::Tensor out, bool add,
                         double post_scale, int64_t bitwidth) {
  check_f32(out, "out");
  const int64_t n = out.numel();
  TORCH_CHECK(n > 0, "empty tensor");
  if (out.is_cuda()) {
    c10::cuda::CUDAGuard guard(out.device());
    HP_CHECK_CUDA(cuda::terngrad_unpack_accum(sources_of(payloads, out), out.data_ptr<float>(), n,
                                              add ? 1 : 0, float(post_scale), cuda::SgdApply{},
                                              status_word_for(out),
                                              at::cuda::getCurrentCUDAStream(), int(bitwidth)));
  } else {
    TORCH_CHECK(!payloads.empty() && payloads.size() <= size_t(cuda::kMaxWorld),
                "between 1 and ", cuda::kMaxWorld, " payloads expected");
    for (auto& p : payloads) check_u8(p, "payload");
    cpu_accumulate(payloads.size(), n, out.data_ptr<float>(), add, post_scale,
                   [&](size_t r, float* dst, bool add_to) {
                     const int64_t cnt = cpu::terngrad_decompress(payloads[r].data_ptr<uint8_t>(),
                                                                  payloads[r].numel(), dst, n, add_to ? 1 : 0);
                     TORCH_CHECK(cnt == n, "payload ", r, " decodes to ", cnt, " elements, expected ", n);
                   });
  }
}

// ------------------------------------------------------------------ sparse
void sparse_compress(const c10::optional<torch::Tensor>& grad, torch::Tensor R, torch::Tensor out,
                     double sample_rate, double keep_fraction, int64_t seed, bool accumulate) {
  check_f32(R, "R");
  check_u8(out, "out");
  check_same_device(R, out);
  const int64_t n = R.numel();
  TORCH_CHECK(n > 0 && n <= 0x7fffffff, "element count out of range");
  TORCH_CHECK(keep_fraction > 0.0 && keep_fraction <= 1.0, "keep_fraction must be in (0, 1]");
  TORCH_CHECK(sample_rate >= 0.0 && sample_rate <= 1.0, "sample_rate must be in [0, 1]");
  TORCH_CHECK(out.numel() >= sparse_payload_bytes(n, keep_fraction), "out needs ",
              sparse_payload_bytes(n, keep_fraction), " bytes");
  const float* g = nullptr;
  if (accumulate) {
    TORCH_CHECK(grad.has_value() && grad->defined(), "accumulate needs grad");
    check_f32(*grad, "grad");
    check_same_device(*grad, R);
    TORCH_CHECK(grad->numel() == n, "grad must have as many elements as R");
    g = grad->data_ptr<float>();
  }
  if (R.is_cuda()) {
    c10::cuda::CUDAGuard guard(R.device());
    // the sparse state lives behind the min/max state other codecs keep in the same scratch
    void* scratch = static_cast<uint8_t*>(scratch_for(R, 16384 + cuda::sparse_scratch_bytes(n))) + 16384;
    HP_CHECK_CUDA(cuda::sparse_compress(g, R.data_ptr<float>(), n, sample_rate, keep_fraction,
                                        uint64_t(seed), accumulate ? 1 : 0, local_target(out),
                                        scratch, at::cuda::getCurrentCUDAStream()));
  } else {
    const int64_t rc = cpu::sparse_compress(g, R.data_ptr<float>(), n, sample_rate, keep_fraction,
                                            uint64_t(seed), accumulate ? 1 : 0,
                                            out.data_ptr<uint8_t>(), out.numel());
    TORCH_CHECK(rc >= 4, "sparse_compress failed");
  }
}

void dgc_momentum_compress(torch::Tensor grad, torch::Tensor u, torch::Tensor v, torch::Tensor out,
                           double sample_rate, double keep_fraction, int64_t seed, double momentum,
                           double clip, bool zero_grad) {
  check_f32(grad, "grad");
  check_f32(u, "u");
  check_f32(v, "v");
  check_u8(out, "out");
  check_same_device(v, out);
  check_same_device(v, grad);
  check_same_device(v, u);
  const int64_t n = v.numel();
  TORCH_CHECK(v.is_cuda(), "dgc_momentum_compress runs on CUDA tensors");
  TORCH_CHECK(n > 0 && n <= 0x7fffffff && grad.numel() == n && u.numel() == n, "grad, u and v must have the same size");
  TORCH_CHECK(keep_fraction > 0.0 && keep_fraction <= 1.0, "keep_fraction must be in (0, 1]");
  TORCH_CHECK(out.numel() >= sparse_payload_bytes(n, keep_fraction), "out needs ",
              sparse_payload_bytes(n, keep_fraction), " bytes");
  c10::cuda::CUDAGuard guard(v.device());
  uint8_t* base = static_cast<uint8_t*>(scratch_for(v, 16384 + cuda::sparse_scratch_bytes(n)));
  cuda::SparseFuse fuse;
  fuse.mode = 2;
  fuse.grad = grad.data_ptr<float>();
  fuse.u = u.data_ptr<float>();
  fuse.momentum = float(momentum);
  fuse.clip = float(clip);
  fuse.sumsq = reinterpret_cast<float*>(base + 12288);
  fuse.zero_grad = zero_grad ? 1 : 0;
  HP_CHECK_CUDA(cuda::sparse_compress_fused(fuse, v.data_ptr<float>(), n, sample_rate, keep_fraction, uint64_t(seed),
                                            local_target(out), base + 16384, at::cuda::getCurrentCUDAStream()));
}

void sparse_decompress(const std::vector<torch::Tensor>& payloads, torch::Tensor out, bool add,
                       double post_scale) {
  check_f32(out, "out");
  const int64_t n = out.numel();
  TORCH_CHECK(n > 0, "empty tensor");
  if (out.is_cuda()) {
    c10::cuda::CUDAGuard guard(out.device());
    HP_CHECK_CUDA(cuda::sparse_unpack_accum(sources_of(payloads, out), out.data_ptr<float>(), n,
                                            add ? 1 : 0, float(post_scale), status_word_for(out),
                                            at::cuda::getCurrentCUDAStream()));
  } else {
    TORCH_CHECK(!payloads.empty(), "at least one payload expected");
    if (!add) out.zero_();
    for (size_t r = 0; r < payloads.size(); ++r) {
      check_u8(payloads[r], "payload");
      if (post_scale == 1.0) {
        const int64_t k = cpu::sparse_decompress(payloads[r].data_ptr<uint8_t>(),
                                                 payloads[r].numel(), out.data_ptr<float>(), n, 1);
        TORCH_CHECK(k >= 0, "malformed sparse payload ", r);
      } else {
        // scaled accumulation: out[idx] += val * scale, like the kernel
        auto tmp = torch::zeros_like(out);
        const int64_t k = cpu::sparse_decompress(payloads[r].data_ptr<uint8_t>(),
                                                 payloads[r].numel(), tmp.data_ptr<float>(), n, 0);
        TORCH_CHECK(k >= 0, "malformed sparse payload ", r);
        float* o = out.data_ptr<float>();
        const float* t = tmp.data_ptr<float>();
        for (int64_t i = 0; i < n; ++i)
          if (t[i] != 0.0f) o[i] = hp_add(o[i], hp_mul(t[i], float(post_scale)));
      }
    }
  }
}

// ------------------------------------------------------------------ ECQ
void ecq_compress(const torch::Tensor& grad, torch::Tensor history, torch::Tensor out, double alpha,
                  double beta, int64_t bitwidth, int64_t seed) {
  check_f32(grad, "grad");
  check_f32(history, "history");
  check_u8(out, "out");
  check_same_device(grad, history);
  check_same_device(grad, out);
  const int64_t n = grad.numel();
  TORCH_CHECK(n > 0, "empty tensor");
  TORCH_CHECK(history.numel() == n, "history must have as many elements as grad");
  TORCH_CHECK(ecq_bitwidth_ok(int(bitwidth)), "bitwidth must be 2, 4 or 8");
  TORCH_CHECK(out.numel() == hipress::ecq_payload_bytes(n, int(bitwidth)), "out must have exactly ",
              hipress::ecq_payload_bytes(n, int(bitwidth)), " bytes");
  if (grad.is_cuda()) {
    c10::cuda::CUDAGuard guard(grad.device());
    void* scratch = scratch_for(grad, cuda::minmax_scratch_bytes());
    HP_CHECK_CUDA(cuda::ecq_compress(grad.data_ptr<float>(), history.data_ptr<float>(), n,
                                     float(alpha), float(beta), int(bitwidth), uint64_t(seed),
                                     local_target(out), scratch, at::cuda::getCurrentCUDAStream()));
  } else {
    const int rc = cpu::ecq_compress(grad.data_ptr<float>(), history.data_ptr<float>(), n,
                                     float(alpha), float(beta), int(bitwidth), uint64_t(seed),
                                     out.data_ptr<uint8_t>(), out.numel());
    TORCH_CHECK(rc == 0, "ecq_compress failed");
  }
}

void ecq_decompress(const std::vector<torch::Tensor>& payloads, torch::Tensor out, bool add,
                    double post_scale) {
  check_f32(out, "out");
  const int64_t n = out.numel();
  TORCH_CHECK(n > 0, "empty tensor");
  if (out.is_cuda()) {
    c10::cuda::CUDAGuard guard(out.device());
    HP_CHECK_CUDA(cuda::ecq_unpack_accum(sources_of(payloads, out), out.data_ptr<float>(), n,
                                         add ? 1 : 0, float(post_scale), status_word_for(out),
                                         at::cuda::getCurrentCUDAStream()));
  } else {
    TORCH_CHECK(!payloads.empty(), "at least one payload expected");
    for (size_t r = 0; r < payloads.size(); ++r) {
      check_u8(payloads[r], "payload");
      const int64_t cnt = cpu::ecq_decompress(payloads[r].data_ptr<uint8_t>(), payloads[r].numel(),
                                              out.data_ptr<float>(), n, (add || r > 0) ? 1 : 0);
      TORCH_CHECK(cnt == n, "payload ", r, " decodes to ", cnt, " elements, expected ", n);
    }
    if (post_scale != 1.0) {
      float* o = out.data_ptr<float>();
      for (int64_t i = 0; i < n; ++i) o[i] = hp_mul(o[i], float(post_scale));
    }
  }
}

// ------------------------------------------------------------------ PowerSGD
namespace {
struct PsgdShape {
  int64_t n, m, r;
};
PsgdShape psgd_shape(const torch::Tensor& M, const torch::Tensor& P, const torch::Tensor& Q) {
  check_f32(M, "M");
  check_f32(P, "P");
  check_f32(Q, "Q");
  TORCH_CHECK(M.dim() == 2 && P.dim() == 2 && Q.dim() == 2, "M, P, Q must be matrices");
  PsgdShape s{M.size(0), M.size(1), P.size(1)};
  TORCH_CHECK(P.size(0) == s.n && Q.size(0) == s.m && Q.size(1) == s.r,
              "shapes must be M[n,m], P[n,r], Q[m,r]");
  TORCH_CHECK(s.r >= 1 && s.r <= 16, "rank must be between 1 and 16");
  check_same_device(M, P);
  check_same_device(M, Q);
  return s;
}
}  // namespace

void psgd_project(int64_t mode, const torch::Tensor& M, const torch::Tensor& X,
                  const std::vector<torch::Tensor>& owners, bool simt) {
  check_f32(M, "M");
  check_f32(X, "X");
  TORCH_CHECK(mode == 0 || mode == 1, "mode must be 0 or 1");
  TORCH_CHECK(M.dim() == 2 && X.dim() == 2, "M and X must be matrices");
  const int64_t n = M.size(0), m = M.size(1), r = X.size(1);
  const int64_t k = mode == 0 ? m : n, out_rows = mode == 0 ? n : m;
  TORCH_CHECK(X.size(0) == k, "X must have ", k, " rows");
  TORCH_CHECK(r >= 1 && r <= 16, "rank must be between 1 and 16");
  TORCH_CHECK(!owners.empty() && owners.size() <= size_t(cuda::kMaxWorld), "1..8 owner tensors expected");
  for (auto& o : owners) {
    check_f32(o, "owner");
    TORCH_CHECK(o.numel() == out_rows * r, "owner tensors must have the output's shape");
  }
  if (M.is_cuda()) {
    c10::cuda::CUDAGuard guard(M.device());
    auto stream = at::cuda::getCurrentCUDAStream();
    cuda::ReduceTargets red;
    red.world = int(owners.size());
    for (size_t p = 0; p < owners.size(); ++p) red.dst[p] = owners[p].data_ptr<float>();
    torch::Tensor xt;
    const float* xt_ptr = nullptr;
    if (!simt && cuda::psgd_tensor_core_eligible(M.data_ptr<float>(), n, m)) {
      const int64_t kp = cuda::psgd_kpad(k);
      xt = torch::empty({16, kp}, M.options());
      HP_CHECK_CUDA(cuda::psgd_transpose_pad(X.data_ptr<float>(), k, int(r), xt.data_ptr<float>(), kp, stream));
      xt_ptr = xt.data_ptr<float>();
    }
    HP_CHECK_CUDA(cuda::psgd_gemm(int(mode), M.data_ptr<float>(), n, m, X.data_ptr<float>(), xt_ptr,
                                  int(r), red, simt ? 1 : 0, status_word_for(M), stream));
  } else {
    TORCH_CHECK(owners.size() == 1, "CPU path supports a single owner");
    auto out = owners[0].view({out_rows, r});
    out.add_(mode == 0 ? at::mm(M, X) : at::mm(M.t(), X));
  }
}

void psgd_project_grouped(int64_t mode, const std::vector<torch::Tensor>& Ms, const std::vector<torch::Tensor>& Xs,
                          const std::vector<torch::Tensor>& outs) {
  TORCH_CHECK(mode == 0 || mode == 1, "mode must be 0 or 1");
  TORCH_CHECK(!Ms.empty() && Ms.size() == Xs.size() && Ms.size() == outs.size(), "one X and one output per matrix");
  TORCH_CHECK(Ms[0].is_cuda(), "CUDA tensors expected");
  c10::cuda::CUDAGuard guard(Ms[0].device());
  auto stream = at::cuda::getCurrentCUDAStream();
  const int64_t r = Xs[0].size(1);
  TORCH_CHECK(r >= 1 && r <= 16, "rank must be between 1 and 16");
  std::vector<cuda::PsgdGemmItem> items(Ms.size());
  std::vector<cuda::PsgdTransposeItem> transposes;
  std::vector<torch::Tensor> keep;
  for (size_t i = 0; i < Ms.size(); ++i) {
    const torch::Tensor& M = Ms[i];
    check_f32(M, "M");
    check_f32(Xs[i], "X");
    check_f32(outs[i], "out");
    TORCH_CHECK(M.dim() == 2 && Xs[i].dim() == 2 && Xs[i].size(1) == r, "matrices of one rank expected");
    const int64_t n = M.size(0), m = M.size(1);
    const int64_t k = mode == 0 ? m : n, out_rows = mode == 0 ? n : m;
    TORCH_CHECK(Xs[i].size(0) == k && outs[i].numel() == out_rows * r, "shape mismatch at matrix ", i);
    cuda::PsgdGemmItem& it = items[i];
    it.Mat = M.data_ptr<float>();
    it.n = n;
    it.m = m;
    it.X = Xs[i].data_ptr<float>();
    it.red.world = 1;
    it.red.dst[0] = outs[i].data_ptr<float>();
    if (cuda::psgd_tensor_core_eligible(it.Mat, n, m)) {
      const int64_t kp = cuda::psgd_kpad(k);
      keep.push_back(torch::empty({16, kp}, M.options()));
      it.Xt = keep.back().data_ptr<float>();
      transposes.push_back(cuda::PsgdTransposeItem{it.X, keep.back().data_ptr<float>(), k, kp, int(r)});
    }
  }
  if (!transposes.empty())
    HP_CHECK_CUDA(cuda::psgd_transpose_pad_batched(transposes.data(), int(transposes.size()), stream));
  HP_CHECK_CUDA(cuda::psgd_gemm_grouped(int(mode), items.data(), int(items.size()), int(r), status_word_for(Ms[0]),
                                        nullptr, stream));
}

void gram_schmidt(torch::Tensor P, double eps) {
  check_f32(P, "P");
  TORCH_CHECK(P.dim() == 2 && P.size(1) >= 1 && P.size(1) <= 16, "P must be n x r with r <= 16");
  if (P.is_cuda()) {
    c10::cuda::CUDAGuard guard(P.device());
    HP_CHECK_CUDA(cuda::gram_schmidt(P.data_ptr<float>(), P.size(0), int(P.size(1)), float(eps),
                                     at::cuda::getCurrentCUDAStream()));
  } else {
    cpu::gram_schmidt(P.data_ptr<float>(), P.size(0), P.size(1), float(eps));
  }
}

void psgd_expand_feedback(const torch::Tensor& P, const torch::Tensor& Q, torch::Tensor M,
                          torch::Tensor grad_out, double post_scale) {
  const PsgdShape s = psgd_shape(M, P, Q);
  check_f32(grad_out, "grad_out");
  const int64_t N = grad_out.numel();
  TORCH_CHECK(N <= s.n * s.m, "grad_out has more elements than M");
  if (M.is_cuda()) {
    c10::cuda::CUDAGuard guard(M.device());
    HP_CHECK_CUDA(cuda::psgd_expand_residual(P.data_ptr<float>(), Q.data_ptr<float>(), s.n, s.m,
                                             int(s.r), M.data_ptr<float>(), nullptr,
                                             grad_out.data_ptr<float>(), N, 1, float(post_scale),
                                             at::cuda::getCurrentCUDAStream()));
  } else {
    auto approx = at::mm(P, Q.t());
    M.sub_(approx);
    grad_out.view(-1).copy_(approx.view(-1).slice(0, 0, N) * post_scale);
  }
}

void psgd_owner_gather(const std::vector<torch::Tensor>& owners, torch::Tensor out, double scale) {
  check_f32(out, "out");
  TORCH_CHECK(out.dim() == 2, "out must be rows x r");
  TORCH_CHECK(!owners.empty() && owners.size() <= size_t(cuda::kMaxWorld), "1..8 owner tensors expected");
  TORCH_CHECK(out.is_cuda(), "CUDA tensors expected");
  cuda::ReduceTargets red;
  red.world = int(owners.size());
  for (size_t p = 0; p < owners.size(); ++p) {
    check_f32(owners[p], "owner");
    TORCH_CHECK(owners[p].numel() == out.numel(), "owner tensors must have out's shape");
    red.dst[p] = owners[p].data_ptr<float>();
  }
  c10::cuda::CUDAGuard guard(out.device());
  HP_CHECK_CUDA(cuda::psgd_owner_gather(red, out.size(0), int(out.size(1)), out.data_ptr<float>(),
                                        float(scale), at::cuda::getCurrentCUDAStream()));
}

void psgd_expand_sgd(const torch::Tensor& P, const torch::Tensor& Q, torch::Tensor M,
                     torch::Tensor param, torch::Tensor momentum, double post_scale, double lr,
                     double mu, double weight_decay, bool first_step) {
  const PsgdShape s = psgd_shape(M, P, Q);
  TORCH_CHECK(M.is_cuda(), "CUDA tensors expected");
  TORCH_CHECK(param.scalar_type() == torch::kFloat32 && momentum.scalar_type() == torch::kFloat32,
              "param and momentum must be float32");
  const int64_t N = param.numel();
  TORCH_CHECK(momentum.numel() == N && N <= s.n * s.m, "param/momentum must fit in M");
  cuda::SgdApply a;
  a.param = param.data_ptr<float>();
  a.momentum = momentum.data_ptr<float>();
  a.lr = float(lr);
  a.mu = float(mu);
  a.weight_decay = float(weight_decay);
  a.first_step = first_step ? 1 : 0;
  c10::cuda::CUDAGuard guard(M.device());
  HP_CHECK_CUDA(cuda::psgd_expand_sgd(P.data_ptr<float>(), Q.data_ptr<float>(), s.n, s.m, int(s.r),
                                      M.data_ptr<float>(), N, float(post_scale), a,
                                      at::cuda::getCurrentCUDAStream()));
}

void psgd_expand_sgd_grouped(const std::vector<torch::Tensor>& Ps, const std::vector<torch::Tensor>& Qs,
                             const std::vector<torch::Tensor>& Ms, const std::vector<torch::Tensor>& params,
                             const std::vector<torch::Tensor>& momenta, double post_scale, double lr, double mu,
                             double weight_decay, bool first_step) {
  const size_t count = Ms.size();
  TORCH_CHECK(count > 0 && Ps.size() == count && Qs.size() == count && params.size() == count &&
                  momenta.size() == count,
              "one P, Q, param and momentum per matrix");
  TORCH_CHECK(Ms[0].is_cuda(), "CUDA tensors expected");
  std::vector<cuda::PsgdExpandItem> items(count);
  int64_t r = -1;
  for (size_t i = 0; i < count; ++i) {
    const PsgdShape s = psgd_shape(Ms[i], Ps[i], Qs[i]);
    TORCH_CHECK(r < 0 || r == s.r, "matrices of one rank expected");
    r = s.r;
    TORCH_CHECK(params[i].scalar_type() == torch::kFloat32 && momenta[i].scalar_type() == torch::kFloat32,
                "param and momentum must be float32");
    const int64_t N = params[i].numel();
    TORCH_CHECK(momenta[i].numel() == N && N <= s.n * s.m, "param/momentum must fit in M");
    cuda::PsgdExpandItem& it = items[i];
    it.P = Ps[i].data_ptr<float>();
    it.Q = Qs[i].data_ptr<float>();
    it.n = s.n;
    it.m = s.m;
    it.N = N;
    it.Mat = Ms[i].data_ptr<float>();
    it.param = params[i].data_ptr<float>();
    it.momentum = momenta[i].data_ptr<float>();
  }
  cuda::SgdApply common;
  common.lr = float(lr);
  common.mu = float(mu);
  common.weight_decay = float(weight_decay);
  common.first_step = first_step ? 1 : 0;
  c10::cuda::CUDAGuard guard(Ms[0].device());
  HP_CHECK_CUDA(cuda::psgd_expand_sgd_grouped(items.data(), int(count), int(r), float(post_scale), common, nullptr,
                                              at::cuda::getCurrentCUDAStream()));
}

void powersgd_encode1(const torch::Tensor& grad, const torch::Tensor& residual,
                      const torch::Tensor& Q, torch::Tensor M, torch::Tensor P) {
  const PsgdShape s = psgd_shape(M, P, Q);
  check_f32(grad, "grad");
  check_f32(residual, "residual");
  const int64_t N = grad.numel();
  TORCH_CHECK(residual.numel() == N && N <= s.n * s.m, "grad/residual must fit in M");
  if (M.is_cuda()) {
    c10::cuda::CUDAGuard guard(M.device());
    HP_CHECK_CUDA(cuda::add_into(grad.data_ptr<float>(), residual.data_ptr<float>(),
                                 M.data_ptr<float>(), N, at::cuda::getCurrentCUDAStream()));
    P.zero_();
    psgd_project(0, M, Q, {P}, false);
  } else {
    cpu::powersgd_encode1(grad.data_ptr<float>(), residual.data_ptr<float>(), N, M.data_ptr<float>(),
                          s.n, s.m, Q.data_ptr<float>(), s.r, P.data_ptr<float>());
  }
}

void powersgd_encode2(torch::Tensor P, const torch::Tensor& M, torch::Tensor Q) {
  const PsgdShape s = psgd_shape(M, P, Q);
  if (M.is_cuda()) {
    gram_schmidt(P, 1e-8);
    Q.zero_();
    psgd_project(1, M, P, {Q}, false);
  } else {
    cpu::powersgd_encode2(P.data_ptr<float>(), M.data_ptr<float>(), s.n, s.m, s.r, Q.data_ptr<float>());
  }
}

void powersgd_decode(const torch::Tensor& P, const torch::Tensor& Q, torch::Tensor M,
                     torch::Tensor residual, torch::Tensor grad) {
  const PsgdShape s = psgd_shape(M, P, Q);
  check_f32(grad, "grad");
  check_f32(residual, "residual");
  const int64_t N = grad.numel();
  TORCH_CHECK(residual.numel() == N && N <= s.n * s.m, "grad/residual must fit in M");
  if (M.is_cuda()) {
    c10::cuda::CUDAGuard guard(M.device());
    HP_CHECK_CUDA(cuda::psgd_expand_residual(P.data_ptr<float>(), Q.data_ptr<float>(), s.n, s.m,
                                             int(s.r), M.data_ptr<float>(), residual.data_ptr<float>(),
                                             grad.data_ptr<float>(), N, 0, 1.0f,
                                             at::cuda::getCurrentCUDAStream()));
  } else {
    cpu::powersgd_decode(P.data_ptr<float>(), Q.data_ptr<float>(), s.n, s.m, s.r, M.data_ptr<float>(),
                         residual.data_ptr<float>(), grad.data_ptr<float>(), N);
  }
}

}  // namespace ops
}  // namespace hipress
