// Python module hipress_b200._C.
//
// Parity surface (ref hp_cuda.cpp:1073-1080): init, end, getResults and the
// three submit_task overloads.  On top of it: the per-algorithm tensor ops, the
// symmetric-memory buffer, the data-parallel engine and a few probes.
#include <torch/extension.h>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <pybind11/stl.h>

#include <cstring>

#include "codec_cpu/codec_cpu.h"
#include "comm/symm_mem.h"
#include "common/codec_math.h"
#include "common/host_utils.h"
#include "common/lcg.h"
#include "kernels/kernels.h"
#include "ops/ops.h"
#include "runtime/ddp_engine.h"
#include "runtime/psgd_engine.h"
#include "runtime/task_runtime.h"

#define HP_CHECK_CUDA(e)                                                                      \
  do {                                                                                        \
    cudaError_t _e = (e);                                                                     \
    TORCH_CHECK(_e == cudaSuccess, "hipress kernel launch failed: ", cudaGetErrorString(_e)); \
  } while (0)

namespace py = pybind11;
using namespace hipress;

namespace {

cudaStream_t current_stream(int device) { return at::cuda::getCurrentCUDAStream(device).stream(); }

torch::Tensor symm_tensor(comm::SymmetricBuffer& buf, int rank, int64_t byte_offset, int64_t numel,
                          const std::string& dtype, int device) {
  torch::ScalarType st = dtype == "float32" ? torch::kFloat32
                       : dtype == "uint8"   ? torch::kUInt8
                       : dtype == "int32"   ? torch::kInt32
                                            : torch::kUInt8;
  const int64_t esz = int64_t(c10::elementSize(st));
  TORCH_CHECK(byte_offset >= 0 && byte_offset + numel * esz <= int64_t(buf.bytes()), "view out of range");
  auto opts = torch::TensorOptions().dtype(st).device(torch::kCUDA, device);
  return torch::from_blob(buf.base(rank) + byte_offset, {numel}, opts);
}

runtime::EngineConfig config_from(const py::dict& d) {
  runtime::EngineConfig c;
  auto get = [&](const char* k, auto dflt) {
    using T = decltype(dflt);
    return d.contains(k) ? d[k].cast<T>() : dflt;
  };
  c.rank = get("rank", 0);
  c.world = get("world", 1);
  c.device = get("device", 0);
  const std::string codec = get("codec", std::string("terngrad"));
  if (codec == "dense") c.codec = runtime::Codec::kDense;
  else if (codec == "tbq") c.codec = runtime::Codec::kTbq;
  else if (codec == "terngrad") c.codec = runtime::Codec::kTernGrad;
  else if (codec == "graddrop" || codec == "dgc" || codec == "sparse") c.codec = runtime::Codec::kSparse;
  else if (codec == "ecq") c.codec = runtime::Codec::kEcq;
  else throw std::invalid_argument("unknown codec " + codec);
  c.threshold = get("threshold", 0.0f);
  c.bitwidth = get("bitwidth", 2);
  c.enable_random = get("enable_random", 1);
  c.error_feedback = get("error_feedback", 1);
  c.sample_rate = get("sample_rate", 0.01);
  c.keep_fraction = get("keep_fraction", 0.001);
  c.sparse_accumulate = get("sparse_accumulate", codec == "dgc" ? 0 : 1);
  c.alpha = get("alpha", 1.0f);
  c.beta = get("beta", 1.0f);
  c.seed = get("seed", uint64_t(1));
  c.average = get("average", 1);
  c.flag_timeout_ns = uint64_t(get("flag_timeout_s", 20.0) * 1e9);
  c.num_workers = get("num_workers", 1);
  c.defer_recv = get("defer_recv", 0);
  c.clear_grad = get("clear_grad", 0);
  c.device_epoch = get("device_epoch", 0);
  c.sharded = get("sharded", 0);
  c.trace = get("trace", 0);
  c.nvls = get("nvls", 0);
  c.momentum_correction = get("momentum_correction", 0);
  c.dgc_momentum = get("dgc_momentum", 0.9f);
  c.dgc_clip = get("dgc_clip", 0.0f);
  return c;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "hipress_b200 native extension (sm_100a kernels, CPU codecs, runtime)";

  // ---------------------------------------------------------------- parity API
  m.def("init",
        [](const std::string& alg, std::unordered_map<std::string, double> params, int device_id,
           int rank_id, int size) {
          return runtime::TaskRuntime::instance().init(alg, std::move(params), device_id, rank_id, size);
        },
        "init(alg_name, alg_paras, device_id, rank_id, size) -> bool", py::arg("alg_name"),
        py::arg("alg_paras"), py::arg("device_id"), py::arg("rank_id"), py::arg("size"));
  m.def("end", [] {
    py::gil_scoped_release nogil;
    return runtime::TaskRuntime::instance().end();
  });
  m.def("getResults", [](int task_id) { return runtime::TaskRuntime::instance().get_results(task_id); });
  m.def("getErrors", [] { return runtime::TaskRuntime::instance().get_errors(); });
  m.def("numThreads", [] { return runtime::TaskRuntime::instance().num_threads(); });
  m.def("submit_task",
        [](const std::string& name, torch::Tensor tensor, torch::Tensor B, torch::Tensor C, int is_root,
           int task_id) {
          return runtime::TaskRuntime::instance().submit_without_residual(name, tensor, B, C, is_root, task_id);
        },
        "submit_task without residual");
  m.def("submit_task",
        [](const std::string& name, torch::Tensor tensor, torch::Tensor residual, torch::Tensor B,
           torch::Tensor C, int is_root, int task_id) {
          return runtime::TaskRuntime::instance().submit_with_residual(name, tensor, residual, B, C, is_root, task_id);
        },
        "submit_task with residual");
  m.def("submit_task",
        [](const std::string& name, torch::Tensor tensor, torch::Tensor residual, torch::Tensor M,
           torch::Tensor P, torch::Tensor Q, int task_id) {
          return runtime::TaskRuntime::instance().submit_powersgd(name, tensor, residual, M, P, Q, task_id);
        },
        "submit_task for powersgd");
  m.attr("COMP_TASK") = runtime::kCompTask;
  m.attr("DECOMP_TASK") = runtime::kDecompTask;
  m.attr("ROOT_DECOMP_COMP_TASK") = runtime::kRootDecompCompTask;
  m.attr("POWERSGD_ENCODE1") = runtime::kPowerSgdEncode1;
  m.attr("POWERSGD_ENCODE2") = runtime::kPowerSgdEncode2;
  m.attr("POWERSGD_DECODE") = runtime::kPowerSgdDecode;

  // ---------------------------------------------------------------- codec ops
  m.def("tbq_payload_bytes", &ops::tbq_payload_bytes);
  m.def("terngrad_payload_bytes", &ops::terngrad_payload_bytes);
  m.def("sparse_payload_bytes", &ops::sparse_payload_bytes);
  m.def("ecq_payload_bytes", &ops::ecq_payload_bytes);
  m.def("tbq_compress", &ops::tbq_compress, py::arg("grad"), py::arg("residual"), py::arg("out"),
        py::arg("threshold"));
  m.def("tbq_decompress", &ops::tbq_decompress, py::arg("payloads"), py::arg("out"),
        py::arg("threshold"), py::arg("add") = false, py::arg("post_scale") = 1.0);
  m.def("terngrad_compress", &ops::terngrad_compress, py::arg("grad"), py::arg("out"),
        py::arg("bitwidth"), py::arg("enable_random"), py::arg("seed"),
        py::arg("residual") = py::none());
  m.def("terngrad_decompress", &ops::terngrad_decompress, py::arg("payloads"), py::arg("out"),
        py::arg("add") = false, py::arg("post_scale") = 1.0, py::arg("bitwidth") = 0);
  m.def("dgc_momentum_compress", &ops::dgc_momentum_compress, py::arg("grad"), py::arg("u"), py::arg("v"),
        py::arg("out"), py::arg("sample_rate"), py::arg("keep_fraction"), py::arg("seed"), py::arg("momentum"),
        py::arg("clip") = 0.0, py::arg("zero_grad") = false);
  m.def("sparse_compress", &ops::sparse_compress, py::arg("grad"), py::arg("R"), py::arg("out"),
        py::arg("sample_rate"), py::arg("keep_fraction"), py::arg("seed"), py::arg("accumulate"));
  m.def("sparse_decompress", &ops::sparse_decompress, py::arg("payloads"), py::arg("out"),
        py::arg("add") = false, py::arg("post_scale") = 1.0);
  m.def("ecq_compress", &ops::ecq_compress, py::arg("grad"), py::arg("history"), py::arg("out"),
        py::arg("alpha"), py::arg("beta"), py::arg("bitwidth"), py::arg("seed"));
  m.def("ecq_decompress", &ops::ecq_decompress, py::arg("payloads"), py::arg("out"),
        py::arg("add") = false, py::arg("post_scale") = 1.0);
  m.def("powersgd_encode1", &ops::powersgd_encode1);
  m.def("powersgd_encode2", &ops::powersgd_encode2);
  m.def("powersgd_decode", &ops::powersgd_decode);
  m.def("psgd_project_grouped", &ops::psgd_project_grouped, py::arg("mode"), py::arg("Ms"), py::arg("Xs"), py::arg("outs"));
  m.def("psgd_project", &ops::psgd_project, py::arg("mode"), py::arg("M"), py::arg("X"),
        py::arg("owners"), py::arg("simt") = false);
  m.def("bn_supported", &ops::bn_supported, py::arg("x"));
  m.def("bn_forward", &ops::bn_forward, py::arg("x"), py::arg("residual"), py::arg("weight"), py::arg("bias"),
        py::arg("running_mean"), py::arg("running_var"), py::arg("num_batches"), py::arg("momentum"),
        py::arg("eps"), py::arg("relu"));
  m.def("bn_backward", &ops::bn_backward, py::arg("dy"), py::arg("x"), py::arg("y"), py::arg("weight"),
        py::arg("stats"), py::arg("relu"), py::arg("want_dres"));
  m.def("maxpool_supported", &ops::maxpool_supported, py::arg("x"));
  m.def("maxpool3x3s2_forward", &ops::maxpool3x3s2_forward, py::arg("x"));
  m.def("maxpool3x3s2_backward", &ops::maxpool3x3s2_backward, py::arg("dy"), py::arg("idx"), py::arg("h"),
        py::arg("w"));
  m.def("bias_relu_supported", &ops::bias_relu_supported, py::arg("x"), py::arg("pool"));
  m.def("bias_relu_forward", &ops::bias_relu_forward, py::arg("x"), py::arg("bias"), py::arg("pool"));
  m.def("bias_relu_backward", &ops::bias_relu_backward, py::arg("dy"), py::arg("y"), py::arg("idx"),
        py::arg("pool"));
  m.def("add_ln_supported", &ops::add_ln_supported, py::arg("x"));
  m.def("add_ln_forward", &ops::add_ln_forward, py::arg("x"), py::arg("delta"), py::arg("weight"), py::arg("bias"),
        py::arg("eps"));
  m.def("add_ln_backward", &ops::add_ln_backward, py::arg("dy"), py::arg("z"), py::arg("stats"), py::arg("weight"));
  m.def("set_cpu_threads", &cpu::set_threads, py::arg("threads"));
  m.def("get_cpu_threads", &cpu::get_threads);
  m.def("linear_wgrad_bgrad", &ops::linear_wgrad_bgrad, py::arg("dy"), py::arg("x"));
  m.def("colsum_supported", &ops::colsum_supported, py::arg("dy"));
  m.def("colsum", &ops::colsum, py::arg("dy"));
  m.def("psgd_kpad", &cuda::psgd_kpad, py::arg("k"));
  m.def("gram_schmidt", &ops::gram_schmidt, py::arg("P"), py::arg("eps") = 1e-8);
  m.def("psgd_expand_feedback", &ops::psgd_expand_feedback, py::arg("P"), py::arg("Q"), py::arg("M"),
        py::arg("grad_out"), py::arg("post_scale") = 1.0);
  m.def("psgd_owner_gather", &ops::psgd_owner_gather, py::arg("owners"), py::arg("out"),
        py::arg("scale") = 1.0);
  m.def("psgd_expand_sgd", &ops::psgd_expand_sgd, py::arg("P"), py::arg("Q"), py::arg("M"),
        py::arg("param"), py::arg("momentum"), py::arg("post_scale"), py::arg("lr"), py::arg("mu"),
        py::arg("weight_decay"), py::arg("first_step"));
  m.def("psgd_expand_sgd_grouped", &ops::psgd_expand_sgd_grouped, py::arg("Ps"), py::arg("Qs"), py::arg("Ms"),
        py::arg("params"), py::arg("momenta"), py::arg("post_scale"), py::arg("lr"), py::arg("mu"),
        py::arg("weight_decay"), py::arg("first_step"));
  m.def("read_status", &ops::read_status, py::arg("like"), py::arg("reset") = true);

  // fused SGD-momentum over flat fp32 buffers
  m.def("sgd_apply",
        [](torch::Tensor grad, torch::Tensor param, torch::Tensor momentum, double scale, double lr,
           double mu, double wd, bool first_step, bool clear_grad) {
          TORCH_CHECK(grad.is_cuda() && param.is_cuda() && momentum.is_cuda(), "CUDA tensors expected");
          TORCH_CHECK(grad.numel() == param.numel() && grad.numel() == momentum.numel(), "size mismatch");
          c10::cuda::CUDAGuard guard(grad.device());
          cuda::SgdApply a;
          a.param = param.data_ptr<float>();
          a.momentum = momentum.data_ptr<float>();
          a.lr = float(lr);
          a.mu = float(mu);
          a.weight_decay = float(wd);
          a.first_step = first_step ? 1 : 0;
          a.clear_grad = clear_grad ? 1 : 0;
          cudaError_t e = cuda::sgd_apply_dense(grad.data_ptr<float>(), float(scale), a, grad.numel(),
                                                current_stream(grad.get_device()));
          TORCH_CHECK(e == cudaSuccess, cudaGetErrorString(e));
        },
        py::arg("grad"), py::arg("param"), py::arg("momentum"), py::arg("scale"), py::arg("lr"),
        py::arg("mu"), py::arg("weight_decay"), py::arg("first_step"), py::arg("clear_grad") = false);

  // fused AdamW (decoupled weight decay, bias correction) over flat fp32 buffers; step is 1-based
  m.def("adamw_apply",
        [](torch::Tensor grad, torch::Tensor param, torch::Tensor exp_avg, torch::Tensor exp_avg_sq,
           double scale, double lr, double beta1, double beta2, double eps, double wd, int64_t step,
           bool clear_grad) {
          TORCH_CHECK(grad.is_cuda() && param.is_cuda() && exp_avg.is_cuda() && exp_avg_sq.is_cuda(),
                      "CUDA tensors expected");
          TORCH_CHECK(grad.numel() == param.numel() && grad.numel() == exp_avg.numel() &&
                      grad.numel() == exp_avg_sq.numel(), "size mismatch");
          c10::cuda::CUDAGuard guard(grad.device());
          cuda::AdamWApply a;
          a.param = param.data_ptr<float>();
          a.exp_avg = exp_avg.data_ptr<float>();
          a.exp_avg_sq = exp_avg_sq.data_ptr<float>();
          a.lr = float(lr);
          a.beta1 = float(beta1);
          a.beta2 = float(beta2);
          a.eps = float(eps);
          a.weight_decay = float(wd);
          a.step = int(step);
          a.clear_grad = clear_grad ? 1 : 0;
          cudaError_t e = cuda::adamw_apply_dense(grad.data_ptr<float>(), float(scale), a, grad.numel(),
                                                  current_stream(grad.get_device()));
          TORCH_CHECK(e == cudaSuccess, cudaGetErrorString(e));
        },
        py::arg("grad"), py::arg("param"), py::arg("exp_avg"), py::arg("exp_avg_sq"), py::arg("scale"),
        py::arg("lr"), py::arg("beta1"), py::arg("beta2"), py::arg("eps"), py::arg("weight_decay"),
        py::arg("step"), py::arg("clear_grad") = false);

  // LCG draws, for checking the generator against the reference's
  m.def("lcg_draws", [](uint32_t seed, int count) {
    std::vector<std::pair<uint32_t, float>> out;
    Lcg32 a(seed), b(seed);
    for (int i = 0; i < count; ++i) out.emplace_back(a.next_below(0x7fffffffu), b.next_unit());
    return out;
  });

  // number of raw values in [start, start + count*stride) for which the reciprocal-multiply
  // form of the unit draw differs from the reference's division form (expected: 0)
  m.def("lcg_unit_mismatches", [](uint64_t start, uint64_t count, uint64_t stride) {
    uint64_t bad = 0;
    for (uint64_t i = 0; i < count; ++i) {
      const uint32_t raw = uint32_t(start + i * stride);
      const float a = Lcg32::unit_from_raw(raw), b = Lcg32::unit_from_raw_by_division(raw);
      bad += std::memcmp(&a, &b, 4) != 0;
    }
    return bad;
  });

  // support-layer utilities (branch-free abs, wall-clock checkpoint timer)
  m.def("fast_abs_i32", [](int32_t v) { return fast_abs(v); });
  m.def("fast_abs_i64", [](int64_t v) { return fast_abs(v); });
  m.def("fast_abs_f32", [](float v) { return fast_abs(v); });
  m.def("fast_abs_f64", [](double v) { return fast_abs(v); });
  py::class_<TimeCost>(m, "TimeCost")
      .def(py::init<>())
      .def("start", &TimeCost::start)
      .def("record", &TimeCost::record)
      .def("intervals", &TimeCost::intervals, py::arg("per_second") = 1e6)
      .def("print_by_us", &TimeCost::print_by_us)
      .def("print_by_ms", &TimeCost::print_by_ms)
      .def("print_by_s", &TimeCost::print_by_s);

  // ---------------------------------------------------------------- probes
  m.def("can_access_peer", &comm::can_access_peer);
  m.def("multicast_supported", &comm::multicast_supported);
  m.def("psgd_tensor_core_eligible", [](const torch::Tensor& M) {
    return M.is_cuda() && M.dim() == 2 && cuda::psgd_tensor_core_eligible(M.data_ptr<float>(), M.size(0), M.size(1));
  });

  // ---------------------------------------------------------------- symmetric memory
  py::class_<comm::SymmetricBuffer>(m, "SymmetricBuffer")
      .def(py::init([](int64_t bytes, int rank, int world, int device) {
             c10::cuda::CUDAGuard guard(c10::Device(c10::kCUDA, device));
             return std::make_unique<comm::SymmetricBuffer>(size_t(bytes), rank, world);
           }),
           py::arg("bytes"), py::arg("rank"), py::arg("world"), py::arg("device"))
      .def(py::init([](const std::vector<uint64_t>& bases, uint64_t multicast, int64_t bytes, int rank, int world) {
             return std::make_unique<comm::SymmetricBuffer>(bases, multicast, size_t(bytes), rank, world);
           }),
           py::arg("bases"), py::arg("multicast"), py::arg("bytes"), py::arg("rank"), py::arg("world"))
      .def_property_readonly("multicast",
                             [](comm::SymmetricBuffer& b) { return uint64_t(reinterpret_cast<uintptr_t>(b.multicast())); })
      .def("export_handle", [](comm::SymmetricBuffer& b) { return py::bytes(b.export_handle()); })
      .def("open_peers",
           [](comm::SymmetricBuffer& b, const std::vector<py::bytes>& handles) {
             std::vector<std::string> hs;
             for (auto& h : handles) hs.push_back(std::string(h));
             b.open_peers(hs);
           })
      .def("adopt_peers", &comm::SymmetricBuffer::adopt_peers)
      .def("base", [](comm::SymmetricBuffer& b, int r) { return uint64_t(reinterpret_cast<uintptr_t>(b.base(r))); })
      .def("tensor", &symm_tensor, py::arg("rank"), py::arg("byte_offset"), py::arg("numel"),
           py::arg("dtype"), py::arg("device"))
      .def_property_readonly("bytes", &comm::SymmetricBuffer::bytes)
      .def_property_readonly("rank", &comm::SymmetricBuffer::rank)
      .def_property_readonly("world", &comm::SymmetricBuffer::world)
      .def_property_readonly("connected", &comm::SymmetricBuffer::connected);

  // flag protocol for protocols orchestrated from Python (PowerSGD factors)
  m.def("bump_epoch",
        [](torch::Tensor epoch_dev) {
          TORCH_CHECK(epoch_dev.is_cuda() && epoch_dev.element_size() == 4 && epoch_dev.numel() >= 1,
                      "epoch_dev must be a 32-bit CUDA tensor");
          c10::cuda::CUDAGuard guard(epoch_dev.device());
          cudaError_t e = cuda::bump_epoch(static_cast<uint32_t*>(epoch_dev.data_ptr()), current_stream(epoch_dev.get_device()));
          TORCH_CHECK(e == cudaSuccess, cudaGetErrorString(e));
        },
        "epoch_dev[0] += 1 on the current stream: first kernel of a step whose epoch lives on the device");
  m.def("signal_flags",
        [](comm::SymmetricBuffer& buf, int64_t flag_offset, uint32_t epoch, int device,
           c10::optional<torch::Tensor> epoch_dev) {
          cuda::PushTargets t;
          t.world = buf.world();
          t.epoch = epoch;
          if (epoch_dev.has_value() && epoch_dev->defined())
            t.epoch_dev = static_cast<const uint32_t*>(epoch_dev->data_ptr());
          for (int p = 0; p < buf.world(); ++p)
            t.flag[p] = reinterpret_cast<uint32_t*>(buf.base(p) + flag_offset) + buf.rank();
          cudaError_t e = cuda::signal_flags(t, current_stream(device));
          TORCH_CHECK(e == cudaSuccess, cudaGetErrorString(e));
        },
        py::arg("buffer"), py::arg("flag_offset"), py::arg("epoch"), py::arg("device"),
        py::arg("epoch_dev") = py::none());
  m.def("wait_flags",
        [](comm::SymmetricBuffer& buf, int64_t flag_offset, uint32_t epoch, double timeout_s,
           const torch::Tensor& like, c10::optional<torch::Tensor> epoch_dev) {
          const uint32_t* ed = (epoch_dev.has_value() && epoch_dev->defined())
                                   ? static_cast<const uint32_t*>(epoch_dev->data_ptr()) : nullptr;
          cudaError_t e = cuda::wait_flags(reinterpret_cast<const uint32_t*>(buf.local() + flag_offset),
                                           buf.world(), epoch, uint64_t(timeout_s * 1e9),
                                           ops::status_word_for(like), current_stream(like.get_device()), ed);
          TORCH_CHECK(e == cudaSuccess, cudaGetErrorString(e));
        },
        py::arg("buffer"), py::arg("flag_offset"), py::arg("epoch"), py::arg("timeout_s"), py::arg("like"),
        py::arg("epoch_dev") = py::none());

  // ---------------------------------------------------------------- PowerSGD step driver
  py::class_<runtime::PsgdEngine>(m, "PsgdEngine")
      .def(py::init([](int world, int r, const torch::Tensor& like) {
             TORCH_CHECK(like.is_cuda(), "PsgdEngine needs a CUDA tensor to pick its device");
             return std::make_unique<runtime::PsgdEngine>(world, r, ops::status_word_for(like));
           }),
           py::arg("world"), py::arg("rank_r"), py::arg("like"))
      .def("add_matrix",
           [](runtime::PsgdEngine& e, torch::Tensor M, torch::Tensor param, torch::Tensor momentum,
              torch::Tensor P, torch::Tensor Q, c10::optional<torch::Tensor> Pt,
              c10::optional<torch::Tensor> Qt, const std::vector<std::vector<torch::Tensor>>& accP,
              const std::vector<std::vector<torch::Tensor>>& accQ) {
             auto f32 = [](const torch::Tensor& t, const char* what) {
               TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kFloat32 && t.is_contiguous(), what,
                           " must be a contiguous float32 CUDA tensor");
               return t.data_ptr<float>();
             };
             TORCH_CHECK(M.dim() == 2 && P.dim() == 2 && Q.dim() == 2, "M, P, Q must be matrices");
             runtime::PsgdMatrix d;
             d.M = f32(M, "M");
             d.n = M.size(0);
             d.m = M.size(1);
             d.param = f32(param, "param");
             d.momentum = f32(momentum, "momentum");
             d.numel = param.numel();
             TORCH_CHECK(momentum.numel() == d.numel && d.numel <= d.n * d.m, "param/momentum must fit in M");
             d.P = f32(P, "P");
             d.Q = f32(Q, "Q");
             TORCH_CHECK(P.size(0) == d.n && Q.size(0) == d.m && P.size(1) == Q.size(1), "P[n,r], Q[m,r] expected");
             if (Pt) {
               TORCH_CHECK(Pt->numel() >= 16 * cuda::psgd_kpad(d.n), "Pt too small");
               d.Pt = f32(*Pt, "Pt");
             }
             if (Qt) {
               TORCH_CHECK(Qt->numel() >= 16 * cuda::psgd_kpad(d.m), "Qt too small");
               d.Qt = f32(*Qt, "Qt");
             }
             TORCH_CHECK(accP.size() == 2 && accQ.size() == 2, "accumulators are given per epoch parity");
             for (int par = 0; par < 2; ++par) {
               TORCH_CHECK(accP[par].size() == accQ[par].size() && accP[par].size() <= size_t(cuda::kMaxWorld),
                           "one accumulator per rank expected");
               for (size_t p = 0; p < accP[par].size(); ++p) {
                 TORCH_CHECK(accP[par][p].numel() == P.numel() && accQ[par][p].numel() == Q.numel(),
                             "accumulators must have the factors' shapes");
                 d.accP[par][p] = f32(accP[par][p], "accP");
                 d.accQ[par][p] = f32(accQ[par][p], "accQ");
               }
             }
             return e.add_matrix(d);
           },
           py::arg("M"), py::arg("param"), py::arg("momentum"), py::arg("P"), py::arg("Q"), py::arg("Pt"),
           py::arg("Qt"), py::arg("accP"), py::arg("accQ"))
      .def("project_p",
           [](runtime::PsgdEngine& e, int parity, int device) {
             c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
             HP_CHECK_CUDA(e.project_p(parity, at::cuda::getCurrentCUDAStream()));
           })
      .def("project_q",
           [](runtime::PsgdEngine& e, int parity, int device) {
             c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
             HP_CHECK_CUDA(e.project_q(parity, at::cuda::getCurrentCUDAStream()));
           })
      .def("apply",
           [](runtime::PsgdEngine& e, int parity, double lr, double mu, double wd, bool first, int device) {
             c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
             HP_CHECK_CUDA(e.apply(parity, float(lr), float(mu), float(wd), first, at::cuda::getCurrentCUDAStream()));
           })
      .def_property_readonly("launches", &runtime::PsgdEngine::launches)
      .def_property_readonly("matrices", &runtime::PsgdEngine::matrices);

  // ---------------------------------------------------------------- DDP engine
  py::class_<runtime::BucketLayout>(m, "BucketLayout")
      .def_readonly("slot_bytes", &runtime::BucketLayout::slot_bytes)
      .def_property_readonly("slots", [](const runtime::BucketLayout& l) { return std::vector<int64_t>{l.slots[0], l.slots[1]}; })
      .def_readonly("flags", &runtime::BucketLayout::flags)
      .def_readonly("shift", &runtime::BucketLayout::shift);

  py::class_<runtime::DdpEngine>(m, "DdpEngine")
      .def(py::init([](const py::dict& cfg, const std::vector<std::tuple<int64_t, int64_t, int>>& buckets,
                       const std::vector<int>& param_bucket) {
             std::vector<runtime::BucketDesc> bs;
             for (auto& t : buckets) {
               runtime::BucketDesc b;
               b.offset = std::get<0>(t);
               b.numel = std::get<1>(t);
               b.num_params = std::get<2>(t);
               bs.push_back(b);
             }
             return std::make_unique<runtime::DdpEngine>(config_from(cfg), bs, param_bucket);
           }),
           py::arg("config"), py::arg("buckets"), py::arg("param_bucket"))
      .def_property_readonly("symmetric_bytes", &runtime::DdpEngine::symmetric_bytes)
      .def("layout", &runtime::DdpEngine::layout)
      .def("payload_capacity", &runtime::DdpEngine::payload_capacity)
      .def("set_buffers",
           [](runtime::DdpEngine& e, torch::Tensor grad, c10::optional<torch::Tensor> residual,
              c10::optional<torch::Tensor> param, c10::optional<torch::Tensor> momentum,
              c10::optional<torch::Tensor> aux, c10::optional<torch::Tensor> second) {
             auto ptr = [](c10::optional<torch::Tensor>& t) -> float* {
               return (t.has_value() && t->defined()) ? t->data_ptr<float>() : nullptr;
             };
             e.set_buffers(grad.data_ptr<float>(), ptr(residual), ptr(param), ptr(momentum), ptr(aux),
                           ptr(second));
           },
           py::arg("grad"), py::arg("residual") = py::none(), py::arg("param") = py::none(),
           py::arg("momentum") = py::none(), py::arg("aux") = py::none(), py::arg("second") = py::none())
      .def("set_symmetric",
           [](runtime::DdpEngine& e, comm::SymmetricBuffer& buf) {
             std::vector<uint8_t*> bases;
             for (int r = 0; r < buf.world(); ++r) bases.push_back(buf.base(r));
             e.set_symmetric(bases, buf.multicast());
           })
      .def("set_sgd", &runtime::DdpEngine::set_sgd, py::arg("lr"), py::arg("momentum"),
           py::arg("weight_decay"), py::arg("fused"))
      .def("set_adamw", &runtime::DdpEngine::set_adamw, py::arg("lr"), py::arg("beta1") = 0.9f,
           py::arg("beta2") = 0.999f, py::arg("eps") = 1e-8f, py::arg("weight_decay") = 0.0f)
      .def("set_keep_fraction", &runtime::DdpEngine::set_keep_fraction)
      .def("begin_step",
           [](runtime::DdpEngine& e, int device) {
             if (device < 0) {
               e.begin_step(nullptr);
               return;
             }
             c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
             e.begin_step(at::cuda::getCurrentCUDAStream());
           },
           py::arg("device") = -1)
      .def("reduce_step", &runtime::DdpEngine::reduce_step)
      .def("end_capture", &runtime::DdpEngine::end_capture)
      .def("note_replay", &runtime::DdpEngine::note_replay, py::arg("count"), py::arg("launches_per_step"))
      .def("grad_ready",
           [](runtime::DdpEngine& e, int param_index, int device) {
             e.grad_ready(param_index, current_stream(device));
           })
      .def("bucket_ready",
           [](runtime::DdpEngine& e, int bucket, int device) { e.bucket_ready(bucket, current_stream(device)); })
      .def("finish_step",
           [](runtime::DdpEngine& e, int device) {
             cudaStream_t s = current_stream(device);
             py::gil_scoped_release nogil;
             e.finish_step(s);
           })
      .def("drain", [](runtime::DdpEngine& e) { py::gil_scoped_release nogil; e.drain(); })
      .def("check_status", &runtime::DdpEngine::check_status)
      .def("set_progress", &runtime::DdpEngine::set_progress, py::arg("steps"), py::arg("epoch"))
      .def("residual2",
           [](runtime::DdpEngine& e, int device) -> c10::optional<torch::Tensor> {
             if (e.residual2() == nullptr) return c10::nullopt;
             // a view of the engine's buffer: valid while the engine lives
             return torch::from_blob(e.residual2(), {e.residual2_elems()},
                                     torch::TensorOptions().dtype(torch::kFloat32).device(torch::kCUDA, device));
           },
           py::arg("device"))
      .def("wait_stats", &runtime::DdpEngine::wait_stats)
      .def("stage_times", &runtime::DdpEngine::stage_times)
      .def("sparse_stats", &runtime::DdpEngine::sparse_stats)
      .def_property_readonly("epoch", &runtime::DdpEngine::epoch)
      .def_property_readonly("steps", &runtime::DdpEngine::steps)
      .def_property_readonly("launches", &runtime::DdpEngine::launches)
      .def_property_readonly("wire_bytes_per_step", &runtime::DdpEngine::wire_bytes_per_step)
      .def_property_readonly("dense_bytes_per_step", &runtime::DdpEngine::dense_bytes_per_step)
      .def("last_error", &runtime::DdpEngine::last_error);
}
