// Weight gradient of a linear layer with the bias gradient taken in the same GEMM.
//
//   dW[out, in] (fp32) = dY^T X,   db[out] (fp32) = column sums of dY       dY: [T, out] bf16, X: [T, in] bf16
//
// This is a plain library GEMM (cuBLASLt) -- the framework's own tensor-core kernels are the
// PowerSGD projections -- asked for its BGRADB epilogue: the reduction of dY over the tokens
// runs inside the GEMM that reads dY anyway, so the bias gradient costs no pass of its own (a
// BERT-large step has 97 such layers; as separate column-sum kernels they were two launches
// and one more read of dY each).  Row-major dW[out, in] is the column-major matrix D[in, out] =
// A[in, T] * B[out, T]^T with A = X and B = dY as cuBLAS sees row-major buffers; the epilogue
// reduces B over T, one value per column of D.
//
// The reference has no model code; this belongs to the model zoo built around its codecs.
//
// Not every (shape, type) combination has an algorithm with this epilogue; `linear_wgrad_bgrad`
// reports that by returning an empty list and the caller keeps its two-kernel path.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cublasLt.h>
#include <torch/extension.h>

#include <map>
#include <mutex>
#include <tuple>

#include "ops.h"

namespace hipress {
namespace ops {

namespace {

struct Plan {
  bool usable = false;
  cublasLtMatmulDesc_t op = nullptr;
  cublasLtMatrixLayout_t a = nullptr, b = nullptr, d = nullptr;
  cublasLtMatmulAlgo_t algo{};
  size_t workspace = 0;
};

constexpr size_t kWorkspaceBytes = 32u << 20;

// key: device, tokens, in features, out features
using Key = std::tuple<int, int64_t, int64_t, int64_t>;
std::mutex g_mu;
std::map<Key, Plan> g_plans;
std::map<int, torch::Tensor> g_workspace;   // one per device, allocated on first use (outside any capture)

bool ok(cublasStatus_t s) { return s == CUBLAS_STATUS_SUCCESS; }

Plan make_plan(cublasLtHandle_t handle, int64_t tokens, int64_t in_f, int64_t out_f) {
  Plan p;
  const cublasOperation_t ta = CUBLAS_OP_N, tb = CUBLAS_OP_T;
  const cublasLtEpilogue_t epi = CUBLASLT_EPILOGUE_BGRADB;
  const cudaDataType_t bias_type = CUDA_R_32F;
  if (!ok(cublasLtMatmulDescCreate(&p.op, CUBLAS_COMPUTE_32F, CUDA_R_32F))) return p;
  bool good = ok(cublasLtMatmulDescSetAttribute(p.op, CUBLASLT_MATMUL_DESC_TRANSA, &ta, sizeof(ta))) &&
              ok(cublasLtMatmulDescSetAttribute(p.op, CUBLASLT_MATMUL_DESC_TRANSB, &tb, sizeof(tb))) &&
              ok(cublasLtMatmulDescSetAttribute(p.op, CUBLASLT_MATMUL_DESC_EPILOGUE, &epi, sizeof(epi))) &&
              ok(cublasLtMatmulDescSetAttribute(p.op, CUBLASLT_MATMUL_DESC_BIAS_DATA_TYPE, &bias_type,
                                                sizeof(bias_type)));
  // column-major views of the row-major buffers: X[T, in] is A[in, T] (ld in); dY[T, out] is B[out, T] (ld out);
  // dW[out, in] is D[in, out] (ld in)
  good = good && ok(cublasLtMatrixLayoutCreate(&p.a, CUDA_R_16BF, in_f, tokens, in_f)) &&
         ok(cublasLtMatrixLayoutCreate(&p.b, CUDA_R_16BF, out_f, tokens, out_f)) &&
         ok(cublasLtMatrixLayoutCreate(&p.d, CUDA_R_32F, in_f, out_f, in_f));
  if (!good) return p;
  cublasLtMatmulPreference_t pref = nullptr;
  if (!ok(cublasLtMatmulPreferenceCreate(&pref))) return p;
  size_t ws = kWorkspaceBytes;
  cublasLtMatmulPreferenceSetAttribute(pref, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &ws, sizeof(ws));
  cublasLtMatmulHeuristicResult_t res{};
  int found = 0;
  // the pointer of the bias gradient must be known to the heuristic only as "present": set a dummy non-null value
  const void* dummy = reinterpret_cast<const void*>(uintptr_t(256));
  cublasLtMatmulDescSetAttribute(p.op, CUBLASLT_MATMUL_DESC_BIAS_POINTER, &dummy, sizeof(dummy));
  const cublasStatus_t st = cublasLtMatmulAlgoGetHeuristic(handle, p.op, p.a, p.b, p.d, p.d, pref, 1, &res, &found);
  cublasLtMatmulPreferenceDestroy(pref);
  if (!ok(st) || found < 1 || !ok(res.state)) return p;
  p.algo = res.algo;
  p.workspace = res.workspaceSize;
  p.usable = true;
  return p;
}

}  // namespace

std::vector<torch::Tensor> linear_wgrad_bgrad(const torch::Tensor& dy, const torch::Tensor& x) {
  TORCH_CHECK(dy.is_cuda() && x.is_cuda() && dy.scalar_type() == torch::kBFloat16 &&
                  x.scalar_type() == torch::kBFloat16,
              "linear_wgrad_bgrad: bf16 CUDA tensors expected");
  TORCH_CHECK(dy.dim() == 2 && x.dim() == 2 && dy.size(0) == x.size(0) && dy.is_contiguous() && x.is_contiguous(),
              "linear_wgrad_bgrad: contiguous [tokens, out] and [tokens, in] expected");
  const int64_t tokens = dy.size(0), out_f = dy.size(1), in_f = x.size(1);
  if (tokens < 1 || (in_f % 8) != 0 || (out_f % 8) != 0) return {};
  if ((reinterpret_cast<uintptr_t>(dy.data_ptr()) & 15) != 0 || (reinterpret_cast<uintptr_t>(x.data_ptr()) & 15) != 0)
    return {};
  c10::cuda::CUDAGuard guard(dy.device());
  const int dev = dy.get_device();
  cublasLtHandle_t handle = at::cuda::getCurrentCUDABlasLtHandle();
  auto stream = at::cuda::getCurrentCUDAStream();

  Plan plan;
  void* workspace = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    const Key key{dev, tokens, in_f, out_f};
    auto it = g_plans.find(key);
    if (it == g_plans.end()) it = g_plans.emplace(key, make_plan(handle, tokens, in_f, out_f)).first;
    plan = it->second;
    if (!plan.usable) return {};
    auto ws = g_workspace.find(dev);
    if (ws == g_workspace.end()) {
      cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
      cudaStreamIsCapturing(stream, &cap);
      if (cap != cudaStreamCaptureStatusNone) return {};   // first use inside a capture: let the caller fall back
      ws = g_workspace.emplace(dev, torch::empty({int64_t(kWorkspaceBytes)}, dy.options().dtype(torch::kUInt8))).first;
    }
    workspace = ws->second.data_ptr();
  }

  auto f32 = dy.options().dtype(torch::kFloat32);
  auto dw = torch::empty({out_f, in_f}, f32);
  auto db = torch::empty({out_f}, f32);
  // the descriptor is shared between calls of one shape: the bias pointer is set under the lock that
  // also covers the launch, so two threads never interleave pointer and launch
  std::lock_guard<std::mutex> lock(g_mu);
  const void* db_ptr = db.data_ptr();
  TORCH_CHECK(ok(cublasLtMatmulDescSetAttribute(plan.op, CUBLASLT_MATMUL_DESC_BIAS_POINTER, &db_ptr, sizeof(db_ptr))),
              "linear_wgrad_bgrad: setting the bias-gradient pointer failed");
  const float one = 1.0f, zero = 0.0f;
  const cublasStatus_t st =
      cublasLtMatmul(handle, plan.op, &one, x.data_ptr(), plan.a, dy.data_ptr(), plan.b, &zero, dw.data_ptr(), plan.d,
                     dw.data_ptr(), plan.d, &plan.algo, workspace, kWorkspaceBytes, stream);
  TORCH_CHECK(ok(st), "linear_wgrad_bgrad: cublasLtMatmul failed with status ", int(st));
  return {dw, db};
}

}  // namespace ops
}  // namespace hipress
