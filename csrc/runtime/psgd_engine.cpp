#include "psgd_engine.h"

#include <stdexcept>

namespace hipress {
namespace runtime {

namespace {
inline int batches(size_t items) { return int((items + cuda::kPsgdBatch - 1) / cuda::kPsgdBatch); }
}  // namespace

PsgdEngine::PsgdEngine(int world, int r, int* status_word) : world_(world), r_(r), status_(status_word) {
  if (world < 1 || world > cuda::kMaxWorld) throw std::invalid_argument("PsgdEngine: world must be 1..8");
  if (r < 1 || r > 16) throw std::invalid_argument("PsgdEngine: rank must be 1..16");
}

int PsgdEngine::add_matrix(const PsgdMatrix& in) {
  PsgdMatrix mat = in;
  if (!mat.M || !mat.P || !mat.Q || !mat.param || !mat.momentum || mat.n < 1 || mat.m < 1 ||
      mat.numel < 1 || mat.numel > mat.n * mat.m)
    throw std::invalid_argument("PsgdEngine: incomplete matrix description");
  for (int par = 0; par < 2; ++par)
    for (int p = 0; p < world_; ++p)
      if (!mat.accP[par][p] || !mat.accQ[par][p])
        throw std::invalid_argument("PsgdEngine: missing accumulator pointer");
  if (!cuda::psgd_tensor_core_eligible(mat.M, mat.n, mat.m)) mat.Pt = mat.Qt = nullptr;
  if (mat.Qt) tq_.push_back({mat.Q, mat.Qt, mat.m, cuda::psgd_kpad(mat.m), r_});
  if (mat.Pt) tp_.push_back({mat.P, mat.Pt, mat.n, cuda::psgd_kpad(mat.n), r_});
  gs_.push_back({mat.P, mat.n, r_});
  for (int par = 0; par < 2; ++par) {
    cuda::PsgdGatherItem a{}, b{};
    for (int p = 0; p < world_; ++p) {
      a.src[p] = mat.accP[par][p];
      b.src[p] = mat.accQ[par][p];
    }
    a.out = mat.P;
    a.rows = mat.n;
    a.r = r_;
    b.out = mat.Q;
    b.rows = mat.m;
    b.r = r_;
    gp_[par].push_back(a);
    gq_[par].push_back(b);
  }
  mats_.push_back(mat);
  return int(mats_.size()) - 1;
}

#define PSGD_TRY(expr)                      \
  do {                                      \
    const cudaError_t e__ = (expr);         \
    if (e__ != cudaSuccess) return e__;     \
  } while (0)

cudaError_t PsgdEngine::project_p(int parity, cudaStream_t stream) {
  parity &= 1;
  if (!tq_.empty()) {
    PSGD_TRY(cuda::psgd_transpose_pad_batched(tq_.data(), int(tq_.size()), stream));
    launches_ += batches(tq_.size());
  }
  // every matrix's P += M Q in one grid (a launch per matrix costs more in ramp-up and drain
  // than the small matrices take to stream)
  std::vector<cuda::PsgdGemmItem> items(mats_.size());
  for (size_t i = 0; i < mats_.size(); ++i) {
    const PsgdMatrix& mat = mats_[i];
    cuda::PsgdGemmItem& it = items[i];
    it.Mat = mat.M;
    it.n = mat.n;
    it.m = mat.m;
    it.X = mat.Q;
    it.Xt = mat.Qt;
    it.red.world = world_;
    for (int p = 0; p < world_; ++p) it.red.dst[p] = mat.accP[parity][p];
  }
  int launched = 0;
  PSGD_TRY(cuda::psgd_gemm_grouped(0, items.data(), int(items.size()), r_, status_, &launched, stream));
  launches_ += launched;
  return cudaSuccess;
}

cudaError_t PsgdEngine::project_q(int parity, cudaStream_t stream) {
  parity &= 1;
  if (mats_.empty()) return cudaSuccess;
  PSGD_TRY(cuda::psgd_owner_gather_batched(gp_[parity].data(), int(gp_[parity].size()), world_,
                                           1.0f / float(world_), stream));
  PSGD_TRY(cuda::gram_schmidt_batched(gs_.data(), int(gs_.size()), 1e-8f, stream));
  launches_ += 2 * batches(gs_.size());
  if (!tp_.empty()) {
    PSGD_TRY(cuda::psgd_transpose_pad_batched(tp_.data(), int(tp_.size()), stream));
    launches_ += batches(tp_.size());
  }
  std::vector<cuda::PsgdGemmItem> items(mats_.size());
  for (size_t i = 0; i < mats_.size(); ++i) {
    const PsgdMatrix& mat = mats_[i];
    cuda::PsgdGemmItem& it = items[i];
    it.Mat = mat.M;
    it.n = mat.n;
    it.m = mat.m;
    it.X = mat.P;
    it.Xt = mat.Pt;
    it.red.world = world_;
    for (int p = 0; p < world_; ++p) it.red.dst[p] = mat.accQ[parity][p];
  }
  int launched = 0;
  PSGD_TRY(cuda::psgd_gemm_grouped(1, items.data(), int(items.size()), r_, status_, &launched, stream));
  launches_ += launched;
  return cudaSuccess;
}

cudaError_t PsgdEngine::apply(int parity, float lr, float mu, float weight_decay, bool first_step,
                              cudaStream_t stream) {
  parity &= 1;
  if (mats_.empty()) return cudaSuccess;
  PSGD_TRY(cuda::psgd_owner_gather_batched(gq_[parity].data(), int(gq_[parity].size()), world_,
                                           1.0f / float(world_), stream));
  launches_ += batches(gq_[parity].size());
  cuda::SgdApply common;
  common.lr = lr;
  common.mu = mu;
  common.weight_decay = weight_decay;
  common.first_step = first_step ? 1 : 0;
  std::vector<cuda::PsgdExpandItem> items(mats_.size());
  for (size_t i = 0; i < mats_.size(); ++i) {
    const PsgdMatrix& mat = mats_[i];
    cuda::PsgdExpandItem& it = items[i];
    it.P = mat.P;
    it.Q = mat.Q;
    it.n = mat.n;
    it.m = mat.m;
    it.N = mat.numel;
    it.Mat = mat.M;
    it.param = mat.param;
    it.momentum = mat.momentum;
  }
  int launched = 0;
  PSGD_TRY(cuda::psgd_expand_sgd_grouped(items.data(), int(items.size()), r_, 1.0f, common, &launched, stream));
  launches_ += launched;
  return cudaSuccess;
}

}  // namespace runtime
}  // namespace hipress
