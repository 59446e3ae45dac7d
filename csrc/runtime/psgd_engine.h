// PowerSGD step driver: owns the per-matrix launch plan of a model and issues each phase of a
// step as a handful of launches -- one batched kernel per kind of small work (operand
// transposes, factor gathers, orthonormalisation), one grouped tcgen05 grid for the projections
// of all matrices and one grouped grid for their expand + SGD pass -- from a single native
// call, so that a model with tens of matrices pays neither a Python round trip nor a kernel's
// ramp-up and drain per matrix and stage.
//
// The reference exposes PowerSGD as three tasks per tensor (encode1 / encode2 / decode:
// ref hp_cuda.cpp:640-772, powersgd_body.h:10-78) that its five worker threads pick up one
// tensor at a time; the all-reduces between the stages are left to the caller.  Here the
// reductions are part of the GEMM epilogues (adds into the owner rank's accumulator over peer
// memory) and the phases below are separated only by the epoch flags the Python wrapper
// signals and waits on.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <vector>

#include "../kernels/kernels.h"

namespace hipress {
namespace runtime {

struct PsgdMatrix {
  float* M = nullptr;         // n x m gradient accumulator with error feedback
  float* param = nullptr;     // numel parameters
  float* momentum = nullptr;  // numel momentum
  float* P = nullptr;         // n x r
  float* Q = nullptr;         // m x r
  float* Pt = nullptr;        // 16 x kpad(n) scratch, may be null (SIMT GEMM then)
  float* Qt = nullptr;        // 16 x kpad(m) scratch, may be null
  int64_t n = 0, m = 0, numel = 0;
  // accumulators of every rank, per epoch parity: [parity][rank]
  float* accP[2][cuda::kMaxWorld] = {};
  float* accQ[2][cuda::kMaxWorld] = {};
};

class PsgdEngine {
 public:
  PsgdEngine(int world, int r, int* status_word);

  // Returns the matrix index.  Pt / Qt are dropped when the matrix is not TMA-eligible.
  int add_matrix(const PsgdMatrix& mat);
  int matrices() const { return int(mats_.size()); }

  // accP[parity][owner] += M Q for every matrix (Q transposed for the tensor-core operand first).
  cudaError_t project_p(int parity, cudaStream_t stream);
  // P = orthonormalise(mean of owners' accP); accQ[parity][owner] += M^T P.
  cudaError_t project_q(int parity, cudaStream_t stream);
  // Q = mean of owners' accQ; M -= P Q^T; fused SGD-momentum step with P Q^T as the gradient.
  cudaError_t apply(int parity, float lr, float mu, float weight_decay, bool first_step,
                    cudaStream_t stream);

  int64_t launches() const { return launches_; }

 private:
  int world_, r_;
  int* status_;
  int64_t launches_ = 0;
  std::vector<PsgdMatrix> mats_;
  std::vector<cuda::PsgdTransposeItem> tq_, tp_;   // Q -> Qt, P -> Pt
  std::vector<cuda::PsgdGsItem> gs_;
  std::vector<cuda::PsgdGatherItem> gp_[2], gq_[2];
};

}  // namespace runtime
}  // namespace hipress
