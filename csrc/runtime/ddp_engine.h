// Data-parallel gradient synchronisation engine.
//
// Gradients live in one flat fp32 buffer cut into buckets.  Backward hooks
// report parameters as ready; when the last parameter of a bucket is in, the
// hook thread records an event on the producing stream and hands the bucket to
// a worker thread, which issues on its own streams
//
//   push stream:  compress bucket -> packed bytes stored straight into every
//                 rank's receive slot (peer memory over NVLink) -> epoch flag
//   recv stream:  bounded wait on the W flags of the bucket -> one-pass
//                 unpack + accumulate of all W payloads (+ optional fused
//                 SGD-momentum update of the flat parameters)
//
// Compress kernels never wait on a peer and all waits sit on the recv stream,
// so ranks cannot deadlock on bucket order.  Receive slots are double-buffered
// by epoch parity; flags carry the epoch and are never reset.
//
// The reference has no such component: its caller submits per-tensor tasks,
// polls for completion and moves CPU buffers with an external transport
// (ref hp_cuda.cpp:904-1060).  This engine is the B200-native replacement for
// that whole loop; nothing here touches the host except launch calls.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <condition_variable>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "../kernels/kernels.h"
#include "worker_pool.h"

namespace hipress {
namespace runtime {

enum class Codec : int { kDense = 0, kTbq = 1, kTernGrad = 2, kSparse = 3, kEcq = 4 };

struct EngineConfig {
  int rank = 0, world = 1, device = 0;
  Codec codec = Codec::kTernGrad;
  // codec parameters
  float threshold = 0.f;                 // tbq
  int bitwidth = 2, enable_random = 1;   // terngrad / ecq
  int error_feedback = 1;                // terngrad: keep a residual
  double sample_rate = 0.01, keep_fraction = 0.001;  // sparse
  int sparse_accumulate = 1;             // 1: R += g inside the codec (GradDrop)
  float alpha = 1.f, beta = 1.f;         // ecq
  // DGC: momentum correction with factor masking and per-bucket local clipping
  int momentum_correction = 0;
  float dgc_momentum = 0.9f;
  float dgc_clip = 0.f;                  // <= 0: off; the caller divides by sqrt(world)
  uint64_t seed = 1;
  int average = 1;                       // divide the sum by world
  uint64_t flag_timeout_ns = 20ull * 1000 * 1000 * 1000;
  int num_workers = 1;
  // Issue the receive half (flag wait + unpack) of every bucket only in
  // finish_step().  Used when several ranks are emulated on one device: the
  // caller lets all ranks push, synchronises, and only then finishes the steps,
  // so that no kernel ever waits for a kernel that has not been launched yet.
  int defer_recv = 0;
  // The fused optimizer kernel leaves zeros in the gradient bucket instead of the averaged
  // gradient (nobody reads it after a fused update), so no separate clearing pass is needed.
  int clear_grad = 0;
  // Keep the step's epoch in device memory (TBQ and TernGrad): kernels read the epoch, pick the
  // slot parity and derive the rounding seed on the device, so that a whole training step --
  // backward hooks and this engine's launches included -- can be captured once in a CUDA graph
  // and replayed.  begin_step() then launches a one-thread kernel that advances the counter.
  int device_epoch = 0;
  // Sharded exchange (TBQ, TernGrad): rank j owns shard j (1/world) of every bucket.  Phase 1:
  // every rank compresses each shard and stores it into the owner's slot (compressed
  // reduce-scatter).  Phase 2: the owner decodes the world payloads of its shard, averages,
  // re-compresses the average with its own residual and stores it to every rank (compressed
  // all-gather).  Phase 3: every rank decodes the world shard payloads (one per owner) and applies
  // the update.  A rank sends 2 x (world-1)/world of one payload instead of world-1 payloads and
  // decodes 2 table look-ups per element instead of world; the price is a second quantisation
  // (the reference's root does the same: decompress-accumulate, then re-compress,
  // ref hp_cuda.cpp:241-271).
  int sharded = 0;
  // Per-stage device timing: one-thread kernels write the device wall clock into a small table
  // at the stage boundaries of every bucket (gradients ready, payload pushed, peers' payloads
  // arrived, update applied) and at the beginning and end of the step; stage_times() reads the
  // last step's table.  Adds four tiny launches per bucket, so it is off unless asked for.  (The
  // time spent inside flag waits is counted always: wait_stats().)
  int trace = 0;
  // Deliver payloads with NVLS multicast stores (multimem.st) where the symmetric buffer has a
  // multicast mapping: one store per packed word reaches every rank's slot through the NVLink
  // switch, instead of one store per destination.  All-gather form of tbq / terngrad / ecq and
  // the sparse codecs; flags, headers and ragged ends stay unicast.  Ignored (plain peer stores)
  // when the buffer has no multicast mapping.
  int nvls = 0;
};

struct BucketDesc {
  int64_t offset = 0;   // first element in the flat buffers
  int64_t numel = 0;
  int num_params = 0;   // hooks that must fire before the bucket is ready
};

// Byte layout of one bucket inside the symmetric buffer.
struct BucketLayout {
  int64_t slot_bytes = 0;      // capacity of one rank's slot (multiple of 256)
  int64_t slots[2] = {0, 0};   // offset of slot array [world][slot_bytes] per parity
  int64_t flags = 0;           // offset of `world` uint32 flags
  int64_t shift = 0;           // payload starts at slot + shift (aligns the data region)
  // sharded exchange only
  int64_t shard_elems = 0;     // elements per shard (multiple of 64)
  int64_t slots2[2] = {0, 0};  // phase-2 slot array [world owners][slot_bytes] per parity
  int64_t flags2 = 0;          // phase-2 flags
};

class DdpEngine {
 public:
  DdpEngine(const EngineConfig& cfg, const std::vector<BucketDesc>& buckets,
            const std::vector<int>& param_bucket);
  ~DdpEngine();

  // Bytes of symmetric memory the buckets need; computed at construction.
  int64_t symmetric_bytes() const { return symmetric_bytes_; }
  const BucketLayout& layout(int b) const { return layouts_.at(static_cast<size_t>(b)); }
  int64_t payload_capacity(int b) const;

  // residual / param / momentum / aux may be null when unused.  `momentum` is
  // the SGD momentum buffer or AdamW's first moment; `aux` is DGC's velocity u;
  // `second` is AdamW's second moment.
  void set_buffers(float* grad, float* residual, float* param, float* momentum,
                   float* aux = nullptr, float* second = nullptr);
  // bases[r]: rank r's symmetric buffer as mapped in this process.
  // multicast: NVLS mapping of the same buffer (stores reach every rank), or null.
  void set_symmetric(const std::vector<uint8_t*>& bases, uint8_t* multicast = nullptr);
  bool nvls_active() const { return cfg_.nvls && mc_base_ != nullptr && cfg_.world > 1; }

  void set_sgd(float lr, float momentum, float weight_decay, bool fused);
  void set_adamw(float lr, float beta1, float beta2, float eps, float weight_decay);
  void set_keep_fraction(double keep_fraction);

  // `consumer`: the stream the step runs on (only used with device_epoch: the kernel that
  // advances the epoch is ordered before the step's backward pass on it).
  void begin_step(cudaStream_t consumer = nullptr);
  // A step issued while a CUDA graph was being captured did not run: take it back out of the
  // host-side counters.  Returns the number of kernel launches the captured step holds.
  int64_t end_capture();
  // A captured step was replayed `count` times: advance the host-side counters to match.
  void note_replay(int64_t count, int64_t launches_per_step);
  // Called from a backward hook; `producer` is the stream the gradient was
  // written on.
  void grad_ready(int param_index, cudaStream_t producer);
  void bucket_ready(int bucket_index, cudaStream_t producer);
  // Blocks until every bucket of this step has been issued, then makes
  // `consumer` wait for the device work.  Buckets whose hooks never fired
  // (unused parameters) are flushed here.
  void finish_step(cudaStream_t consumer);
  // defer_recv + sharded: issues phase 2 (owner reduce + re-compress) of every bucket.  The
  // caller emulating several ranks on one device calls it for every rank between a device
  // synchronise after the pushes and another before finish_step().
  void reduce_step();
  // Blocks until every job handed to the workers so far has been issued to the device.
  void drain() { if (pool_) pool_->drain(); }

  // Synchronises and returns the device status word (cuda::Status); resets it.
  int check_status();
  // Continue from a checkpoint: `steps` optimizer steps have been taken and the exchange is at
  // `epoch` (flag value, slot parity, rounding seed and AdamW's bias-correction step all derive
  // from these).  Every rank must restore the same values before its next step.
  void set_progress(int64_t steps, uint32_t epoch);
  // Residual of the owner's re-compression in the sharded exchange (device pointer, elements).
  float* residual2() const { return residual2_; }
  int64_t residual2_elems() const { return residual2_elems_; }
  // {total ns inside flag waits, longest single wait in ns, number of waits} since the last
  // call (synchronises the device; the counters are reset).
  std::vector<unsigned long long> wait_stats();
  // With EngineConfig::trace: device wall-clock stamps (ns) of the last step, relative to the
  // step's begin: per bucket {ready, pushed, arrived, done}, then {step end}.  Zero where a stage
  // did not run.  Synchronises the device.
  std::vector<int64_t> stage_times();
  // With EngineConfig::trace and a sparse codec: per bucket {elements sent, candidates over the
  // sampled threshold, threshold (bit pattern of a float), candidates dropped so far} of the
  // last step.  Synchronises the device.
  std::vector<unsigned int> sparse_stats();
  uint32_t epoch() const { return epoch_; }
  int64_t steps() const { return steps_; }
  // kernels launched by the engine since construction
  int64_t launches() const { return launches_.load(); }
  // wire bytes (compressed) and dense bytes of one step, for metrics
  int64_t wire_bytes_per_step() const;
  int64_t dense_bytes_per_step() const;
  std::string last_error() { return pool_ ? pool_->last_error() : std::string(); }

 private:
  struct WorkerCtx {
    cudaStream_t push = nullptr, recv = nullptr;
    void* scratch = nullptr;       // zeroed; minmax + sparse scratch
    unsigned int* done = nullptr;  // last-CTA counter for publish
    cudaEvent_t tail = nullptr;    // last recorded event on recv
    cudaEvent_t pushed = nullptr;  // this rank's payload and flag of the latest bucket are out
    bool used = false;
  };
  enum Stamp : int { kStampReady = 0, kStampPushed = 1, kStampArrived = 2, kStampDone = 3, kStampCount = 4 };
  void stamp(int b, int which, cudaStream_t stream);
  cuda::SgdApply sgd_apply_for(int b) const;
  void issue_adamw(int b, cudaStream_t stream, int clear_grad = -1);  // -1: as configured
  void issue_bucket(int b, int worker);
  void issue_push(int b, int worker);
  void issue_recv(int b, int worker);
  // sharded exchange: the three phases of one bucket
  void issue_shard_push(int b, int worker);
  void issue_shard_reduce(int b, int worker);
  void issue_shard_final(int b, int worker);
  int64_t shard_len(int b, int j) const;
  cuda::PushTargets targets_for(int b, WorkerCtx& w) const;
  cuda::UnpackSources sources_for(int b) const;

  EngineConfig cfg_;
  std::vector<BucketDesc> buckets_;
  std::vector<BucketLayout> layouts_;
  std::vector<int> param_bucket_;
  int64_t symmetric_bytes_ = 0;

  float *grad_ = nullptr, *residual_ = nullptr, *param_ = nullptr, *momentum_ = nullptr;
  float *aux_ = nullptr, *second_ = nullptr;
  bool adamw_ = false;
  float beta1_ = 0.9f, beta2_ = 0.999f, eps_ = 1e-8f;
  std::vector<uint8_t*> bases_;
  uint8_t* mc_base_ = nullptr;
  float lr_ = 0.f, sgd_mu_ = 0.f, wd_ = 0.f;
  bool fused_sgd_ = false;
  double keep_fraction_;

  uint32_t epoch_ = 0;
  int64_t steps_ = 0;
  uint32_t* epoch_dev_ = nullptr;   // device copy of epoch_ (device_epoch mode)
  float* residual2_ = nullptr;      // sharded: residual of the owner's re-compression, per bucket shard
  int64_t residual2_elems_ = 0;
  unsigned long long* wait_ns_ = nullptr;  // device: {total, max, count} of the flag waits
  unsigned long long* stamps_ = nullptr;   // device: [buckets][kStampCount] + {begin, end}; trace only
  unsigned int* sparse_stats_host_ = nullptr;  // pinned: [buckets][4]; trace + sparse codec only
  std::vector<int64_t> residual2_off_;
  int64_t launches_at_begin_ = 0;
  std::vector<std::atomic<int>> pending_params_;
  std::vector<std::atomic<int>> submitted_;
  std::vector<cudaEvent_t> ready_events_;
  std::vector<WorkerCtx> workers_;
  int* status_ = nullptr;

  std::mutex mu_;
  std::condition_variable cv_;
  int issued_ = 0;
  std::atomic<int64_t> launches_{0};

  std::unique_ptr<WorkerPool> pool_;
};

}  // namespace runtime
}  // namespace hipress
