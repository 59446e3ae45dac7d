#include "ddp_engine.h"

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <stdexcept>

#include <nvtx3/nvToolsExt.h>

#include "../common/codec_math.h"

namespace hipress {
namespace runtime {

namespace {

void check(cudaError_t e, const char* what) {
  if (e != cudaSuccess)
    throw std::runtime_error(std::string("hipress engine: ") + what + ": " + cudaGetErrorString(e));
}
int64_t round_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

constexpr size_t kScratchBytes = 256 * 1024;

// Named range on the calling thread's timeline for an attached tool; a no-op test when tracing is off.
struct TraceRange {
  bool on;
  TraceRange(bool enabled, const char* what, int bucket) : on(enabled) {
    if (!on) return;
    char name[48];
    snprintf(name, sizeof(name), "hipress %s b%d", what, bucket);
    nvtxRangePushA(name);
  }
  ~TraceRange() {
    if (on) nvtxRangePop();
  }
  TraceRange(const TraceRange&) = delete;
  TraceRange& operator=(const TraceRange&) = delete;
};

}  // namespace

int64_t DdpEngine::payload_capacity(int b) const {
  const int64_t n = buckets_.at(static_cast<size_t>(b)).numel;
  switch (cfg_.codec) {
    case Codec::kDense: return n * 4;
    case Codec::kTbq: return tbq_payload_bytes(n);
    case Codec::kTernGrad: return tern_payload_bytes(n, cfg_.bitwidth);
    case Codec::kSparse:
      return sparse_payload_bytes(std::min<int64_t>(n, sparse_expected_k(n, cfg_.keep_fraction)));
    case Codec::kEcq: return ecq_payload_bytes(n, cfg_.bitwidth);
  }
  return 0;
}

DdpEngine::DdpEngine(const EngineConfig& cfg, const std::vector<BucketDesc>& buckets,
                     const std::vector<int>& param_bucket)
    : cfg_(cfg), buckets_(buckets), param_bucket_(param_bucket), keep_fraction_(cfg.keep_fraction),
      pending_params_(buckets.size()), submitted_(buckets.size()) {
  if (cfg.world < 1 || cfg.world > cuda::kMaxWorld) throw std::invalid_argument("world must be 1..8");
  if (cfg.rank < 0 || cfg.rank >= cfg.world) throw std::invalid_argument("bad rank");
  if (cfg.codec == Codec::kTernGrad && !tern_bitwidth_ok(cfg.bitwidth))
    throw std::invalid_argument("terngrad bitwidth must be 1, 2, 4 or 8");
  if (cfg.codec == Codec::kEcq && !ecq_bitwidth_ok(cfg.bitwidth))
    throw std::invalid_argument("ecq bitwidth must be 2, 4 or 8");
  for (int pb : param_bucket)
    if (pb < 0 || pb >= static_cast<int>(buckets.size())) throw std::invalid_argument("bad param->bucket map");

  if (cfg.sharded) {
    if (cfg.codec != Codec::kTbq && cfg.codec != Codec::kTernGrad)
      throw std::invalid_argument("the sharded exchange is implemented for the tbq and terngrad codecs");
  }
  // symmetric layout: [flags of all buckets][slots parity 0][slots parity 1] per bucket
  int64_t off = 0;
  layouts_.resize(buckets.size());
  for (size_t b = 0; b < buckets.size(); ++b) {
    layouts_[b].flags = off;
    off += round_up(int64_t(cfg.world) * 4, 128);
    if (cfg.sharded) {
      layouts_[b].flags2 = off;
      off += round_up(int64_t(cfg.world) * 4, 128);
    }
  }
  off = round_up(off, 1024);
  int64_t res2 = 0;
  residual2_off_.assign(buckets.size(), 0);
  for (size_t b = 0; b < buckets.size(); ++b) {
    BucketLayout& L = layouts_[b];
    // header-bearing payloads start 6 bytes into the slot so that the data
    // region after the 10-byte header is 16-byte aligned for vector stores
    L.shift = (cfg.codec == Codec::kTernGrad || cfg.codec == Codec::kEcq) ? 6 : 0;
    if (cfg.sharded) {
      // shards of a multiple of 4,096 elements: every shard starts 16-byte aligned in the dense
      // buffers and no 512-byte payload chunk of any bitwidth straddles two shards
      L.shard_elems = round_up((buckets[b].numel + cfg.world - 1) / cfg.world, 4096);
      const int64_t cap = cfg.codec == Codec::kTbq ? tbq_payload_bytes(L.shard_elems)
                                                   : tern_payload_bytes(L.shard_elems, cfg.bitwidth);
      L.slot_bytes = round_up(cap + L.shift, 256);
      residual2_off_[b] = res2;
      res2 += L.shard_elems;
    } else {
      L.slot_bytes = round_up(payload_capacity(int(b)) + L.shift, 256);
    }
    for (int p = 0; p < 2; ++p) {
      L.slots[p] = off;
      off += L.slot_bytes * cfg.world;
    }
    if (cfg.sharded) {
      for (int p = 0; p < 2; ++p) {
        L.slots2[p] = off;
        off += L.slot_bytes * cfg.world;
      }
    }
  }
  symmetric_bytes_ = round_up(off, 1024);

  check(cudaSetDevice(cfg.device), "cudaSetDevice");
  ready_events_.resize(buckets.size());
  for (auto& e : ready_events_) check(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "event");
  check(cudaMalloc(reinterpret_cast<void**>(&status_), 64), "cudaMalloc status");
  check(cudaMemset(status_, 0, 64), "memset status");
  if (cfg.sharded && res2 > 0) {
    check(cudaMalloc(reinterpret_cast<void**>(&residual2_), size_t(res2) * sizeof(float)), "cudaMalloc residual2");
    check(cudaMemset(residual2_, 0, size_t(res2) * sizeof(float)), "memset residual2");
    residual2_elems_ = res2;
  }
  check(cudaMalloc(reinterpret_cast<void**>(&wait_ns_), 64), "cudaMalloc wait stats");
  check(cudaMemset(wait_ns_, 0, 64), "memset wait stats");
  if (cfg.trace) {
    const size_t bytes = (buckets.size() * kStampCount + 2) * sizeof(unsigned long long);
    check(cudaMalloc(reinterpret_cast<void**>(&stamps_), bytes), "cudaMalloc stamps");
    check(cudaMemset(stamps_, 0, bytes), "memset stamps");
  }
  if (cfg.device_epoch) {
    if (cfg.num_workers >= 1)
      throw std::invalid_argument("device_epoch needs inline issue (num_workers = 0): a captured step is issued by the capturing thread");
    check(cudaMalloc(reinterpret_cast<void**>(&epoch_dev_), 64), "cudaMalloc epoch");
    check(cudaMemset(epoch_dev_, 0, 64), "memset epoch");
  }

  const int nw = cfg.num_workers < 1 ? 1 : cfg.num_workers;
  workers_.resize(static_cast<size_t>(nw));
  // per worker: min/max reduction state (first 16 KB, second region at 128 KB for the sharded
  // exchange's owner phase); the sparse codecs' state, sample keys and candidate pool behind it
  size_t scratch_bytes = kScratchBytes;
  if (cfg.codec == Codec::kSparse) {
    size_t need = 0;
    for (auto& b : buckets) need = std::max(need, cuda::sparse_scratch_bytes(b.numel));
    scratch_bytes = std::max(scratch_bytes, size_t(16384) + need);
    if (cfg.trace) {
      check(cudaHostAlloc(reinterpret_cast<void**>(&sparse_stats_host_), buckets.size() * 4 * sizeof(unsigned int),
                          cudaHostAllocDefault),
            "cudaHostAlloc stats");
      std::memset(sparse_stats_host_, 0, buckets.size() * 4 * sizeof(unsigned int));
    }
  }
  int lo = 0, hi = 0;
  check(cudaDeviceGetStreamPriorityRange(&lo, &hi), "priority range");
  for (auto& w : workers_) {
    check(cudaStreamCreateWithPriority(&w.push, cudaStreamNonBlocking, hi), "stream");
    check(cudaStreamCreateWithPriority(&w.recv, cudaStreamNonBlocking, hi), "stream");
    check(cudaMalloc(&w.scratch, scratch_bytes), "cudaMalloc scratch");
    check(cudaMemset(w.scratch, 0, scratch_bytes), "memset scratch");
    check(cudaMalloc(reinterpret_cast<void**>(&w.done), 64), "cudaMalloc counter");
    check(cudaMemset(w.done, 0, 64), "memset counter");
    check(cudaEventCreateWithFlags(&w.tail, cudaEventDisableTiming), "event");
    check(cudaEventCreateWithFlags(&w.pushed, cudaEventDisableTiming), "event");
  }
  check(cudaDeviceSynchronize(), "sync");
  const int device = cfg.device;
  // num_workers == 0: no threads; the thread that reports a bucket ready issues its kernels
  if (cfg.num_workers >= 1)
    pool_ = std::make_unique<WorkerPool>(nw, [device](int) { cudaSetDevice(device); });
}

DdpEngine::~DdpEngine() {
  if (pool_) {
    try {
      pool_->drain();
    } catch (...) {
    }
    pool_->shutdown();
  }
  cudaSetDevice(cfg_.device);
  cudaDeviceSynchronize();
  for (auto& w : workers_) {
    if (w.push) cudaStreamDestroy(w.push);
    if (w.recv) cudaStreamDestroy(w.recv);
    if (w.scratch) cudaFree(w.scratch);
    if (w.done) cudaFree(w.done);
    if (w.tail) cudaEventDestroy(w.tail);
    if (w.pushed) cudaEventDestroy(w.pushed);
  }
  for (auto& e : ready_events_) cudaEventDestroy(e);
  if (status_) cudaFree(status_);
  if (epoch_dev_) cudaFree(epoch_dev_);
  if (residual2_) cudaFree(residual2_);
  if (wait_ns_) cudaFree(wait_ns_);
  if (sparse_stats_host_) cudaFreeHost(sparse_stats_host_);
  if (stamps_) cudaFree(stamps_);
}

void DdpEngine::set_buffers(float* grad, float* residual, float* param, float* momentum, float* aux,
                            float* second) {
  grad_ = grad;
  residual_ = residual;
  param_ = param;
  momentum_ = momentum;
  aux_ = aux;
  second_ = second;
}

void DdpEngine::set_adamw(float lr, float beta1, float beta2, float eps, float weight_decay) {
  lr_ = lr;
  beta1_ = beta1;
  beta2_ = beta2;
  eps_ = eps;
  wd_ = weight_decay;
  adamw_ = true;
  fused_sgd_ = false;
}

void DdpEngine::set_symmetric(const std::vector<uint8_t*>& bases, uint8_t* multicast) {
  if (static_cast<int>(bases.size()) != cfg_.world) throw std::invalid_argument("one base pointer per rank");
  bases_ = bases;
  mc_base_ = multicast;
}

void DdpEngine::set_sgd(float lr, float momentum, float weight_decay, bool fused) {
  lr_ = lr;
  sgd_mu_ = momentum;
  wd_ = weight_decay;
  fused_sgd_ = fused;
}

void DdpEngine::set_keep_fraction(double keep_fraction) {
  if (keep_fraction <= 0.0 || keep_fraction > cfg_.keep_fraction)
    throw std::invalid_argument("keep_fraction must be in (0, configured maximum]");
  keep_fraction_ = keep_fraction;
}

void DdpEngine::begin_step(cudaStream_t consumer) {
  if (grad_ == nullptr || bases_.empty()) throw std::runtime_error("hipress engine: buffers not set");
  ++epoch_;
  launches_at_begin_ = launches_.load();
  if (epoch_dev_) {
    // ordered after the previous step (finish_step made `consumer` wait for its last kernels)
    // and before this step's gradients, whose ready events are recorded on `consumer`
    check(cuda::bump_epoch(epoch_dev_, consumer), "bump_epoch");
    launches_ += 1;
  }
  if (stamps_) {
    check(cuda::stamp_time(stamps_ + buckets_.size() * kStampCount, consumer), "stamp");
    launches_ += 1;
  }
  for (size_t b = 0; b < buckets_.size(); ++b) {
    pending_params_[b].store(buckets_[b].num_params);
    submitted_[b].store(0);
  }
  std::lock_guard<std::mutex> lk(mu_);
  issued_ = 0;
  for (auto& w : workers_) w.used = false;
}

void DdpEngine::grad_ready(int param_index, cudaStream_t producer) {
  const int b = param_bucket_.at(static_cast<size_t>(param_index));
  if (pending_params_[static_cast<size_t>(b)].fetch_sub(1) == 1) bucket_ready(b, producer);
}

void DdpEngine::bucket_ready(int b, cudaStream_t producer) {
  if (submitted_.at(static_cast<size_t>(b)).exchange(1) != 0) return;
  check(cudaEventRecord(ready_events_[static_cast<size_t>(b)], producer), "cudaEventRecord");
  const int worker = b % static_cast<int>(workers_.size());
  if (!pool_) {
    issue_bucket(b, worker);
    std::lock_guard<std::mutex> lk(mu_);
    ++issued_;
    return;
  }
  pool_->submit_to(worker, [this, b](int w) {
    try {
      issue_bucket(b, w);
    } catch (...) {
      {
        std::lock_guard<std::mutex> lk(mu_);
        ++issued_;
      }
      cv_.notify_all();
      throw;
    }
    {
      std::lock_guard<std::mutex> lk(mu_);
      ++issued_;
    }
    cv_.notify_all();
  });
}

int64_t DdpEngine::end_capture() {
  const int64_t per_step = launches_.load() - launches_at_begin_;
  --epoch_;
  --steps_;
  launches_ -= per_step;
  return per_step;
}

void DdpEngine::note_replay(int64_t count, int64_t launches_per_step) {
  epoch_ += static_cast<uint32_t>(count);
  steps_ += count;
  launches_ += count * launches_per_step;
}

cuda::PushTargets DdpEngine::targets_for(int b, WorkerCtx& w) const {
  const BucketLayout& L = layouts_[static_cast<size_t>(b)];
  const int parity = epoch_dev_ ? 0 : int(epoch_ & 1u);
  cuda::PushTargets t;
  t.world = cfg_.world;
  t.epoch = epoch_;
  t.done = w.done;
  t.epoch_dev = epoch_dev_;
  t.parity_stride = L.slots[1] - L.slots[0];
  t.guard = status_;
  for (int p = 0; p < cfg_.world; ++p) {
    uint8_t* base = bases_[static_cast<size_t>(p)];
    t.payload[p] = base + L.slots[parity] + int64_t(cfg_.rank) * L.slot_bytes + L.shift;
    t.flag[p] = reinterpret_cast<uint32_t*>(base + L.flags) + cfg_.rank;
  }
  if (nvls_active()) t.mc = mc_base_ + L.slots[parity] + int64_t(cfg_.rank) * L.slot_bytes + L.shift;
  return t;
}

cuda::UnpackSources DdpEngine::sources_for(int b) const {
  const BucketLayout& L = layouts_[static_cast<size_t>(b)];
  const int parity = epoch_dev_ ? 0 : int(epoch_ & 1u);
  cuda::UnpackSources s;
  s.world = cfg_.world;
  s.epoch_dev = epoch_dev_;
  s.parity_stride = L.slots[1] - L.slots[0];
  s.guard = status_;
  uint8_t* base = bases_[static_cast<size_t>(cfg_.rank)];
  for (int r = 0; r < cfg_.world; ++r) {
    s.payload[r] = base + L.slots[parity] + int64_t(r) * L.slot_bytes + L.shift;
    s.payload_bytes[r] = L.slot_bytes - L.shift;
  }
  return s;
}

void DdpEngine::issue_bucket(int b, int worker) {
  if (cfg_.sharded) {
    issue_shard_push(b, worker);
    if (!cfg_.defer_recv) {
      issue_shard_reduce(b, worker);
      issue_shard_final(b, worker);
    }
    return;
  }
  issue_push(b, worker);
  if (!cfg_.defer_recv) issue_recv(b, worker);
}

// ------------------------------------------------------------------ sharded exchange
int64_t DdpEngine::shard_len(int b, int j) const {
  const int64_t S = layouts_[static_cast<size_t>(b)].shard_elems;
  const int64_t left = buckets_[static_cast<size_t>(b)].numel - int64_t(j) * S;
  return left <= 0 ? 0 : (left < S ? left : S);
}

cuda::SgdApply DdpEngine::sgd_apply_for(int b) const {
  cuda::SgdApply apply;
  if (fused_sgd_) {
    const BucketDesc& B = buckets_[static_cast<size_t>(b)];
    apply.param = param_ + B.offset;
    apply.momentum = momentum_ + B.offset;
    apply.lr = lr_;
    apply.mu = sgd_mu_;
    apply.weight_decay = wd_;
    // buf = g on the first step equals mu * buf + g with the zero-initialised momentum the
    // wrappers allocate; a captured step must not bake the first-step flag in
    apply.first_step = (steps_ == 0 && !epoch_dev_) ? 1 : 0;
    apply.clear_grad = cfg_.clear_grad;
    apply.guard = status_;
  }
  return apply;
}

void DdpEngine::issue_adamw(int b, cudaStream_t stream, int clear_grad) {
  if (!param_ || !momentum_ || !second_) throw std::runtime_error("AdamW needs param and both moment buffers");
  const BucketDesc& B = buckets_[static_cast<size_t>(b)];
  cuda::AdamWApply aw;
  aw.param = param_ + B.offset;
  aw.exp_avg = momentum_ + B.offset;
  aw.exp_avg_sq = second_ + B.offset;
  aw.lr = lr_;
  aw.beta1 = beta1_;
  aw.beta2 = beta2_;
  aw.eps = eps_;
  aw.weight_decay = wd_;
  aw.step = int(steps_) + 1;
  aw.step_dev = epoch_dev_;   // one epoch per step: the device counter is the 1-based step count
  aw.clear_grad = clear_grad < 0 ? cfg_.clear_grad : clear_grad;
  aw.guard = status_;
  check(cuda::adamw_apply_dense(grad_ + B.offset, 1.0f, aw, B.numel, stream), "adamw_apply_dense");
}

// Phase 1: every shard of the bucket is compressed as a payload of its own and stored into the
// slot [rank] of the shard's owner -- one launch (two for TernGrad) over the whole bucket, the
// kernels switching destination from shard to shard (PushTargets::shard_elems).
void DdpEngine::issue_shard_push(int b, int worker) {
  TraceRange range(cfg_.trace != 0, "shard push", b);
  WorkerCtx& w = workers_[static_cast<size_t>(worker)];
  const BucketDesc& B = buckets_[static_cast<size_t>(b)];
  const BucketLayout& L = layouts_[static_cast<size_t>(b)];
  const int parity = epoch_dev_ ? 0 : int(epoch_ & 1u);
  check(cudaStreamWaitEvent(w.push, ready_events_[static_cast<size_t>(b)], 0), "wait ready");
  stamp(b, kStampReady, w.push);
  cuda::PushTargets dst;
  dst.world = cfg_.world;
  dst.epoch = epoch_;
  dst.done = w.done;
  dst.epoch_dev = epoch_dev_;
  dst.parity_stride = L.slots[1] - L.slots[0];
  dst.shard_elems = L.shard_elems;
  dst.guard = status_;
  for (int j = 0; j < cfg_.world; ++j) {
    uint8_t* base = bases_[static_cast<size_t>(j)];
    dst.payload[j] = base + L.slots[parity] + int64_t(cfg_.rank) * L.slot_bytes + L.shift;
    dst.flag[j] = reinterpret_cast<uint32_t*>(base + L.flags) + cfg_.rank;
  }
  // the kernels add the shard term (and, with the epoch on the device, the epoch term)
  const uint64_t seed = cfg_.seed + (epoch_dev_ ? 0 : uint64_t(epoch_) * cuda::kEpochSeedStride) +
                        uint64_t(b) * 0x632BE59BD9B4E019ull;
  float* res = residual_ ? residual_ + B.offset : nullptr;
  if (cfg_.codec == Codec::kTbq) {
    if (!res) throw std::runtime_error("tbq needs a residual buffer");
    check(cuda::tbq_compress(grad_ + B.offset, res, B.numel, cfg_.threshold, dst, w.push), "tbq_compress");
    launches_ += 1;
  } else {
    check(cuda::terngrad_compress(grad_ + B.offset, cfg_.error_feedback ? res : nullptr, B.numel, cfg_.bitwidth,
                                  cfg_.enable_random, seed, dst, w.scratch, w.push),
          "terngrad_compress");
    launches_ += 2;
  }
  stamp(b, kStampPushed, w.push);
  check(cudaEventRecord(w.pushed, w.push), "record pushed");
}

// Phase 2: the owner decodes the `world` payloads of its shard in one pass, averages, and
// re-compresses the average with its own residual into slot [rank] of every rank's phase-2 area.
void DdpEngine::issue_shard_reduce(int b, int worker) {
  TraceRange range(cfg_.trace != 0, "shard reduce", b);
  WorkerCtx& w = workers_[static_cast<size_t>(worker)];
  const BucketDesc& B = buckets_[static_cast<size_t>(b)];
  const BucketLayout& L = layouts_[static_cast<size_t>(b)];
  const int parity = epoch_dev_ ? 0 : int(epoch_ & 1u);
  const int me = cfg_.rank;
  const int64_t n_me = shard_len(b, me);
  const int64_t off = B.offset + int64_t(me) * L.shard_elems;
  uint8_t* mine = bases_[static_cast<size_t>(me)];
  int launched = 0;
  check(cudaStreamWaitEvent(w.recv, w.pushed, 0), "wait pushed");
  // every rank's payload of my shard has arrived
  check(cuda::wait_flags(reinterpret_cast<const uint32_t*>(mine + L.flags), cfg_.world, epoch_,
                         cfg_.flag_timeout_ns, status_, w.recv, epoch_dev_, wait_ns_),
        "wait_flags");
  launched += 1;
  stamp(b, kStampArrived, w.recv);
  // where the averaged, re-compressed shard goes: slot [me] of every rank's phase-2 area
  cuda::PushTargets dst;
  dst.world = cfg_.world;
  dst.epoch = epoch_;
  dst.epoch_dev = epoch_dev_;
  dst.parity_stride = L.slots2[1] - L.slots2[0];
  dst.guard = status_;
  dst.done = w.done + 4;  // its own last-CTA counter: the push stream may be compressing the next bucket
  for (int p = 0; p < cfg_.world; ++p) {
    uint8_t* base = bases_[static_cast<size_t>(p)];
    dst.payload[p] = base + L.slots2[parity] + int64_t(me) * L.slot_bytes + L.shift;
    dst.flag[p] = reinterpret_cast<uint32_t*>(base + L.flags2) + me;
  }
  if (nvls_active()) dst.mc = mc_base_ + L.slots2[parity] + int64_t(me) * L.slot_bytes + L.shift;
  if (n_me == 0) {
    check(cuda::signal_flags(dst, w.recv), "signal_flags");
    launches_ += launched + 1;
    return;
  }
  cuda::UnpackSources src;
  src.world = cfg_.world;
  src.epoch_dev = epoch_dev_;
  src.parity_stride = L.slots[1] - L.slots[0];
  src.guard = status_;
  for (int r = 0; r < cfg_.world; ++r) {
    src.payload[r] = mine + L.slots[parity] + int64_t(r) * L.slot_bytes + L.shift;
    src.payload_bytes[r] = L.slot_bytes - L.shift;
  }
  const float post = cfg_.average ? 1.0f / float(cfg_.world) : 1.0f;
  float* g = grad_ + off;
  float* res2 = residual2_ + residual2_off_[static_cast<size_t>(b)];
  const uint64_t seed = cfg_.seed + (epoch_dev_ ? 0 : uint64_t(epoch_) * cuda::kEpochSeedStride) +
                        uint64_t(b) * 0x632BE59BD9B4E019ull + 0xA24BAED4963EE407ull;
  if (cfg_.codec == Codec::kTbq) {
    check(cuda::tbq_unpack_accum(src, cfg_.threshold, g, n_me, 0, post, cuda::SgdApply{}, w.recv), "tbq_unpack");
    check(cuda::tbq_compress(g, res2, n_me, cfg_.threshold, dst, w.recv), "tbq_compress");
    launched += 2;
  } else {
    check(cuda::terngrad_unpack_accum(src, g, n_me, 0, post, cuda::SgdApply{}, status_, w.recv, cfg_.bitwidth),
          "tern_unpack");
    // its own scratch region: the push stream may be reducing the next bucket's min/max
    void* scratch2 = static_cast<uint8_t*>(w.scratch) + 131072;
    check(cuda::terngrad_compress(g, cfg_.error_feedback ? res2 : nullptr, n_me, cfg_.bitwidth,
                                  cfg_.enable_random, seed, dst, scratch2, w.recv),
          "terngrad_compress");
    launched += 3;
  }
  launches_ += launched;
}

// Phase 3: one pass over the whole bucket that decodes every shard from its owner's payload
// (UnpackSources::shard_elems) and applies the update.
void DdpEngine::issue_shard_final(int b, int worker) {
  TraceRange range(cfg_.trace != 0, "shard final", b);
  WorkerCtx& w = workers_[static_cast<size_t>(worker)];
  const BucketDesc& B = buckets_[static_cast<size_t>(b)];
  const BucketLayout& L = layouts_[static_cast<size_t>(b)];
  const int parity = epoch_dev_ ? 0 : int(epoch_ & 1u);
  uint8_t* mine = bases_[static_cast<size_t>(cfg_.rank)];
  int launched = 0;
  check(cuda::wait_flags(reinterpret_cast<const uint32_t*>(mine + L.flags2), cfg_.world, epoch_,
                         cfg_.flag_timeout_ns, status_, w.recv, epoch_dev_, wait_ns_),
        "wait_flags");
  launched += 1;
  cuda::UnpackSources src;
  src.world = cfg_.world;
  src.epoch_dev = epoch_dev_;
  src.parity_stride = L.slots2[1] - L.slots2[0];
  src.shard_elems = L.shard_elems;
  src.guard = status_;
  for (int j = 0; j < cfg_.world; ++j) {
    src.payload[j] = mine + L.slots2[parity] + int64_t(j) * L.slot_bytes + L.shift;
    src.payload_bytes[j] = L.slot_bytes - L.shift;
  }
  const cuda::SgdApply apply = sgd_apply_for(b);
  if (cfg_.codec == Codec::kTbq) {
    check(cuda::tbq_unpack_accum(src, cfg_.threshold, grad_ + B.offset, B.numel, 0, 1.0f, apply, w.recv), "tbq_unpack");
    launched += 1;
  } else if (cfg_.bitwidth == 2) {
    check(cuda::terngrad_unpack_accum(src, grad_ + B.offset, B.numel, 0, 1.0f, apply, status_, w.recv, cfg_.bitwidth),
          "tern_unpack");
    launched += 1;
  } else {
    // the one-pass form over concatenated shards exists for 2-bit payloads: one launch per shard
    for (int j = 0; j < cfg_.world; ++j) {
      const int64_t nj = shard_len(b, j);
      if (nj == 0) continue;
      const int64_t off = int64_t(j) * L.shard_elems;
      cuda::UnpackSources one = src;
      one.world = 1;
      one.shard_elems = 0;
      one.payload[0] = src.payload[j];
      cuda::SgdApply ap = apply;
      if (ap.param) {
        ap.param += off;
        ap.momentum += off;
      }
      check(cuda::terngrad_unpack_accum(one, grad_ + B.offset + off, nj, 0, 1.0f, ap, status_, w.recv, cfg_.bitwidth),
            "tern_unpack");
      launched += 1;
    }
  }
  if (adamw_) {
    issue_adamw(b, w.recv);
    launched += 1;
  }
  stamp(b, kStampDone, w.recv);
  check(cudaEventRecord(w.tail, w.recv), "record tail");
  w.used = true;
  launches_ += launched;
}

void DdpEngine::reduce_step() {
  if (!cfg_.sharded || !cfg_.defer_recv) return;
  for (size_t b = 0; b < buckets_.size(); ++b) {
    const int worker = int(b) % static_cast<int>(workers_.size());
    if (pool_) pool_->submit_to(worker, [this, b](int w) { issue_shard_reduce(int(b), w); });
    else issue_shard_reduce(int(b), worker);
  }
  if (pool_) pool_->drain();
}

void DdpEngine::issue_push(int b, int worker) {
  TraceRange range(cfg_.trace != 0, "push", b);
  WorkerCtx& w = workers_[static_cast<size_t>(worker)];
  const BucketDesc& B = buckets_[static_cast<size_t>(b)];
  const BucketLayout& L = layouts_[static_cast<size_t>(b)];
  const int64_t n = B.numel;
  float* g = grad_ + B.offset;
  float* res = residual_ ? residual_ + B.offset : nullptr;
  // with the epoch on the device the kernel adds the epoch term itself
  const uint64_t seed = cfg_.seed + (epoch_dev_ ? 0 : uint64_t(epoch_) * cuda::kEpochSeedStride) +
                        uint64_t(b) * 0x632BE59BD9B4E019ull;
  // ---- push stream: compress and deliver
  check(cudaStreamWaitEvent(w.push, ready_events_[static_cast<size_t>(b)], 0), "wait ready");
  stamp(b, kStampReady, w.push);
  cuda::PushTargets dst = targets_for(b, w);
  int launched = 0;
  switch (cfg_.codec) {
    case Codec::kTbq:
      if (!res) throw std::runtime_error("tbq needs a residual buffer");
      check(cuda::tbq_compress(g, res, n, cfg_.threshold, dst, w.push), "tbq_compress");
      launched += 1;
      break;
    case Codec::kTernGrad:
      check(cuda::terngrad_compress(g, cfg_.error_feedback ? res : nullptr, n, cfg_.bitwidth,
                                    cfg_.enable_random, seed, dst, w.scratch, w.push),
            "terngrad_compress");
      launched += 2;
      break;
    case Codec::kSparse: {
      if (!res) throw std::runtime_error("sparse codecs need a residual buffer");
      // one fused pipeline: the codec's state update (GradDrop's R += G, or DGC's momentum
      // correction with clipping and factor masking) happens inside the compressor's single pass
      // over the bucket, which also leaves zeros in the gradient: the dense gradient is rebuilt
      // from the payloads by the receive half
      cuda::SparseFuse fuse;
      fuse.zero_grad = 1;
      if (cfg_.momentum_correction) {
        if (!aux_) throw std::runtime_error("momentum correction needs the velocity buffer");
        fuse.mode = 2;
        fuse.grad = g;
        fuse.u = aux_ + B.offset;
        fuse.momentum = cfg_.dgc_momentum;
        fuse.clip = cfg_.dgc_clip;
        fuse.sumsq = reinterpret_cast<float*>(static_cast<uint8_t*>(w.scratch) + 12288);
      } else if (cfg_.sparse_accumulate) {
        fuse.mode = 1;
        fuse.grad = g;
      } else {
        // plain DGC selects from the caller's accumulator; the gradient itself is not an input
        fuse.mode = 0;
        check(cudaMemsetAsync(g, 0, size_t(n) * 4, w.push), "clear grad");
      }
      void* sparse_scratch = static_cast<uint8_t*>(w.scratch) + 16384;
      check(cuda::sparse_compress_fused(fuse, res, n, cfg_.sample_rate, keep_fraction_, seed, dst, sparse_scratch,
                                        w.push),
            "sparse_compress");
      launched += 6 + (fuse.mode == 2 && fuse.clip > 0.f ? 1 : 0);
      if (sparse_stats_host_)
        check(cuda::sparse_read_stats(sparse_scratch, sparse_stats_host_ + 4 * b, w.push), "sparse stats");
      break;
    }
    case Codec::kEcq:
      if (!res) throw std::runtime_error("ecq needs a history buffer");
      check(cuda::ecq_compress(g, res, n, cfg_.alpha, cfg_.beta, cfg_.bitwidth, seed, dst,
                               w.scratch, w.push),
            "ecq_compress");
      launched += 2;
      break;
    case Codec::kDense: {
      // own slot in local memory; peers pull it
      if (epoch_dev_) {
        float* even = reinterpret_cast<float*>(bases_[static_cast<size_t>(cfg_.rank)] + L.slots[0] +
                                               int64_t(cfg_.rank) * L.slot_bytes);
        check(cuda::dense_stage(g, even, (L.slots[1] - L.slots[0]) / 4, epoch_dev_, n, w.push), "dense_stage");
      } else {
        uint8_t* slot = bases_[static_cast<size_t>(cfg_.rank)] + L.slots[epoch_ & 1u] +
                        int64_t(cfg_.rank) * L.slot_bytes;
        check(cudaMemcpyAsync(slot, g, size_t(n) * 4, cudaMemcpyDeviceToDevice, w.push), "copy");
      }
      check(cuda::signal_flags(dst, w.push), "signal_flags");
      launched += 1;
      break;
    }
  }

  stamp(b, kStampPushed, w.push);
  check(cudaEventRecord(w.pushed, w.push), "record pushed");
  launches_ += launched;
}

void DdpEngine::issue_recv(int b, int worker) {
  TraceRange range(cfg_.trace != 0, "recv", b);
  WorkerCtx& w = workers_[static_cast<size_t>(worker)];
  const BucketDesc& B = buckets_[static_cast<size_t>(b)];
  const BucketLayout& L = layouts_[static_cast<size_t>(b)];
  const int64_t n = B.numel;
  float* g = grad_ + B.offset;
  const float post = cfg_.average ? 1.0f / float(cfg_.world) : 1.0f;
  const cuda::SgdApply apply = sgd_apply_for(b);
  int launched = 0;
  // The receive half starts once this rank's own payload and flag are out: the flag wait below
  // then only ever waits for other GPUs, never for a kernel of this GPU that might not have
  // been scheduled yet (and, under stream capture, this is what brings the recv stream into
  // the capture).
  check(cudaStreamWaitEvent(w.recv, w.pushed, 0), "wait pushed");
  // ---- recv stream: wait for all ranks, decode everything in one pass
  const uint32_t* flags = reinterpret_cast<const uint32_t*>(bases_[static_cast<size_t>(cfg_.rank)] + L.flags);
  check(cuda::wait_flags(flags, cfg_.world, epoch_, cfg_.flag_timeout_ns, status_, w.recv, epoch_dev_, wait_ns_),
        "wait_flags");
  launched += 1;
  stamp(b, kStampArrived, w.recv);
  cuda::UnpackSources src = sources_for(b);
  bool applied = false;
  switch (cfg_.codec) {
    case Codec::kTbq:
      check(cuda::tbq_unpack_accum(src, cfg_.threshold, g, n, 0, post, apply, w.recv), "tbq_unpack");
      applied = fused_sgd_;
      launched += 1;
      break;
    case Codec::kTernGrad:
      check(cuda::terngrad_unpack_accum(src, g, n, 0, post, apply, status_, w.recv, cfg_.bitwidth), "tern_unpack");
      applied = fused_sgd_;
      launched += 1;
      break;
    case Codec::kSparse:
      // the compressor left zeros in the bucket: the payloads are added onto them
      check(cuda::sparse_unpack_accum(src, g, n, 1, post, status_, w.recv), "sparse_unpack");
      launched += cfg_.world;
      break;
    case Codec::kEcq:
      check(cuda::ecq_unpack_accum(src, g, n, 0, post, status_, w.recv), "ecq_unpack");
      launched += 1;
      break;
    case Codec::kDense: {
      const float* srcs[cuda::kMaxWorld];
      for (int r = 0; r < cfg_.world; ++r)
        srcs[r] = reinterpret_cast<const float*>(bases_[static_cast<size_t>(r)] +
                                                 L.slots[epoch_dev_ ? 0 : (epoch_ & 1u)] + int64_t(r) * L.slot_bytes);
      check(cuda::dense_gather_sum(srcs, cfg_.world, g, n, post, w.recv, epoch_dev_, (L.slots[1] - L.slots[0]) / 4,
                                   status_),
            "dense_gather_sum");
      launched += 1;
      break;
    }
  }
  // Sparse codecs: the dense gradient holds the scattered payload entries and zeros.  Instead of
  // letting the optimizer kernel write zeros over all of it again, only the scattered positions
  // are cleared afterwards.
  const bool sparse_clear = cfg_.codec == Codec::kSparse && cfg_.clear_grad && (fused_sgd_ || adamw_);
  if (fused_sgd_ && !applied) {
    cuda::SgdApply dense = apply;
    if (sparse_clear) dense.clear_grad = 0;
    check(cuda::sgd_apply_dense(g, 1.0f, dense, n, w.recv), "sgd_apply_dense");
    launched += 1;
  }
  if (adamw_) {
    issue_adamw(b, w.recv, sparse_clear ? 0 : cfg_.clear_grad);
    launched += 1;
  }
  if (sparse_clear) {
    check(cuda::sparse_clear(src, g, n, w.recv), "sparse_clear");
    launched += 1;
  }
  stamp(b, kStampDone, w.recv);
  check(cudaEventRecord(w.tail, w.recv), "record tail");
  w.used = true;
  launches_ += launched;
}

void DdpEngine::finish_step(cudaStream_t consumer) {
  // flush buckets whose hooks did not all fire (parameters without gradient)
  for (size_t b = 0; b < buckets_.size(); ++b)
    if (submitted_[b].load() == 0) bucket_ready(int(b), consumer);
  {
    std::unique_lock<std::mutex> lk(mu_);
    cv_.wait(lk, [&] { return issued_ >= static_cast<int>(buckets_.size()); });
  }
  if (cfg_.defer_recv) {
    for (size_t b = 0; b < buckets_.size(); ++b) {
      const int worker = int(b) % static_cast<int>(workers_.size());
      if (cfg_.sharded) {
        if (pool_) pool_->submit_to(worker, [this, b](int w) { issue_shard_final(int(b), w); });
        else issue_shard_final(int(b), worker);
      } else if (pool_) {
        pool_->submit_to(worker, [this, b](int w) { issue_recv(int(b), w); });
      } else {
        issue_recv(int(b), worker);
      }
    }
    if (pool_) pool_->drain();
  }
  if (pool_ && pool_->error_count() > 0) {
    const std::string err = pool_->last_error();
    throw std::runtime_error("hipress engine: worker failed: " + err);
  }
  for (auto& w : workers_)
    if (w.used) check(cudaStreamWaitEvent(consumer, w.tail, 0), "wait tail");
  if (stamps_) {
    check(cuda::stamp_time(stamps_ + buckets_.size() * kStampCount + 1, consumer), "stamp");
    launches_ += 1;
  }
  ++steps_;
}

void DdpEngine::stamp(int b, int which, cudaStream_t stream) {
  if (!stamps_) return;
  check(cuda::stamp_time(stamps_ + size_t(b) * kStampCount + which, stream), "stamp");
  launches_ += 1;
}

void DdpEngine::set_progress(int64_t steps, uint32_t epoch) {
  steps_ = steps;
  epoch_ = epoch;
  if (epoch_dev_) {
    check(cudaDeviceSynchronize(), "sync");
    check(cudaMemcpy(epoch_dev_, &epoch, sizeof(epoch), cudaMemcpyHostToDevice), "restore epoch");
  }
}

std::vector<unsigned long long> DdpEngine::wait_stats() {
  std::vector<unsigned long long> host(3, 0ull);
  check(cudaDeviceSynchronize(), "sync");
  check(cudaMemcpy(host.data(), wait_ns_, 3 * sizeof(unsigned long long), cudaMemcpyDeviceToHost), "read wait stats");
  check(cudaMemset(wait_ns_, 0, 64), "reset wait stats");
  return host;
}

std::vector<unsigned int> DdpEngine::sparse_stats() {
  std::vector<unsigned int> out;
  if (!sparse_stats_host_) return out;
  check(cudaDeviceSynchronize(), "sync");
  out.assign(sparse_stats_host_, sparse_stats_host_ + buckets_.size() * 4);
  return out;
}

std::vector<int64_t> DdpEngine::stage_times() {
  std::vector<int64_t> out;
  if (!stamps_) return out;
  const size_t count = buckets_.size() * kStampCount + 2;
  std::vector<unsigned long long> host(count, 0ull);
  check(cudaDeviceSynchronize(), "sync");
  check(cudaMemcpy(host.data(), stamps_, count * sizeof(unsigned long long), cudaMemcpyDeviceToHost), "read stamps");
  const unsigned long long t0 = host[buckets_.size() * kStampCount];
  for (size_t i = 0; i < count; ++i) {
    if (i == buckets_.size() * kStampCount) continue;  // the begin stamp itself
    out.push_back(host[i] == 0 ? 0 : int64_t(host[i]) - int64_t(t0));
  }
  return out;
}

int DdpEngine::check_status() {
  int host[4] = {0, 0, 0, 0};
  check(cudaDeviceSynchronize(), "sync");
  check(cudaMemcpy(host, status_, sizeof(host), cudaMemcpyDeviceToHost), "read status");
  if (host[0] != 0) check(cudaMemset(status_, 0, 64), "reset status");
  return host[0];
}

int64_t DdpEngine::wire_bytes_per_step() const {
  int64_t total = 0;
  for (size_t b = 0; b < buckets_.size(); ++b) total += payload_capacity(int(b));
  return total * (cfg_.world - 1);
}
int64_t DdpEngine::dense_bytes_per_step() const {
  int64_t total = 0;
  for (auto& b : buckets_) total += b.numel * 4;
  return total;
}

}  // namespace runtime
}  // namespace hipress
