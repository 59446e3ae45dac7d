// Allocation-free variant of the TernGrad compressor: same kernels as
// terngrad_compress, but the min/max reduction scratch is a file-scope device
// array instead of memory obtained from an allocator.  See noalloc.h for who
// needs this and the rules of use.
#include "noalloc.h"

#include <mutex>

#include "../common/codec_math.h"
#include "kernels.h"
#include "reduce.cuh"

namespace {

// One copy per GPU that loads this library; zero-initialised at module load.
// In host code this name is only a handle for cudaGetSymbolAddress -- it is not
// a device address and must never be passed to a kernel.
static __device__ __align__(256) unsigned char g_noalloc_scratch[HIPRESS_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
void* g_scratch_addr[kMaxDevices] = {};
thread_local const char* t_last_error = "";

// Device address of the scratch on the current device, resolved once per device.
cudaError_t scratch_for_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) return e;
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return cudaSuccess;
}

}  // namespace

extern "C" int hipress_terngrad_compress_noalloc(const float* grad, float* residual, long long n,
                                                 int bitwidth, int enable_random,
                                                 unsigned long long seed, unsigned char* out,
                                                 long long out_bytes, void* stream) {
  static_assert(sizeof(hipress::cuda::MinMaxScratch) <= HIPRESS_NOALLOC_SCRATCH_BYTES,
                "the built-in scratch must hold the min/max reduction state");
  if (grad == nullptr || out == nullptr || n <= 0 || !hipress::tern_bitwidth_ok(bitwidth)) {
    t_last_error = "bad argument";
    return HIPRESS_ERR_ARGUMENT;
  }
  if (n > HIPRESS_NOALLOC_MAX_ELEMS) {
    t_last_error = "n exceeds HIPRESS_NOALLOC_MAX_ELEMS";
    return HIPRESS_ERR_TOO_LARGE;
  }
  if (out_bytes != hipress::tern_payload_bytes(n, bitwidth)) {
    t_last_error = "out_bytes must be 10 + ceil(n / (8 / bitwidth))";
    return HIPRESS_ERR_ARGUMENT;
  }
  if (hipress::cuda::minmax_scratch_bytes() > size_t(HIPRESS_NOALLOC_SCRATCH_BYTES)) {
    t_last_error = "built-in scratch smaller than the reduction state";
    return HIPRESS_ERR_ARGUMENT;
  }
  void* scratch = nullptr;
  cudaError_t e = scratch_for_current_device(&scratch);
  if (e != cudaSuccess) {
    t_last_error = cudaGetErrorString(e);
    return HIPRESS_ERR_CUDA;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // The array keeps whatever the previous call (possibly an interrupted one)
  // left behind; the reduction's arrival counter and partials must start at 0.
  e = cudaMemsetAsync(scratch, 0, hipress::cuda::minmax_scratch_bytes(), s);
  if (e != cudaSuccess) {
    t_last_error = cudaGetErrorString(e);
    return HIPRESS_ERR_CUDA;
  }
  hipress::cuda::PushTargets dst;
  dst.world = 1;
  dst.payload[0] = out;
  e = hipress::cuda::terngrad_compress(grad, residual, n, bitwidth, enable_random, seed, dst, scratch, s);
  if (e != cudaSuccess) {
    t_last_error = cudaGetErrorString(e);
    return HIPRESS_ERR_CUDA;
  }
  t_last_error = "";
  return HIPRESS_OK;
}

extern "C" const char* hipress_noalloc_last_error(void) { return t_last_error; }
