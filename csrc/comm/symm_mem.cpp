#include "symm_mem.h"

#include <cstring>
#include <stdexcept>

namespace hipress {
namespace comm {

namespace {
void check(cudaError_t e, const char* what) {
  if (e != cudaSuccess)
    throw std::runtime_error(std::string("hipress symmetric memory: ") + what + ": " +
                             cudaGetErrorString(e));
}
}  // namespace

SymmetricBuffer::SymmetricBuffer(size_t bytes, int rank, int world)
    : bytes_(bytes), rank_(rank), world_(world), ptr_(static_cast<size_t>(world), nullptr),
      opened_(static_cast<size_t>(world), false) {
  if (world < 1 || rank < 0 || rank >= world) throw std::invalid_argument("bad rank/world");
  void* p = nullptr;
  check(cudaMalloc(&p, bytes), "cudaMalloc");
  check(cudaMemset(p, 0, bytes), "cudaMemset");
  check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
  ptr_[static_cast<size_t>(rank)] = static_cast<uint8_t*>(p);
  if (world == 1) connected_ = true;
}

SymmetricBuffer::SymmetricBuffer(const std::vector<uint64_t>& bases, uint64_t multicast, size_t bytes, int rank,
                                 int world)
    : bytes_(bytes), rank_(rank), world_(world), connected_(true), owned_(false),
      multicast_(reinterpret_cast<uint8_t*>(multicast)), ptr_(static_cast<size_t>(world), nullptr),
      opened_(static_cast<size_t>(world), false) {
  if (world < 1 || rank < 0 || rank >= world || static_cast<int>(bases.size()) != world)
    throw std::invalid_argument("bad rank/world or base pointer count");
  for (int r = 0; r < world; ++r) {
    if (bases[static_cast<size_t>(r)] == 0) throw std::invalid_argument("null base pointer");
    ptr_[static_cast<size_t>(r)] = reinterpret_cast<uint8_t*>(bases[static_cast<size_t>(r)]);
  }
}

SymmetricBuffer::~SymmetricBuffer() {
  if (!owned_) return;
  for (int r = 0; r < world_; ++r)
    if (opened_[static_cast<size_t>(r)]) cudaIpcCloseMemHandle(ptr_[static_cast<size_t>(r)]);
  if (ptr_[static_cast<size_t>(rank_)]) cudaFree(ptr_[static_cast<size_t>(rank_)]);
}

std::string SymmetricBuffer::export_handle() const {
  cudaIpcMemHandle_t h;
  check(cudaIpcGetMemHandle(&h, ptr_[static_cast<size_t>(rank_)]), "cudaIpcGetMemHandle");
  return std::string(reinterpret_cast<const char*>(&h), sizeof(h));
}

void SymmetricBuffer::open_peers(const std::vector<std::string>& handles) {
  if (static_cast<int>(handles.size()) != world_) throw std::invalid_argument("need one handle per rank");
  for (int r = 0; r < world_; ++r) {
    if (r == rank_) continue;
    if (handles[static_cast<size_t>(r)].size() != sizeof(cudaIpcMemHandle_t))
      throw std::invalid_argument("malformed IPC handle");
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handles[static_cast<size_t>(r)].data(), sizeof(h));
    void* p = nullptr;
    check(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
    ptr_[static_cast<size_t>(r)] = static_cast<uint8_t*>(p);
    opened_[static_cast<size_t>(r)] = true;
  }
  connected_ = true;
}

void SymmetricBuffer::adopt_peers(const std::vector<uint64_t>& base_pointers) {
  if (static_cast<int>(base_pointers.size()) != world_) throw std::invalid_argument("need one pointer per rank");
  for (int r = 0; r < world_; ++r) {
    if (r == rank_) continue;
    ptr_[static_cast<size_t>(r)] = reinterpret_cast<uint8_t*>(base_pointers[static_cast<size_t>(r)]);
  }
  connected_ = true;
}

bool can_access_peer(int dev, int peer) {
  int ok = 0;
  if (cudaDeviceCanAccessPeer(&ok, dev, peer) != cudaSuccess) return false;
  return ok != 0;
}

bool multicast_supported(int dev) {
  // cudaDevAttr has no multicast entry in every runtime version; query the
  // driver attribute (CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED = 132) through
  // the runtime's driver entry point so that no libcuda link is needed.
  typedef int (*GetAttr)(int*, int, int);
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuDeviceGetAttribute", &fn, cudaEnableDefault, &q) != cudaSuccess ||
      fn == nullptr)
    return false;
  int v = 0;
  if (reinterpret_cast<GetAttr>(fn)(&v, 132, dev) != 0) return false;
  return v != 0;
}

}  // namespace comm
}  // namespace hipress
