// Symmetric receive memory: every rank allocates one buffer of the same size,
// exports it, and maps every peer's buffer into its own address space, so that
// kernels can store packed payloads straight into a peer GPU's memory over
// NVLink / NVSwitch.  The reference has no transport at all: it stages payloads
// through a CPU tensor for an external one (ref hp_cuda.cpp:307, 468, 616).
//
// Handle exchange is the caller's job (the Python layer all-gathers the
// 64-byte handles through torch.distributed); this class only owns memory.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

namespace hipress {
namespace comm {

class SymmetricBuffer {
 public:
  // Allocates and zero-fills `bytes` on the current device.
  SymmetricBuffer(size_t bytes, int rank, int world);
  // Adopts memory that somebody else allocated, mapped and owns: bases[r] is rank r's buffer as
  // mapped in this process, multicast an address whose stores reach the same offset of every
  // rank's buffer through the NVLink switch (0 when there is none).  Nothing is freed here.
  SymmetricBuffer(const std::vector<uint64_t>& bases, uint64_t multicast, size_t bytes, int rank, int world);
  ~SymmetricBuffer();
  SymmetricBuffer(const SymmetricBuffer&) = delete;
  SymmetricBuffer& operator=(const SymmetricBuffer&) = delete;

  // Opaque cudaIpcMemHandle_t of the local buffer.
  std::string export_handle() const;
  // handles[r] is rank r's exported handle (entry `rank` is ignored).
  void open_peers(const std::vector<std::string>& handles);
  // Single-process emulation of several ranks on one device (tests): take the
  // peers' base pointers as they are.
  void adopt_peers(const std::vector<uint64_t>& base_pointers);

  uint8_t* base(int r) const { return ptr_.at(static_cast<size_t>(r)); }
  uint8_t* local() const { return ptr_.at(static_cast<size_t>(rank_)); }
  // NVLS multicast mapping of the buffer, or null.
  uint8_t* multicast() const { return multicast_; }
  size_t bytes() const { return bytes_; }
  int rank() const { return rank_; }
  int world() const { return world_; }
  bool connected() const { return connected_; }

 private:
  size_t bytes_;
  int rank_, world_;
  bool connected_ = false;
  bool owned_ = true;
  uint8_t* multicast_ = nullptr;
  std::vector<uint8_t*> ptr_;
  std::vector<bool> opened_;
};

// True when `dev` can map device `peer`'s memory (NVLink or PCIe P2P).
bool can_access_peer(int dev, int peer);
// CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED of the device (NVLS capability probe;
// host attribute only, nothing is bound).
bool multicast_supported(int dev);

}  // namespace comm
}  // namespace hipress
