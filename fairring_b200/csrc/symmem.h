// Symmetric device memory: every rank allocates the same amount, and every
// rank maps everybody's allocation (peer memory over NVLink) plus, when the
// fabric offers it, one multicast alias that fans stores out to / reduces
// loads over all ranks inside the NVSwitch (NVLS).
//
// This replaces the four NCCL communicator families the reference bootstraps
// through the store (fairring/machine.cc:290-382): what is exchanged here are
// memory handles, not communicator ids.
//
// Two transports:
//   VMM : cuMemCreate + POSIX file-descriptor handles passed over a unix
//         socket; required for the multicast alias.
//   IPC : cudaMalloc + cudaIpcMemHandle passed through the store; the fallback
//         when the driver refuses shareable VMM handles.
#pragma once

#include <chrono>
#include <memory>
#include <string>
#include <vector>

#include "kvstore.h"

namespace fairring {

struct SymmRegion {
  size_t bytes = 0;           // usable bytes per rank
  std::vector<void*> ptrs;    // ptrs[r]: rank r's memory as mapped here; ptrs[rank] is local
  void* mc_ptr = nullptr;     // multicast alias, or null
  bool vmm = false;
};

enum class SymmTransport { AUTO, VMM, IPC };
enum class NvlsMode { AUTO, ON, OFF };

class SymmAllocator {
 public:
  // Collective: every rank of the group constructs it at the same point.
  // The CUDA device must already be current.
  SymmAllocator(std::shared_ptr<KvStore> store, int rank, int world, int device,
                SymmTransport transport, NvlsMode nvls, std::chrono::milliseconds timeout);
  ~SymmAllocator();
  SymmAllocator(const SymmAllocator&) = delete;
  SymmAllocator& operator=(const SymmAllocator&) = delete;

  // Collective.  Memory is zero-filled and all ranks have mapped it on return.
  SymmRegion allocate(size_t bytes, bool want_multicast);
  // Collective.  Unmaps peers, then releases the local memory.
  void release(SymmRegion& region);

  bool usingVmm() const { return use_vmm_; }
  bool multicastAvailable() const { return mc_ok_; }
  const std::string& describe() const { return desc_; }

 private:
  struct Impl;
  std::unique_ptr<Impl> impl_;
  std::shared_ptr<KvStore> store_;
  int rank_, world_, device_;
  bool use_vmm_ = false;
  bool mc_ok_ = false;
  std::chrono::milliseconds timeout_;
  std::string desc_;
  int alloc_seq_ = 0;
};

}  // namespace fairring
