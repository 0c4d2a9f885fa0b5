#include "symmem.h"

#include <cuda.h>
#include <cuda_runtime.h>
#include <sys/socket.h>
#include <sys/time.h>
#include <sys/un.h>
#include <unistd.h>

#include <cerrno>
#include <cstring>
#include <map>
#include <random>
#include <sstream>
#include <thread>

#include "check.h"
#include "layout.h"

namespace fairring {

namespace {

// The driver API is reached through the runtime (cudaGetDriverEntryPoint), so
// the library neither links libcuda nor fails to load on a machine without a
// driver; only allocate() needs it.
struct Drv {
#define FR_DRV_SYMBOLS(X)           \
  X(cuGetErrorString)               \
  X(cuDeviceGet)                    \
  X(cuDeviceGetAttribute)           \
  X(cuMemCreate)                    \
  X(cuMemRelease)                   \
  X(cuMemAddressReserve)            \
  X(cuMemAddressFree)               \
  X(cuMemMap)                       \
  X(cuMemUnmap)                     \
  X(cuMemSetAccess)                 \
  X(cuMemExportToShareableHandle)   \
  X(cuMemImportFromShareableHandle) \
  X(cuMemGetAllocationGranularity)  \
  X(cuMulticastCreate)              \
  X(cuMulticastAddDevice)           \
  X(cuMulticastBindMem)             \
  X(cuMulticastUnbind)              \
  X(cuMulticastGetGranularity)
#define X(name) decltype(&::name) name = nullptr;
  FR_DRV_SYMBOLS(X)
#undef X
  bool ok = false;
  std::string why;

  static Drv& get() {
    static Drv d = load();
    return d;
  }

 private:
  static Drv load() {
    Drv d;
    d.ok = true;
#define X(name)                                                                          \
  {                                                                                      \
    void* fn = nullptr;                                                                  \
    cudaDriverEntryPointQueryResult q;                                                   \
    cudaError_t e = cudaGetDriverEntryPoint(#name, &fn, cudaEnableDefault, &q);          \
    if (e != cudaSuccess || fn == nullptr || q != cudaDriverEntryPointSuccess) {         \
      d.ok = false;                                                                      \
      if (d.why.empty()) d.why = std::string("driver entry point ") + #name + " missing"; \
      (void)cudaGetLastError();                                                          \
    } else {                                                                             \
      d.name = reinterpret_cast<decltype(d.name)>(fn);                                   \
    }                                                                                    \
  }
    FR_DRV_SYMBOLS(X)
#undef X
    return d;
  }
};

std::string cuErr(CUresult r) {
  const char* s = nullptr;
  if (Drv::get().cuGetErrorString) Drv::get().cuGetErrorString(r, &s);
  return s ? s : ("CUresult " + std::to_string((int)r));
}

#define FR_CU(expr)                                                                     \
  do {                                                                                  \
    CUresult fr_r_ = (expr);                                                            \
    if (fr_r_ != CUDA_SUCCESS)                                                          \
      ::fairring::detail::fail(__FILE__, __LINE__, "driver call failed: " #expr, cuErr(fr_r_)); \
  } while (0)

struct FdMsg {
  int32_t src;
  int32_t tag;
};

}  // namespace

struct SymmAllocator::Impl {
  int sock = -1;
  std::string token;
  std::map<std::pair<int, int>, int> inbox;  // (src, tag) -> fd

  struct VmmBook {
    size_t size = 0;
    CUmemGenericAllocationHandle local = 0;
    std::vector<CUmemGenericAllocationHandle> imported;  // [world], 0 for self
    std::vector<CUdeviceptr> va;                         // [world]
    CUmemGenericAllocationHandle mc = 0;
    CUdeviceptr mc_va = 0;
    bool mc_bound = false;
  };
  std::map<void*, VmmBook> vmm_books;  // keyed by local ptr
  std::map<void*, std::vector<void*>> ipc_books;

  static sockaddr_un addrOf(const std::string& token, int rank, socklen_t* len) {
    sockaddr_un a{};
    a.sun_family = AF_UNIX;
    std::string name = "fairring-" + token + "-" + std::to_string(rank);
    FR_CHECK(name.size() + 1 < sizeof(a.sun_path), "socket name too long");
    a.sun_path[0] = '\0';  // abstract namespace: nothing to unlink, vanishes with the process
    std::memcpy(a.sun_path + 1, name.data(), name.size());
    *len = (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + name.size());
    return a;
  }

  void openSocket(int rank, std::chrono::milliseconds timeout) {
    sock = ::socket(AF_UNIX, SOCK_DGRAM, 0);
    FR_CHECK(sock >= 0, "socket(): ", std::strerror(errno));
    socklen_t len;
    sockaddr_un a = addrOf(token, rank, &len);
    FR_CHECK(::bind(sock, (sockaddr*)&a, len) == 0, "bind(): ", std::strerror(errno));
    timeval tv;
    tv.tv_sec = (long)(timeout.count() / 1000);
    tv.tv_usec = (long)((timeout.count() % 1000) * 1000);
    if (tv.tv_sec == 0 && tv.tv_usec == 0) tv.tv_sec = 1;
    ::setsockopt(sock, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
    ::setsockopt(sock, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof(tv));
  }

  void sendFd(int my_rank, int dst, int tag, int fd) {
    FdMsg m{my_rank, tag};
    iovec iov{&m, sizeof(m)};
    alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))] = {};
    msghdr msg{};
    socklen_t len;
    sockaddr_un a = addrOf(token, dst, &len);
    msg.msg_name = &a;
    msg.msg_namelen = len;
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    msg.msg_control = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    cmsghdr* c = CMSG_FIRSTHDR(&msg);
    c->cmsg_level = SOL_SOCKET;
    c->cmsg_type = SCM_RIGHTS;
    c->cmsg_len = CMSG_LEN(sizeof(int));
    std::memcpy(CMSG_DATA(c), &fd, sizeof(int));
    ssize_t n = ::sendmsg(sock, &msg, 0);
    FR_CHECK(n == (ssize_t)sizeof(m), "sendmsg() to rank ", dst, ": ", std::strerror(errno));
  }

  int recvFd(int src, int tag) {
    for (;;) {
      auto it = inbox.find({src, tag});
      if (it != inbox.end()) {
        int fd = it->second;
        inbox.erase(it);
        return fd;
      }
      FdMsg m{};
      iovec iov{&m, sizeof(m)};
      alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))] = {};
      msghdr msg{};
      msg.msg_iov = &iov;
      msg.msg_iovlen = 1;
      msg.msg_control = ctrl;
      msg.msg_controllen = sizeof(ctrl);
      ssize_t n = ::recvmsg(sock, &msg, 0);
      FR_CHECK(n == (ssize_t)sizeof(m), "recvmsg() waiting for a handle from rank ", src, ": ",
               n < 0 ? std::strerror(errno) : "short message");
      cmsghdr* c = CMSG_FIRSTHDR(&msg);
      FR_CHECK(c != nullptr && c->cmsg_type == SCM_RIGHTS, "message without a file descriptor");
      int fd;
      std::memcpy(&fd, CMSG_DATA(c), sizeof(int));
      inbox[{m.src, m.tag}] = fd;
    }
  }
};

namespace {
// Every rank contributes a yes/no; true only if all said yes.
bool vote(KvStore& s, const std::string& name, int world, bool mine,
          std::chrono::milliseconds timeout) {
  s.add(name + "/yes", mine ? 1 : 0);
  s.barrier(name + "/n", world, timeout);
  return s.add(name + "/yes", 0) == world;
}
}  // namespace

SymmAllocator::SymmAllocator(std::shared_ptr<KvStore> store, int rank, int world, int device,
                             SymmTransport transport, NvlsMode nvls,
                             std::chrono::milliseconds timeout)
    : impl_(new Impl), store_(std::move(store)), rank_(rank), world_(world), device_(device),
      timeout_(timeout) {
  // Can this rank share VMM allocations by file descriptor, and multicast?
  bool vmm_here = false, mc_here = false;
  std::string why;
  if (transport != SymmTransport::IPC) {
    Drv& d = Drv::get();
    if (!d.ok) {
      why = d.why;
    } else {
      CUdevice dev;
      int v = 0;
      if (d.cuDeviceGet(&dev, device) == CUDA_SUCCESS &&
          d.cuDeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED,
                                 dev) == CUDA_SUCCESS &&
          v != 0) {
        vmm_here = true;
        int m = 0;
        if (nvls != NvlsMode::OFF && world > 1 &&
            d.cuDeviceGetAttribute(&m, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) == CUDA_SUCCESS)
          mc_here = m != 0;
      } else {
        why = "device does not support POSIX fd memory handles";
      }
    }
  }
  use_vmm_ = vote(*store_, "symm/cap_vmm", world, vmm_here, timeout_);
  FR_CHECK(use_vmm_ || transport != SymmTransport::VMM, "VMM transport demanded but unavailable: ",
           why);
  mc_ok_ = use_vmm_ && vote(*store_, "symm/cap_mc", world, mc_here, timeout_);
  FR_CHECK(mc_ok_ || nvls != NvlsMode::ON || world == 1,
           "FAIRRING_NVLS=1 but multicast is not supported on every rank");

  if (use_vmm_ && world > 1) {
    if (rank == 0) {
      std::random_device rd;
      std::ostringstream os;
      os << std::hex << rd() << rd() << "-" << ::getpid();
      store_->setString("symm/token", os.str());
    }
    impl_->token = store_->getString("symm/token");
    impl_->openSocket(rank, timeout_);
    store_->barrier("symm/sockets", world, timeout_);
  }
  desc_ = std::string(use_vmm_ ? "vmm" : "ipc") + (mc_ok_ ? "+multicast" : "");
}

SymmAllocator::~SymmAllocator() {
  if (impl_ && impl_->sock >= 0) ::close(impl_->sock);
  for (auto& kv : impl_->inbox) ::close(kv.second);
}

SymmRegion SymmAllocator::allocate(size_t bytes, bool want_multicast) {
  FR_CHECK(bytes > 0, "empty symmetric allocation");
  const std::string pfx = "symm/a" + std::to_string(alloc_seq_++);
  SymmRegion reg;
  reg.ptrs.assign(world_, nullptr);
  FR_CUDA(cudaSetDevice(device_));

  if (!use_vmm_) {
    size_t size = (size_t)roundUp((int64_t)bytes, 2 << 20);
    void* p = nullptr;
    FR_CUDA(cudaMalloc(&p, size));
    FR_CUDA(cudaMemset(p, 0, size));
    FR_CUDA(cudaDeviceSynchronize());
    reg.bytes = size;
    reg.ptrs[rank_] = p;
    if (world_ > 1) {
      cudaIpcMemHandle_t h;
      FR_CUDA(cudaIpcGetMemHandle(&h, p));
      store_->setPod(pfx + "/ipc/" + std::to_string(rank_), h);
      for (int r = 0; r < world_; ++r) {
        if (r == rank_) continue;
        auto ph = store_->getPod<cudaIpcMemHandle_t>(pfx + "/ipc/" + std::to_string(r));
        void* q = nullptr;
        FR_CUDA(cudaIpcOpenMemHandle(&q, ph, cudaIpcMemLazyEnablePeerAccess));
        reg.ptrs[r] = q;
      }
      store_->barrier(pfx + "/mapped", world_, timeout_);
    }
    impl_->ipc_books[p] = reg.ptrs;
    return reg;
  }

  Drv& d = Drv::get();
  Impl::VmmBook book;
  book.imported.assign(world_, 0);
  book.va.assign(world_, 0);

  CUmemAllocationProp prop{};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device_;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t gran = 0;
  FR_CU(d.cuMemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));

  const bool try_mc = want_multicast && mc_ok_ && world_ > 1;
  CUmulticastObjectProp mp{};
  size_t mgran = 0;
  if (try_mc) {
    mp.numDevices = (unsigned)world_;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    mp.flags = 0;
    mp.size = (size_t)roundUp((int64_t)bytes, (int64_t)gran);
    if (d.cuMulticastGetGranularity(&mgran, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) !=
        CUDA_SUCCESS)
      mgran = 0;
  }
  size_t align = gran;
  if (mgran > align) align = mgran;
  const size_t size = (size_t)roundUp((int64_t)bytes, (int64_t)align);
  book.size = size;
  reg.bytes = size;
  reg.vmm = true;

  CUmemAccessDesc acc{};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device_;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;

  FR_CU(d.cuMemCreate(&book.local, size, &prop, 0));
  FR_CU(d.cuMemAddressReserve(&book.va[rank_], size, align, 0, 0));
  FR_CU(d.cuMemMap(book.va[rank_], size, 0, book.local, 0));
  FR_CU(d.cuMemSetAccess(book.va[rank_], size, &acc, 1));
  reg.ptrs[rank_] = reinterpret_cast<void*>(book.va[rank_]);
  FR_CUDA(cudaMemset(reg.ptrs[rank_], 0, size));
  FR_CUDA(cudaDeviceSynchronize());

  if (world_ > 1) {
    const int tag = alloc_seq_ * 2;
    int fd = -1;
    FR_CU(d.cuMemExportToShareableHandle(&fd, book.local, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR,
                                         0));
    for (int k = 1; k < world_; ++k) impl_->sendFd(rank_, (rank_ + k) % world_, tag, fd);
    for (int k = 1; k < world_; ++k) {
      const int r = (rank_ + world_ - k) % world_;
      int pfd = impl_->recvFd(r, tag);
      FR_CU(d.cuMemImportFromShareableHandle(&book.imported[r], (void*)(uintptr_t)pfd,
                                             CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
      ::close(pfd);
      FR_CU(d.cuMemAddressReserve(&book.va[r], size, align, 0, 0));
      FR_CU(d.cuMemMap(book.va[r], size, 0, book.imported[r], 0));
      FR_CU(d.cuMemSetAccess(book.va[r], size, &acc, 1));
      reg.ptrs[r] = reinterpret_cast<void*>(book.va[r]);
    }
    ::close(fd);
    store_->barrier(pfx + "/mapped", world_, timeout_);

    if (try_mc) {
      // Rank 0 creates the multicast object; everybody adds its device, then
      // (after all devices are in) binds its memory and maps the alias.  Any
      // refusal makes all ranks drop NVLS together and carry on with peer loads.
      mp.size = size;
      bool ok = true;
      if (rank_ == 0) {
        ok = d.cuMulticastCreate(&book.mc, &mp) == CUDA_SUCCESS;
        store_->setPod<int32_t>(pfx + "/mc_created", ok ? 1 : 0);
        if (ok) {
          int mfd = -1;
          FR_CU(d.cuMemExportToShareableHandle(&mfd, book.mc,
                                               CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
          for (int r = 1; r < world_; ++r) impl_->sendFd(rank_, r, tag + 1, mfd);
          ::close(mfd);
        }
      } else {
        ok = store_->getPod<int32_t>(pfx + "/mc_created") == 1;
        if (ok) {
          int mfd = impl_->recvFd(0, tag + 1);
          ok = d.cuMemImportFromShareableHandle(&book.mc, (void*)(uintptr_t)mfd,
                                                CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) ==
               CUDA_SUCCESS;
          ::close(mfd);
        }
      }
      CUdevice dev = 0;
      if (ok) ok = d.cuDeviceGet(&dev, device_) == CUDA_SUCCESS;
      if (ok) ok = d.cuMulticastAddDevice(book.mc, dev) == CUDA_SUCCESS;
      ok = vote(*store_, pfx + "/mc_added", world_, ok, timeout_);
      if (ok) {
        bool bound = d.cuMulticastBindMem(book.mc, 0, book.local, 0, size, 0) == CUDA_SUCCESS;
        book.mc_bound = bound;
        if (bound) {
          bound = d.cuMemAddressReserve(&book.mc_va, size, align, 0, 0) == CUDA_SUCCESS &&
                  d.cuMemMap(book.mc_va, size, 0, book.mc, 0) == CUDA_SUCCESS &&
                  d.cuMemSetAccess(book.mc_va, size, &acc, 1) == CUDA_SUCCESS;
        }
        ok = vote(*store_, pfx + "/mc_bound", world_, bound, timeout_);
      }
      if (ok) {
        reg.mc_ptr = reinterpret_cast<void*>(book.mc_va);
      } else {
        if (book.mc_va) {
          d.cuMemUnmap(book.mc_va, size);
          d.cuMemAddressFree(book.mc_va, size);
          book.mc_va = 0;
        }
        if (book.mc_bound) d.cuMulticastUnbind(book.mc, dev, 0, size);
        book.mc_bound = false;
        if (book.mc) d.cuMemRelease(book.mc);
        book.mc = 0;
      }
    }
  }
  impl_->vmm_books[reg.ptrs[rank_]] = book;
  return reg;
}

void SymmAllocator::release(SymmRegion& reg) {
  if (reg.ptrs.empty() || reg.ptrs[rank_] == nullptr) return;
  cudaSetDevice(device_);
  cudaDeviceSynchronize();
  // Nobody may still be reading this rank's memory: wait for all ranks, but do
  // not hang shutdown on a rank that is already gone.
  const std::string pfx = "symm/r" + std::to_string(alloc_seq_++);
  if (world_ > 1) {
    try {
      store_->barrier(pfx, world_, std::chrono::milliseconds(5000));
    } catch (const std::exception&) {
    }
  }
  void* local = reg.ptrs[rank_];
  if (!reg.vmm) {
    auto it = impl_->ipc_books.find(local);
    if (it != impl_->ipc_books.end()) {
      for (int r = 0; r < world_; ++r)
        if (r != rank_ && it->second[r]) cudaIpcCloseMemHandle(it->second[r]);
      impl_->ipc_books.erase(it);
    }
    cudaFree(local);
  } else {
    Drv& d = Drv::get();
    auto it = impl_->vmm_books.find(local);
    if (it != impl_->vmm_books.end()) {
      Impl::VmmBook& b = it->second;
      if (b.mc_va) {
        d.cuMemUnmap(b.mc_va, b.size);
        d.cuMemAddressFree(b.mc_va, b.size);
      }
      if (b.mc) {
        CUdevice dev = 0;
        d.cuDeviceGet(&dev, device_);
        if (b.mc_bound) d.cuMulticastUnbind(b.mc, dev, 0, b.size);
        d.cuMemRelease(b.mc);
      }
      for (int r = 0; r < world_; ++r) {
        if (b.va[r]) {
          d.cuMemUnmap(b.va[r], b.size);
          d.cuMemAddressFree(b.va[r], b.size);
        }
        if (r != rank_ && b.imported[r]) d.cuMemRelease(b.imported[r]);
      }
      d.cuMemRelease(b.local);
      impl_->vmm_books.erase(it);
    }
  }
  reg = SymmRegion{};
}

}  // namespace fairring
