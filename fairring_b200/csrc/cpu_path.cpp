#include "cpu_path.h"

#include <c10/util/BFloat16.h>
#include <c10/util/Half.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <cerrno>
#include <cstring>
#include <random>
#include <sstream>
#include <thread>
#include <type_traits>

#include "check.h"

namespace fairring {

namespace {
constexpr size_t kFlagStride = 64;                         // one cache line per source rank
constexpr size_t kHeaderBytes = 4096;                      // flags live here, staging after

template <typename T> struct HostAcc { using type = int64_t; };
template <> struct HostAcc<float> { using type = float; };
template <> struct HostAcc<double> { using type = double; };
template <> struct HostAcc<c10::Half> { using type = float; };
template <> struct HostAcc<c10::BFloat16> { using type = float; };

template <typename A>
inline A combineHost(A a, A b, RedOp op) {
  switch (op) {
    case RedOp::SUM: return a + b;
    case RedOp::MAX: return a > b ? a : b;
    default: return a < b ? a : b;
  }
}
template <typename T>
inline typename HostAcc<T>::type up(T x) { return static_cast<typename HostAcc<T>::type>(x); }
template <typename T>
inline T down(typename HostAcc<T>::type a) { return static_cast<T>(a); }

inline int64_t lenOf(const Seg& s, int c) {
  int64_t n = s.chunk_len;
  int64_t lim = s.limit - (int64_t)c * s.chunk_stride;
  if (lim < n) n = lim;
  return n < 0 ? 0 : n;
}
}  // namespace

struct CpuEngine::Shm {
  std::vector<char*> base;  // [world]
  size_t bytes = 0;
  ~Shm() {
    for (char* p : base)
      if (p) ::munmap(p, bytes);
  }
};

CpuEngine::CpuEngine(std::shared_ptr<KvStore> store, const Topo& topo, const MemoryPlan& plan,
                     std::chrono::milliseconds wait_timeout)
    : store_(std::move(store)), topo_(topo), plan_(plan), wait_timeout_(wait_timeout),
      shm_(new Shm) {
  const int W = topo_.world, me = topo_.rank;
  FR_CHECK(W <= kMaxRanks, "the shared-memory path serves at most ", kMaxRanks, " ranks");
  if (me == 0) {
    std::random_device rd;
    std::ostringstream os;
    os << std::hex << rd() << rd() << "-" << ::getpid();
    store_->setString("shm/token", os.str());
  }
  const std::string token = store_->getString("shm/token");
  auto nameOf = [&](int r) { return "/fairring-" + token + "-" + std::to_string(r); };
  shm_->bytes = kHeaderBytes + (size_t)plan_.half_bytes * 2;
  shm_->base.assign(W, nullptr);

  int fd = ::shm_open(nameOf(me).c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
  FR_CHECK(fd >= 0, "shm_open: ", std::strerror(errno));
  FR_CHECK(::ftruncate(fd, (off_t)shm_->bytes) == 0, "ftruncate: ", std::strerror(errno));
  void* p = ::mmap(nullptr, shm_->bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  ::close(fd);
  FR_CHECK(p != MAP_FAILED, "mmap: ", std::strerror(errno));
  shm_->base[me] = static_cast<char*>(p);
  std::memset(p, 0, kHeaderBytes);
  const auto boot_timeout = std::chrono::milliseconds(60000);
  store_->barrier("shm/created", W, boot_timeout);
  for (int r = 0; r < W; ++r) {
    if (r == me) continue;
    int pfd = ::shm_open(nameOf(r).c_str(), O_RDWR, 0600);
    FR_CHECK(pfd >= 0, "shm_open of rank ", r, " (is it on another host?): ", std::strerror(errno));
    void* q = ::mmap(nullptr, shm_->bytes, PROT_READ | PROT_WRITE, MAP_SHARED, pfd, 0);
    ::close(pfd);
    FR_CHECK(q != MAP_FAILED, "mmap of rank ", r, ": ", std::strerror(errno));
    shm_->base[r] = static_cast<char*>(q);
  }
  store_->barrier("shm/mapped", W, boot_timeout);
  ::shm_unlink(nameOf(me).c_str());  // mappings stay; nothing is left behind on a crash
}

CpuEngine::~CpuEngine() = default;

char* CpuEngine::stage(int rank, int64_t vec) const {
  const uint64_t half = (seq_ & 1u) ? (uint64_t)plan_.half_bytes : 0;
  return shm_->base[rank] + kHeaderBytes + half + (uint64_t)vec * kVecBytes;
}

void CpuEngine::barrier(BarrierKind kind, int idx) {
  const Topo& t = topo_;
  const uint32_t epoch = seq_ * (uint32_t)kBarriersPerOp + (uint32_t)idx + 1u;
  const int n = kind == kAll ? t.world : (kind == kGroup ? t.D : t.M);
  auto peerOf = [&](int i) {
    return kind == kAll ? i : (kind == kGroup ? rankOf(t, t.m, i) : rankOf(t, i, t.d));
  };
  auto flagOf = [&](int owner, int src) {
    return reinterpret_cast<std::atomic<uint32_t>*>(shm_->base[owner] + (size_t)src * kFlagStride);
  };
  bool skip = false;
  if (skip_signals_ > 0) {
    --skip_signals_;
    skip = true;
  }
  if (!skip)
    for (int i = 0; i < n; ++i) {
      const int p = peerOf(i);
      if (p != t.rank) flagOf(p, t.rank)->store(epoch, std::memory_order_release);
    }
  const auto t0 = std::chrono::steady_clock::now();
  for (int i = 0; i < n; ++i) {
    const int p = peerOf(i);
    if (p == t.rank) continue;
    uint64_t spins = 0;
    while ((int32_t)(flagOf(t.rank, p)->load(std::memory_order_acquire) - epoch) < 0) {
      if ((++spins & 255) == 0) {
        FR_CHECK(std::chrono::steady_clock::now() - t0 < wait_timeout_,
                 "timed out after ", wait_timeout_.count(), " ms waiting for rank ", p,
                 " at barrier ", idx, " of collective ", seq_);
        std::this_thread::yield();
      }
    }
  }
}

template <typename T>
void CpuEngine::pushPhase(const T* in, const Seg& s, float scale) {
  using A = typename HostAcc<T>::type;
  const Topo& t = topo_;
  for (int dd = 0; dd < t.D; ++dd)
    for (int j = 0; j < t.M; ++j) {
      const int chunk = rankOf(t, j, dd);
      T* dst = reinterpret_cast<T*>(stage(rankOf(t, t.m, dd), stagingVec(t, s, t.d, j)));
      const T* src = in + (int64_t)chunk * s.chunk_stride;
      const int64_t n = lenOf(s, chunk);
      if (std::is_floating_point<A>::value && scale != 1.0f) {
        for (int64_t i = 0; i < n; ++i) dst[i] = down<T>(up(src[i]) * (A)scale);
      } else {
        std::memcpy(dst, src, (size_t)n * sizeof(T));
      }
    }
}

template <typename T>
void CpuEngine::localReducePhase(const Seg& s, RedOp op, T* out) {
  using A = typename HostAcc<T>::type;
  const Topo& t = topo_;
  for (int j = 0; j < t.M; ++j) {
    const int chunk = rankOf(t, j, t.d);
    const int64_t n = lenOf(s, chunk);
    T* dst = out ? out : reinterpret_cast<T*>(stage(t.rank, stagingVec(t, s, t.d, j)));
    for (int64_t i = 0; i < n; ++i) {
      A acc = up(reinterpret_cast<const T*>(stage(t.rank, stagingVec(t, s, 0, j)))[i]);
      for (int k = 1; k < t.D; ++k)
        acc = combineHost(acc, up(reinterpret_cast<const T*>(stage(t.rank, stagingVec(t, s, k, j)))[i]),
                          op);
      dst[i] = down<T>(acc);
    }
  }
}

template <typename T>
void CpuEngine::serverReducePhase(const Seg& s, RedOp op, T* out) {
  using A = typename HostAcc<T>::type;
  const Topo& t = topo_;
  const int64_t shard = stagingVec(t, s, t.d, t.m);
  const int64_t n = lenOf(s, t.rank);
  for (int64_t i = 0; i < n; ++i) {
    A acc = up(reinterpret_cast<const T*>(stage(rankOf(t, 0, t.d), shard))[i]);
    for (int k = 1; k < t.M; ++k)
      acc = combineHost(acc, up(reinterpret_cast<const T*>(stage(rankOf(t, k, t.d), shard))[i]), op);
    if (out) {
      out[i] = down<T>(acc);
    } else {
      for (int k = 0; k < t.M; ++k)
        reinterpret_cast<T*>(stage(rankOf(t, k, t.d), shard))[i] = down<T>(acc);
    }
  }
}

template <typename T>
void CpuEngine::gatherPhase(T* out, const Seg& s) {
  const Topo& t = topo_;
  for (int dd = 0; dd < t.D; ++dd)
    for (int j = 0; j < t.M; ++j) {
      const int chunk = rankOf(t, j, dd);
      const T* src = reinterpret_cast<const T*>(stage(rankOf(t, t.m, dd), stagingVec(t, s, dd, j)));
      std::memcpy(out + (int64_t)chunk * s.chunk_stride, src, (size_t)lenOf(s, chunk) * sizeof(T));
    }
}

template <typename T>
void CpuEngine::diffusePhase(const T* in, const Seg& s) {
  const Topo& t = topo_;
  const int64_t shard = stagingVec(t, s, t.d, t.m);
  for (int k = 0; k < t.M; ++k)
    std::memcpy(stage(rankOf(t, k, t.d), shard), in, (size_t)s.chunk_len * sizeof(T));
}

template <typename T>
void CpuEngine::pushAllPhase(const T* in, const Seg& s, float scale) {
  using A = typename HostAcc<T>::type;
  const Topo& t = topo_;
  const int W = t.world;
  for (int p = 0; p < W; ++p)
    for (int c = 0; c < W; ++c) {
      T* dst = reinterpret_cast<T*>(stage(p, ((int64_t)t.rank * W + c) * s.qv));
      const T* src = in + (int64_t)c * s.chunk_stride;
      const int64_t n = lenOf(s, c);
      if (std::is_floating_point<A>::value && scale != 1.0f) {
        for (int64_t i = 0; i < n; ++i) dst[i] = down<T>(up(src[i]) * (A)scale);
      } else {
        std::memcpy(dst, src, (size_t)n * sizeof(T));
      }
    }
}

template <typename T>
void CpuEngine::reduceAllPhase(T* out, const Seg& s, RedOp op) {
  using A = typename HostAcc<T>::type;
  const Topo& t = topo_;
  const int W = t.world;
  for (int c = 0; c < W; ++c) {
    const int64_t n = lenOf(s, c);
    for (int64_t i = 0; i < n; ++i) {
      A acc = up(reinterpret_cast<const T*>(stage(t.rank, ((int64_t)0 * W + c) * s.qv))[i]);
      for (int k = 1; k < W; ++k)
        acc = combineHost(
            acc, up(reinterpret_cast<const T*>(stage(t.rank, ((int64_t)k * W + c) * s.qv))[i]), op);
      out[(int64_t)c * s.chunk_stride + i] = down<T>(acc);
    }
  }
}

void CpuEngine::finishOp() {
  ++seq_;
  ++stats_.slices;
}

template <typename T>
void CpuEngine::allReduceT(const T* in, T* out, int64_t numel, RedOp op, float scale) {
  const Topo& t = topo_;
  const int W = t.world;
  const int esize = (int)sizeof(T);
  const int64_t bytes = numel * esize;
  {
    const Seg s = allreduceSeg(numel, esize, W);
    if (bytes <= oneshotMaxBytes && (int64_t)W * W * s.qv * kVecBytes <= plan_.half_bytes) {
      pushAllPhase<T>(in, s, scale);
      barrier(kAll, 0);
      reduceAllPhase<T>(out, s, op);
      ++stats_.oneshot;
      finishOp();
      return;
    }
  }
  const SlicePlan sp = planSlices(numel, esize, W, plan_.max_slice_bytes);
  for (int64_t k = 0; k < sp.num_slices; ++k) {
    const int64_t off = k * sp.slice_elems;
    const int64_t n = std::min(sp.slice_elems, numel - off);
    const Seg s = allreduceSeg(n, esize, W);
    pushPhase<T>(in + off, s, scale);
    barrier(kAll, 0);
    localReducePhase<T>(s, op, nullptr);
    if (t.M > 1) {
      barrier(kRail, 1);
      serverReducePhase<T>(s, op, nullptr);
      barrier(kRail, 2);
      ++stats_.hierarchical;
    } else {
      ++stats_.twoshot;
    }
    barrier(kGroup, 3);
    gatherPhase<T>(out + off, s);
    finishOp();
  }
}

template <typename T>
void CpuEngine::reduceScatterT(const T* in, T* out, int64_t per_rank, RedOp op, float scale) {
  const Topo& t = topo_;
  const int W = t.world;
  const int esize = (int)sizeof(T);
  const int64_t V = kVecBytes / esize;
  int64_t max_len = roundDown(plan_.max_slice_bytes / esize / W, V);
  if (max_len < V) max_len = V;
  for (int64_t off = 0; off < per_rank; off += max_len) {
    const int64_t len = std::min(max_len, per_rank - off);
    const Seg s = scatterSeg(len, per_rank, esize);
    pushPhase<T>(in + off, s, scale);
    barrier(kAll, 0);
    if (t.M == 1) {
      localReducePhase<T>(s, op, out + off);
    } else {
      localReducePhase<T>(s, op, nullptr);
      barrier(kRail, 1);
      serverReducePhase<T>(s, op, out + off);
    }
    finishOp();
  }
}

template <typename T>
void CpuEngine::allGatherT(const T* in, T* out, int64_t per_rank) {
  const int W = topo_.world;
  const int esize = (int)sizeof(T);
  const int64_t V = kVecBytes / esize;
  int64_t max_len = roundDown(plan_.max_slice_bytes / esize / W, V);
  if (max_len < V) max_len = V;
  for (int64_t off = 0; off < per_rank; off += max_len) {
    const int64_t len = std::min(max_len, per_rank - off);
    const Seg s = scatterSeg(len, per_rank, esize);
    diffusePhase<T>(in + off, s);
    barrier(kAll, 0);
    barrier(kGroup, 3);
    gatherPhase<T>(out + off, s);
    finishOp();
  }
}

#define FR_HOST_DISPATCH(dt, CALL)                                          \
  switch (dt) {                                                             \
    case DType::U8: { using T = uint8_t; CALL; break; }                     \
    case DType::I8: { using T = int8_t; CALL; break; }                      \
    case DType::I32: { using T = int32_t; CALL; break; }                    \
    case DType::I64: { using T = int64_t; CALL; break; }                    \
    case DType::F16: { using T = c10::Half; CALL; break; }                  \
    case DType::BF16: { using T = c10::BFloat16; CALL; break; }             \
    case DType::F32: { using T = float; CALL; break; }                      \
    case DType::F64: { using T = double; CALL; break; }                     \
    default: FR_CHECK(false, "unsupported dtype");                          \
  }

void CpuEngine::allReduce(const void* in, void* out, int64_t numel, DType dt, RedOp op,
                          float scale) {
  ++stats_.collectives;
  if (numel == 0) return;
  FR_HOST_DISPATCH(dt, allReduceT<T>(static_cast<const T*>(in), static_cast<T*>(out), numel, op, scale));
}

void CpuEngine::reduceScatter(const void* in, void* out, int64_t per_rank, DType dt, RedOp op,
                              float scale) {
  ++stats_.collectives;
  if (per_rank == 0) return;
  FR_HOST_DISPATCH(dt, reduceScatterT<T>(static_cast<const T*>(in), static_cast<T*>(out), per_rank, op, scale));
}

void CpuEngine::allGather(const void* in, void* out, int64_t per_rank, DType dt) {
  ++stats_.collectives;
  if (per_rank == 0) return;
  FR_HOST_DISPATCH(dt, allGatherT<T>(static_cast<const T*>(in), static_cast<T*>(out), per_rank));
}

}  // namespace fairring
