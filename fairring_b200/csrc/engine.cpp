#include "engine.h"

#include <algorithm>
#include <cstring>
#include <sstream>

#include <nvtx3/nvToolsExt.h>

#include <cstdlib>

#include "check.h"
#include "kernels/local_kernels.h"

namespace fairring {

const char* algoName(Algo a) {
  switch (a) {
    case Algo::AUTO: return "auto";
    case Algo::ONESHOT: return "oneshot";
    case Algo::TWOSHOT: return "twoshot";
    case Algo::HIER: return "hier";
    case Algo::NVLS: return "nvls";
    case Algo::NVLS_ONESHOT: return "nvls_oneshot";
    case Algo::PIPE: return "pipe";
    case Algo::LL: return "ll";
    case Algo::LL2: return "ll2";
  }
  return "?";
}

Algo parseAlgo(const std::string& s) {
  for (Algo a : {Algo::AUTO, Algo::ONESHOT, Algo::TWOSHOT, Algo::HIER, Algo::NVLS, Algo::NVLS_ONESHOT,
                 Algo::PIPE, Algo::LL, Algo::LL2})
    if (s == algoName(a)) return a;
  FR_CHECK(false, "unknown FAIRRING_ALGO '", s,
           "' (auto, oneshot, twoshot, hier, nvls, nvls_oneshot, pipe, ll, ll2)");
  return Algo::AUTO;
}

namespace {
constexpr size_t kFlagPadBytes = (size_t)kMaxRanks * kMaxBlocks * sizeof(uint32_t);
constexpr size_t kTraceLen = 256;
}  // namespace

Engine::Engine(std::shared_ptr<KvStore> store, const Topo& topo, int device,
               const EngineConfig& cfg)
    : store_(std::move(store)), topo_(topo), device_(device), cfg_(cfg) {
  FR_CHECK(topo_.world <= kMaxRanks, "the peer-memory path serves at most ", kMaxRanks,
           " ranks, got ", topo_.world);
  FR_CHECK(cfg_.blocks >= 1 && cfg_.blocks <= kMaxBlocks, "FAIRRING_BLOCKS must be in 1..",
           kMaxBlocks);
  if (const char* e = std::getenv("FAIRRING_NVTX")) nvtx_ = e[0] == '1';
  FR_CUDA(cudaSetDevice(device_));
  // Kernels of different channels wait on their peers while resident.  If more
  // blocks were in flight than the GPU can hold at once, two GPUs could each
  // keep resident exactly the blocks whose partners are still queued on the
  // other GPU, and nobody would move.  So: the blocks of all channels together
  // never exceed the SM count.  Every kernel here occupies a whole SM per block
  // (__launch_bounds__(512, 1), 128 registers per thread; the pipelined kernel
  // also takes most of the shared memory).
  int sms = 0;
  FR_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device_));
  sm_count_ = sms;
  const bool want_pipe = cfg_.pipe != "off" && topo_.world > 1 && topo_.M == 1;
  if (cfg_.pipe_blocks < 1) cfg_.pipe_blocks = 1;
  if (cfg_.pipe_blocks > kMaxBlocks) cfg_.pipe_blocks = kMaxBlocks;
  // FAIRRING_SM_BUDGET further limits how many SMs the collectives may hold at
  // once, so that backward keeps most of the GPU while gradients are reduced.
  // The budget counts the staged kernels (`blocks` each).  A pipelined launch
  // may be wider, but only the first pipe_channels channels ever run one, and
  // large ordinary tensors are not what runs under backward.
  const int budget = std::max(cfg_.blocks, std::min(sms, cfg_.sm_budget));
  const int max_channels = std::max(1, budget / cfg_.blocks);
  if (cfg_.parallelism > max_channels) cfg_.parallelism = max_channels;
  // The flag-in-data areas come off the top of the budget (a quarter at most):
  // fewer channels first, then smaller messages.
  int64_t ll_total = 0;
  if (cfg_.ll_max_bytes > 0 && topo_.world > 1) {
    ll_channels_ = std::max(1, std::min(cfg_.ll_channels, cfg_.parallelism));
    auto halfFor = [&](int64_t one, int64_t two) {
      const int64_t a = (int64_t)kMaxRanks * roundUp(ceilDiv(one, 8), 64) * 16;
      const int64_t b = roundUp(4 * two + 32 * kMaxRanks * 64, 4096);
      return std::max(a, two > 0 ? b : 0);
    };
    ll_half_bytes_ = halfFor(cfg_.ll_max_bytes, cfg_.ll2_max_bytes);
    const int64_t cap = cfg_.total_memory / 4;
    while (ll_channels_ > 1 && 2 * ll_half_bytes_ * ll_channels_ > cap) --ll_channels_;
    while (2 * ll_half_bytes_ > cap && (cfg_.ll2_max_bytes > 0 || cfg_.ll_max_bytes > 4096)) {
      if (cfg_.ll2_max_bytes > cfg_.ll_max_bytes)
        cfg_.ll2_max_bytes /= 2;
      else if (cfg_.ll2_max_bytes > 0)
        cfg_.ll2_max_bytes = 0;
      else
        cfg_.ll_max_bytes /= 2;
      ll_half_bytes_ = halfFor(cfg_.ll_max_bytes, cfg_.ll2_max_bytes);
    }
    if (2 * ll_half_bytes_ > cap) {
      ll_channels_ = 0;
      ll_half_bytes_ = 0;
    }
    ll_total = 2 * ll_half_bytes_ * ll_channels_;
  }
  const int64_t rest = cfg_.total_memory - ll_total;
  // With the pipelined kernel the rest is cut in three: two thirds for the
  // staging slots of the channels, one third for its rings.
  plan_ = planMemory(want_pipe ? rest / 3 * 2 : rest, cfg_.slice_bytes, cfg_.parallelism,
                     topo_.world, cfg_.min_half_bytes);

  alloc_.reset(new SymmAllocator(store_, topo_.rank, topo_.world, device_, cfg_.transport,
                                 cfg_.nvls, cfg_.bootstrap_timeout));
  flags_bytes_ = (size_t)roundUp((int64_t)(kFlagPadBytes * plan_.channels), 64 << 10);
  region_ = alloc_->allocate(flags_bytes_ + (size_t)plan_.slot_bytes * plan_.channels,
                             /*want_multicast=*/true);

  if (want_pipe) {
    pipe_channels_ = std::max(1, std::min<int>(cfg_.pipe_channels, plan_.channels));
    // Residency: every kernel that can be in flight at once must fit on the GPU
    // (a channel runs one kernel at a time: the wider of the two on a pipe channel).
    auto resident = [&] {
      return pipe_channels_ * std::max(cfg_.blocks, cfg_.pipe_blocks) +
             (plan_.channels - pipe_channels_) * cfg_.blocks;
    };
    while (resident() > sms && pipe_channels_ > 1) --pipe_channels_;
    while (resident() > sms && cfg_.pipe_blocks > cfg_.blocks) --cfg_.pipe_blocks;
    if (cfg_.pipe_slots < 2) cfg_.pipe_slots = 2;
    const int64_t ring_total = rest / 3;
    pipe_slot_bytes_ = roundDown(ring_total / pipe_channels_ / cfg_.pipe_slots, 4096);
    if (pipe_slot_bytes_ > (32ll << 20)) pipe_slot_bytes_ = 32ll << 20;
    if (pipe_slot_bytes_ < 4096) {
      pipe_channels_ = 0;  // no room for rings: ordinary tensors take the staged kernels
    } else {
      pipe_flags_bytes_ = (size_t)roundUp((int64_t)(kPipeFlagBytes * pipe_channels_), 64 << 10);
      pipe_region_ = alloc_->allocate(
          pipe_flags_bytes_ + (size_t)pipe_slot_bytes_ * cfg_.pipe_slots * pipe_channels_,
          /*want_multicast=*/true);
      FR_CUDA(cudaMalloc(&pipe_seq_dev_, sizeof(uint32_t) * kMaxBlocks * pipe_channels_));
      FR_CUDA(cudaMemset(pipe_seq_dev_, 0, sizeof(uint32_t) * kMaxBlocks * pipe_channels_));
    }
  }

  if (ll_channels_ > plan_.channels) ll_channels_ = plan_.channels;
  if (ll_channels_ > 0)
    ll_region_ = alloc_->allocate((size_t)(2 * ll_half_bytes_) * ll_channels_, /*want_multicast=*/false);

  FR_CUDA(cudaMalloc(&seq_dev_, sizeof(uint32_t) * kMaxBlocks * plan_.channels));
  FR_CUDA(cudaMemset(seq_dev_, 0, sizeof(uint32_t) * kMaxBlocks * plan_.channels));
  const size_t status_words = (size_t)plan_.channels * kStatusWords + 16;
  FR_CUDA(cudaHostAlloc((void**)&status_host_, status_words * sizeof(uint32_t),
                        cudaHostAllocMapped));
  std::memset(status_host_, 0, status_words * sizeof(uint32_t));
  FR_CUDA(cudaHostGetDevicePointer((void**)&status_dev_, status_host_, 0));

  int lo = 0, hi = 0;
  FR_CUDA(cudaDeviceGetStreamPriorityRange(&lo, &hi));
  channels_.resize(plan_.channels);
  for (int c = 0; c < plan_.channels; ++c) {
    Channel& ch = channels_[c];
    FR_CUDA(cudaStreamCreateWithPriority(&ch.stream, cudaStreamNonBlocking,
                                         cfg_.high_priority ? hi : lo));
    FR_CUDA(cudaEventCreateWithFlags(&ch.done, cudaEventDisableTiming));
    FR_CUDA(cudaEventCreateWithFlags(&ch.last_done, cudaEventDisableTiming));
    ch.last_stream = ch.stream;
    for (int r = 0; r < topo_.world; ++r) {
      char* base = static_cast<char*>(region_.ptrs[r]);
      ch.dev.flags[r] = reinterpret_cast<uint32_t*>(base + kFlagPadBytes * c);
      ch.dev.staging[r] = base + flags_bytes_ + (size_t)plan_.slot_bytes * c;
      ch.dev.ll[r] = c < ll_channels_ ? static_cast<char*>(ll_region_.ptrs[r]) +
                                            (size_t)(2 * ll_half_bytes_) * c
                                      : nullptr;
    }
    ch.dev.ll_half_bytes = (uint64_t)ll_half_bytes_;
    ch.dev.mc_staging = region_.mc_ptr
                            ? static_cast<char*>(region_.mc_ptr) + flags_bytes_ +
                                  (size_t)plan_.slot_bytes * c
                            : nullptr;
    ch.dev.seq = seq_dev_ + (size_t)kMaxBlocks * c;
    ch.dev.status = status_dev_ + (size_t)kStatusWords * c;
    ch.dev.abort_flag = status_dev_ + (size_t)kStatusWords * plan_.channels;
    ch.dev.half_bytes = (uint64_t)plan_.half_bytes;
    ch.dev.timeout_ns = cfg_.device_timeout_ns;
    ch.dev.topo = topo_;
  }
  // The kernels read the channel description from device memory.
  FR_CUDA(cudaMalloc(&channels_dev_, sizeof(ChannelDev) * plan_.channels));
  for (int c = 0; c < plan_.channels; ++c)
    FR_CUDA(cudaMemcpy(channels_dev_ + c, &channels_[c].dev, sizeof(ChannelDev),
                       cudaMemcpyHostToDevice));
  if (pipe_channels_ > 0) {
    std::vector<PipeChannelDev> pcs(pipe_channels_);
    const size_t ring_bytes = (size_t)pipe_slot_bytes_ * cfg_.pipe_slots;
    for (int c = 0; c < pipe_channels_; ++c) {
      PipeChannelDev& pc = pcs[c];
      std::memset(&pc, 0, sizeof(pc));
      for (int r = 0; r < topo_.world; ++r) {
        char* base = static_cast<char*>(pipe_region_.ptrs[r]);
        pc.flags[r] = reinterpret_cast<uint32_t*>(base + kPipeFlagBytes * c);
        pc.ring[r] = base + pipe_flags_bytes_ + ring_bytes * c;
      }
      pc.ring_mc = pipe_region_.mc_ptr
                       ? static_cast<char*>(pipe_region_.mc_ptr) + pipe_flags_bytes_ + ring_bytes * c
                       : nullptr;
      pc.seq = pipe_seq_dev_ + (size_t)kMaxBlocks * c;
      pc.status = channels_[c].dev.status;
      pc.abort_flag = channels_[c].dev.abort_flag;
      pc.slot_bytes = (uint64_t)pipe_slot_bytes_;
      pc.timeout_ns = cfg_.device_timeout_ns;
      pc.slots = cfg_.pipe_slots;
      pc.world = topo_.world;
      pc.rank = topo_.rank;
    }
    FR_CUDA(cudaMalloc(&pipe_channels_dev_, sizeof(PipeChannelDev) * pipe_channels_));
    FR_CUDA(cudaMemcpy(pipe_channels_dev_, pcs.data(), sizeof(PipeChannelDev) * pipe_channels_,
                       cudaMemcpyHostToDevice));
  }
  FR_CUDA(cudaDeviceSynchronize());
  store_->barrier("engine/ready", topo_.world, cfg_.bootstrap_timeout);

  if (cfg_.command_thread) {
    worker_ = std::thread([this] {
      cudaSetDevice(device_);
      for (;;) {
        auto fn = queue_.pop();
        if (!fn) break;
        fn();
      }
    });
  }
}

Engine::~Engine() {
  if (worker_.joinable()) {
    queue_.push(std::function<void()>());
    worker_.join();
  }
  cudaSetDevice(device_);
  cudaDeviceSynchronize();
  try {
    for (auto& kv : user_regions_) alloc_->release(kv.second.reg);
    alloc_->release(pipe_region_);
    alloc_->release(ll_region_);
    alloc_->release(region_);
  } catch (const std::exception&) {
  }
  for (auto& ch : channels_) {
    // The side streams are deliberately never destroyed.  Tensors that were
    // used on them carry a record of that in the caching allocator, which will
    // record an event on the stream when such a tensor is finally freed --
    // possibly long after this engine is gone.  A destroyed stream there means
    // an exception from inside a destructor.  (The reference leaks its merge
    // streams for the same reason, fairring/machine.cc:162-175.)
    if (ch.done) cudaEventDestroy(ch.done);
    if (ch.last_done) cudaEventDestroy(ch.last_done);
  }
  for (auto& e : free_events_)
    if (e) cudaEventDestroy(e);
  if (pipe_seq_dev_) cudaFree(pipe_seq_dev_);
  if (pipe_channels_dev_) cudaFree(pipe_channels_dev_);
  if (seq_dev_) cudaFree(seq_dev_);
  if (channels_dev_) cudaFree(channels_dev_);
  if (status_host_) cudaFreeHost(status_host_);
}

cudaEvent_t Engine::begin(cudaStream_t caller) {
  cudaEvent_t e = nullptr;
  {
    std::lock_guard<std::mutex> lk(events_mu_);
    if (!free_events_.empty()) {
      e = free_events_.back();
      free_events_.pop_back();
    }
  }
  if (e == nullptr) FR_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  FR_CUDA(cudaEventRecord(e, caller));
  return e;
}

void Engine::releaseEvent(cudaEvent_t e) {
  if (e == nullptr) return;
  std::lock_guard<std::mutex> lk(events_mu_);
  free_events_.push_back(e);
}

void Engine::submit(std::function<void()> fn) {
  if (cfg_.command_thread)
    queue_.push(std::move(fn));
  else
    fn();
}

uint32_t Engine::health(std::string* what) const {
  for (int c = 0; c < plan_.channels; ++c) {
    const volatile uint32_t* s = status_host_ + (size_t)kStatusWords * c;
    if (s[0] != kStatusOk) {
      if (what) {
        std::ostringstream os;
        os << "channel " << c << ": " << (s[0] == kStatusTimeout ? "timed out" : "aborted")
           << " waiting for rank " << s[2];
        if (s[1] >= 100)
          os << " in the pipelined kernel (wait " << s[1] << ") at chunk " << s[3];
        else
          os << " at barrier " << s[1] << " of collective " << s[3];
        *what = os.str();
      }
      return s[0];
    }
  }
  return kStatusOk;
}

void Engine::checkHealth() {
  std::string what;
  if (poisoned_ || health(&what) != kStatusOk) {
    poisoned_ = true;
    if (what.empty()) what = "an earlier collective failed";
    FR_CHECK(false, "the fairring engine is in a failed state (", what,
             "); call reset() on every rank to recover");
  }
}

void Engine::abort() {
  status_host_[(size_t)kStatusWords * plan_.channels] = 1;
  poisoned_ = true;
}

void Engine::reset() {
  std::lock_guard<std::mutex> lk(mu_);
  FR_CUDA(cudaSetDevice(device_));
  FR_CUDA(cudaDeviceSynchronize());
  const std::string pfx = "engine/reset" + std::to_string(reset_count_++);
  store_->barrier(pfx + "/quiet", topo_.world, cfg_.bootstrap_timeout);
  FR_CUDA(cudaMemset(region_.ptrs[topo_.rank], 0, flags_bytes_));
  FR_CUDA(cudaMemset(seq_dev_, 0, sizeof(uint32_t) * kMaxBlocks * plan_.channels));
  if (pipe_channels_ > 0) {
    FR_CUDA(cudaMemset(pipe_region_.ptrs[topo_.rank], 0, pipe_flags_bytes_));
    FR_CUDA(cudaMemset(pipe_seq_dev_, 0, sizeof(uint32_t) * kMaxBlocks * pipe_channels_));
  }
  FR_CUDA(cudaDeviceSynchronize());
  std::memset(status_host_, 0, ((size_t)plan_.channels * kStatusWords + 16) * sizeof(uint32_t));
  poisoned_ = false;
  // Ranks may have issued different numbers of collectives before the failure:
  // start the round-robin over channels from the same place everywhere.
  next_channel_ = 0;
  next_pipe_ = 0;
  next_ll_ = 0;
  // (The flag-in-data areas need no clearing: sequence numbers restart at 0, and
  // a word only counts when it carries the number of the collective that reads
  // it; clear them anyway so that an old word cannot match a restarted count.)
  if (ll_channels_ > 0) {
    FR_CUDA(cudaMemset(ll_region_.ptrs[topo_.rank], 0, (size_t)(2 * ll_half_bytes_) * ll_channels_));
    FR_CUDA(cudaDeviceSynchronize());
  }
  store_->barrier(pfx + "/clean", topo_.world, cfg_.bootstrap_timeout);
}

void* Engine::allocSymmetric(size_t bytes) {
  std::lock_guard<std::mutex> lk(mu_);
  FR_CUDA(cudaSetDevice(device_));
  releaseFreedLocked();  // every rank is here: a good moment to let go of dead regions
  UserRegion u;
  u.reg = alloc_->allocate(bytes, /*want_multicast=*/true);
  u.id = next_region_id_++;
  void* p = u.reg.ptrs[topo_.rank];
  stats_.symmetric_regions += 1;
  stats_.symmetric_bytes += u.reg.bytes;
  user_regions_[reinterpret_cast<uintptr_t>(p)] = std::move(u);
  return p;
}

void Engine::freeSymmetric(void* p) {
  std::lock_guard<std::mutex> lk(mu_);
  auto it = user_regions_.find(reinterpret_cast<uintptr_t>(p));
  if (it == user_regions_.end() || it->second.freed) return;
  it->second.freed = true;
  stats_.symmetric_pending += 1;
}

// Unmapping is collective (peers hold mappings of this rank's memory, and the
// allocator numbers its store keys), while a tensor dies whenever its last
// reference goes.  So a dead region only waits here, and is released once every
// rank reports it dead: each rank publishes the ids it has freed, all read all
// lists, and the intersection is released in id order.
int Engine::releaseFreedSymmetric() {
  std::lock_guard<std::mutex> lk(mu_);
  return releaseFreedLocked();
}

int Engine::releaseFreedLocked() {
  if (topo_.world == 1 && stats_.symmetric_pending == 0) return 0;
  FR_CUDA(cudaSetDevice(device_));
  const std::string pfx = "engine/symfree" + std::to_string(release_round_++);
  std::string mine = "L";  // never an empty value
  for (auto& kv : user_regions_)
    if (kv.second.freed) mine += std::to_string(kv.second.id) + ",";
  store_->setString(pfx + "/" + std::to_string(topo_.rank), mine);
  std::map<uint64_t, int> votes;
  for (int r = 0; r < topo_.world; ++r) {
    const std::string theirs = store_->getString(pfx + "/" + std::to_string(r));
    size_t pos = 1;
    while (pos < theirs.size()) {
      const size_t comma = theirs.find(',', pos);
      if (comma == std::string::npos) break;
      ++votes[std::stoull(theirs.substr(pos, comma - pos))];
      pos = comma + 1;
    }
  }
  int released = 0;
  for (auto& v : votes) {  // ascending id: the same order on every rank
    if (v.second != topo_.world) continue;
    for (auto it = user_regions_.begin(); it != user_regions_.end(); ++it) {
      if (it->second.id != v.first) continue;
      for (auto& ch : channels_) FR_CUDA(cudaStreamSynchronize(ch.stream));
      stats_.symmetric_regions -= 1;
      stats_.symmetric_bytes -= it->second.reg.bytes;
      stats_.symmetric_pending -= 1;
      alloc_->release(it->second.reg);
      user_regions_.erase(it);
      ++released;
      break;
    }
  }
  return released;
}

bool Engine::findSymmetric(const void* p, size_t bytes, const SymmRegion** reg, size_t* off) const {
  const uintptr_t q = reinterpret_cast<uintptr_t>(p);
  auto it = user_regions_.upper_bound(q);
  if (it == user_regions_.begin()) return false;
  --it;
  if (it->second.freed || q + bytes > it->first + it->second.reg.bytes) return false;
  *reg = &it->second.reg;
  *off = (size_t)(q - it->first);
  return true;
}

// Whether an all-reduce can run in place on symmetric memory.
bool Engine::directEligible(const CollectiveDesc& d) const {
  if (cfg_.direct == "off" || d.kind != CollKind::ALLREDUCE || topo_.M != 1 || topo_.world < 2)
    return false;
  if (d.in != d.out || d.io != d.wire) return false;
  const size_t bytes = (size_t)d.numel * dtypeSize(d.io);
  if ((reinterpret_cast<uintptr_t>(d.out) & 15u) != 0 || bytes % kVecBytes != 0) return false;
  if ((int64_t)bytes <= cfg_.oneshot_max_bytes) return false;  // one barrier beats two
  const SymmRegion* reg = nullptr;
  size_t off = 0;
  if (!findSymmetric(d.out, bytes, &reg, &off)) return false;
  if (cfg_.direct == "nvls" && !(reg->mc_ptr != nullptr && nvlsSupported(d.wire, d.op))) return false;
  return true;
}

// All-reduce in place on symmetric memory.  Returns false if the tensor does
// not qualify (then the staged path is taken).
bool Engine::runDirect(const CollectiveDesc& d, const std::function<Channel&(int)>& take) {
  if (!directEligible(d)) return false;
  const int es = dtypeSize(d.io);
  const size_t bytes = (size_t)d.numel * es;
  const SymmRegion* reg = nullptr;
  size_t off = 0;
  if (!findSymmetric(d.out, bytes, &reg, &off)) return false;
  // Two ranks gain nothing from the switch (measured: peer loads 590 GB/s, NVLS
  // 375 GB/s at 128 MiB); from three ranks on the in-switch reduction wins.
  bool nvls = reg->mc_ptr != nullptr && nvlsSupported(d.wire, d.op) && cfg_.direct != "p2p";
  if (cfg_.direct == "auto" && topo_.world <= 2) nvls = false;
  if (cfg_.direct == "nvls" && !nvls) return false;
  const int W = topo_.world;
  const int64_t V = kVecBytes / es;
  // Two kernels in flight already saturate the links (measured on 8 GPUs at
  // 128 MiB: 757 GB/s with 2 channels, 743 with 4, 673 with 8).
  int64_t nslices = (int64_t)bytes / cfg_.direct_min_slice_bytes;
  if (nslices > (int64_t)channels_.size()) nslices = (int64_t)channels_.size();
  // ... while the peer-load variant keeps gaining up to 64 blocks (2 GPUs at
  // 128 MiB: 456 GB/s with 2 channels of 16 blocks, 582 with 4).
  if (nvls && nslices > cfg_.direct_max_slices) nslices = cfg_.direct_max_slices;
  if (nslices < 1) nslices = 1;
  const int64_t slice_elems = roundUp(ceilDiv(d.numel, nslices), V * W);
  for (int64_t start = 0; start < d.numel; start += slice_elems) {
    const int64_t n = std::min(slice_elems, d.numel - start);
    OpArgs a{};
    a.seg = allreduceSeg(n, es, W);
    a.scale = d.scale;
    a.op = (int32_t)d.op;
    a.io_dtype = (int32_t)d.io;
    a.wire_dtype = (int32_t)d.wire;
    a.flags = kAdvanceSeq;
    a.unroll = cfg_.direct_unroll;
    a.full_blocks = cfg_.blocks;
    const size_t o = off + (size_t)start * es;
    for (int r = 0; r < W; ++r) a.peer[r] = static_cast<char*>(reg->ptrs[r]) + o;
    a.mc = nvls ? static_cast<char*>(reg->mc_ptr) + o : nullptr;
    a.in[0] = a.out[0] = a.peer[topo_.rank];
    const int nb = nvls && cfg_.direct_blocks > 0 ? std::min(cfg_.direct_blocks, cfg_.blocks) : cfg_.blocks;
    launch(take(-1), nvls ? KernelId::NVLS_DIRECT : KernelId::P2P_DIRECT, a, nb);
    ++stats_.slices;
  }
  stats_.wire_bytes += bytes;
  return true;
}

// Ordinary tensor: ONE launch of the pipelined kernel whatever the size.  The
// message is not sliced: the kernel walks its chunks through the channel's
// ring.  Consecutive messages alternate between the rings so that two launches
// can overlap.
bool Engine::runPipe(const CollectiveDesc& d, const std::function<Channel&(int)>& take) {
  if (pipe_channels_ == 0 || d.kind != CollKind::ALLREDUCE || d.io != d.wire) return false;
  const bool forced = cfg_.algo == Algo::PIPE;
  if (!forced && cfg_.algo != Algo::AUTO) return false;
  const int es = dtypeSize(d.io);
  const int64_t bytes = d.numel * es;
  if (bytes <= 0) return false;
  if (!forced && bytes < cfg_.pipe_min_bytes) return false;
  // The threshold was measured with the configured chunk: without room for it
  // in the ring the staged kernels are the better choice.
  if (!forced && cfg_.pipe_chunk_bytes > pipe_slot_bytes_) return false;
  // Every chunk costs a fixed 13-15 us of publication fences (8 GPUs): with
  // slots under 4 MiB the kernel cannot amortise them.
  if (!forced && pipe_slot_bytes_ < (4ll << 20)) return false;
  if (((reinterpret_cast<uintptr_t>(d.in) | reinterpret_cast<uintptr_t>(d.out)) & 15u) != 0)
    return false;  // bulk copies need 16-byte aligned addresses
  const int W = topo_.world;
  bool nvls = pipe_region_.mc_ptr != nullptr && nvlsSupported(d.wire, d.op) && cfg_.direct != "p2p";
  if (cfg_.direct == "auto" && W <= 2) nvls = false;
  // Small messages: fewer blocks, so that a block's piece of a sub-chunk stays
  // worth a bulk copy (8 KiB or more).
  int blocks = (int)std::min<int64_t>(cfg_.pipe_blocks, std::max<int64_t>(1, bytes / ((int64_t)W * 8192)));
  // Chunk, when none is configured: 16 MiB (or the slot, if smaller) for the
  // large messages that come here by themselves; when the kernel is forced on a
  // small message, the whole message up to 1 MiB, else an eighth of it.
  const int64_t quantum = (int64_t)kVecBytes * W * blocks;
  int64_t chunk = cfg_.pipe_chunk_bytes;
  if (chunk <= 0) {
    if (!forced)
      chunk = 16ll << 20;
    else
      chunk = bytes <= (1 << 20) ? bytes : std::max<int64_t>(512 << 10, bytes / 8);
  }
  chunk = roundUp(chunk, quantum);
  if (chunk > pipe_slot_bytes_) chunk = roundDown(pipe_slot_bytes_, kVecBytes);
  const int pc = (int)(next_pipe_++ % (uint64_t)pipe_channels_);
  Channel& ch = take(pc);
  PipeArgs a{};
  a.in[0] = d.in;
  a.out[0] = d.out;
  a.nbytes = bytes;
  a.chunk_bytes = chunk;
  a.scale = d.scale;
  a.op = (int32_t)d.op;
  a.dtype = (int32_t)d.io;
  a.nvls = nvls ? 1 : 0;
  a.stage_bytes = cfg_.pipe_stage_bytes;
  a.stages = cfg_.pipe_stages;
  cudaError_t e = launchPipeAllreduce(pipe_channels_dev_ + pc, a, blocks, ch.stream);
  FR_CHECK(e == cudaSuccess, "launch of pipe_allreduce failed: ", cudaGetErrorString(e));
  ++stats_.launches[(size_t)KernelId::PIPE];
  if (cur_.launches == 0) cur_.first_kernel = (int32_t)KernelId::PIPE;
  ++cur_.launches;
  ++stats_.slices;
  stats_.wire_bytes += (uint64_t)bytes;
  return true;
}

EngineStats Engine::stats() const { return stats_; }

std::vector<TraceEntry> Engine::trace() const {
  std::vector<TraceEntry> out;
  const uint64_t n = stats_.collectives;
  const uint64_t first = n > kTraceLen ? n - kTraceLen : 0;
  for (uint64_t i = first; i < n && i - first < trace_.size(); ++i) out.push_back(trace_[i % kTraceLen]);
  return out;
}

std::vector<cudaStream_t> Engine::streams() const {
  std::vector<cudaStream_t> v;
  for (auto& ch : channels_) v.push_back(ch.stream);
  return v;
}

std::string Engine::describe() const {
  std::ostringstream os;
  os << "ll=" << (ll_channels_ > 0 ? cfg_.ll_max_bytes : 0) << "B+" << (ll_channels_ > 0 ? cfg_.ll2_max_bytes : 0)
     << "B/" << ll_channels_ << "ch "
     << "world=" << topo_.world << " grouping=" << topo_.M << "x" << topo_.D
     << (topo_.favorable ? " (device-major ranks)" : " (machine-major ranks)")
     << " transport=" << alloc_->describe() << " nvls=" << (nvlsAvailable() ? "yes" : "no")
     << " channels=" << plan_.channels << " half_slot=" << plan_.half_bytes
     << "B max_slice=" << plan_.max_slice_bytes << "B blocks=" << cfg_.blocks
     << " algo=" << algoName(cfg_.algo) << " pipe=";
  if (pipe_channels_ > 0)
    os << pipe_channels_ << "x" << cfg_.pipe_slots << "x" << pipe_slot_bytes_ << "B/" << cfg_.pipe_blocks
       << "blocks";
  else
    os << "no";
  return os.str();
}

Algo Engine::chooseAllreduce(int64_t wire_bytes, DType wire, RedOp op) const {
  const int W = topo_.world;
  const int64_t qv = std::max<int64_t>(1, ceilDiv(ceilDiv(wire_bytes, kVecBytes), W));
  const bool oneshot_fits = (int64_t)W * W * qv * kVecBytes <= plan_.half_bytes;
  const bool nvls_ok = nvlsAvailable() && nvlsSupported(wire, op);
  Algo a = cfg_.algo;
  if (a == Algo::ONESHOT && !oneshot_fits) a = Algo::AUTO;
  if ((a == Algo::NVLS || a == Algo::NVLS_ONESHOT) && !nvls_ok) a = Algo::AUTO;
  if (a == Algo::PIPE || a == Algo::LL || a == Algo::LL2) a = Algo::AUTO;  // did not qualify for that kernel
  if (a == Algo::TWOSHOT && topo_.M > 1) a = Algo::HIER;
  if (a != Algo::AUTO) return a;
  if (wire_bytes <= cfg_.oneshot_max_bytes && oneshot_fits) return Algo::ONESHOT;
  if (topo_.M > 1) return Algo::HIER;
  if (nvls_ok) {
    if (wire_bytes <= cfg_.nvls_oneshot_max_bytes) return Algo::NVLS_ONESHOT;
    if (wire_bytes >= cfg_.nvls_min_bytes) return Algo::NVLS;
  }
  return Algo::TWOSHOT;
}

int Engine::llKind(const CollectiveDesc& d) const {
  if (ll_channels_ == 0 || d.kind != CollKind::ALLREDUCE || d.io != d.wire || d.numel <= 0) return 0;
  const int64_t bytes = d.numel * dtypeSize(d.wire);
  const bool any = cfg_.algo == Algo::AUTO;
  if ((any || cfg_.algo == Algo::LL) && bytes <= cfg_.ll_max_bytes) return 1;
  // Past the one-shot sizes a tensor in symmetric memory is reduced in place
  // (8 GPUs, 1 MiB: 27 us in place, 37 us through the flag-in-data area).
  if (any && bytes > cfg_.ll_max_bytes && directEligible(d)) return 0;
  if (any || cfg_.algo == Algo::LL2) {
    const int64_t cu = ceilDiv(ceilDiv(bytes, 8), topo_.world);
    if (bytes <= cfg_.ll2_max_bytes && 2 * (int64_t)topo_.world * cu * 16 <= ll_half_bytes_) return 2;
  }
  return 0;
}

bool Engine::fitsInline(const CollectiveDesc& d) const {
  std::lock_guard<std::mutex> lk(mu_);
  return cfg_.inline_small && !cfg_.command_thread && llKind(d) != 0;
}

void Engine::launchLL(Channel& ch, const CollectiveDesc& d, cudaStream_t stream) {
  OpArgs a{};
  a.in[0] = d.in;
  a.out[0] = d.out;
  a.seg = allreduceSeg(d.numel, dtypeSize(d.wire), topo_.world);
  a.scale = d.scale;
  a.op = (int32_t)d.op;
  a.io_dtype = a.wire_dtype = (int32_t)d.io;
  a.flags = kAdvanceSeq;
  // Always the channel's full grid: every block keeps its own count of the
  // channel's collectives, so every launch on a channel must run every block.
  const KernelId id = llKind(d) == 2 ? KernelId::LL_TWOSHOT : KernelId::LL_ONESHOT;
  cudaError_t e = launchCollective(id, channels_dev_ + (&ch - channels_.data()), a, cfg_.blocks, stream);
  FR_CHECK(e == cudaSuccess, "launch of ", kernelName(id), " failed: ", cudaGetErrorString(e));
  ++stats_.launches[(size_t)id];
  if (cur_.launches == 0) cur_.first_kernel = (int32_t)id;
  ++cur_.launches;
  ++stats_.slices;
  stats_.wire_bytes += (uint64_t)(d.numel * dtypeSize(d.wire));
}

// A channel's kernels must run one after the other (they share its sequence
// number, flags and areas).  On the channel's own stream that is stream order;
// a kernel launched on a caller's stream is tied in with two events.
void Engine::runInline(const CollectiveDesc& d, cudaStream_t caller) {
  std::lock_guard<std::mutex> lk(mu_);
  checkHealth();
  Channel& ch = channels_[(size_t)(next_ll_++ % (uint64_t)ll_channels_)];
  cur_ = TraceEntry{};
  cur_.seq = stats_.collectives;
  cur_.kind = (int32_t)d.kind;
  cur_.bytes = d.numel * dtypeSize(d.wire);
  if (ch.last_stream != caller) FR_CUDA(cudaStreamWaitEvent(caller, ch.last_done, 0));
  launchLL(ch, d, caller);
  FR_CUDA(cudaEventRecord(ch.last_done, caller));
  ch.last_stream = caller;
  cur_.slices = 1;
  cur_.channels = 0;
  if (trace_.size() < kTraceLen) trace_.resize(kTraceLen);
  trace_[cur_.seq % kTraceLen] = cur_;
  ++stats_.collectives;
  ++stats_.inline_collectives;
}

void Engine::setOption(const std::string& name, int64_t v) {
  std::lock_guard<std::mutex> lk(mu_);
  const int nch = (int)channels_.size();
  if (name == "blocks") {
    FR_CHECK(v >= 1 && v <= kMaxBlocks && v * nch <= sm_count_, "blocks x channels exceeds the SM count");
    // Blocks that did not run so far have a stale count of the channel's
    // collectives: give every block the count of block 0.
    FR_CUDA(cudaSetDevice(device_));
    FR_CUDA(cudaDeviceSynchronize());
    std::vector<uint32_t> seq((size_t)kMaxBlocks * nch);
    FR_CUDA(cudaMemcpy(seq.data(), seq_dev_, seq.size() * sizeof(uint32_t), cudaMemcpyDeviceToHost));
    for (int c = 0; c < nch; ++c)
      for (int b = 1; b < kMaxBlocks; ++b) seq[(size_t)c * kMaxBlocks + b] = seq[(size_t)c * kMaxBlocks];
    FR_CUDA(cudaMemcpy(seq_dev_, seq.data(), seq.size() * sizeof(uint32_t), cudaMemcpyHostToDevice));
    cfg_.blocks = (int32_t)v;
  } else if (name == "pipe_blocks") {
    FR_CHECK(v >= 1 && v <= kMaxBlocks && v * pipe_channels_ + (int64_t)cfg_.blocks * (nch - pipe_channels_) <= sm_count_,
             "pipe_blocks exceeds the SM count");
    cfg_.pipe_blocks = (int32_t)v;
  } else if (name == "pipe_chunk_bytes") {
    cfg_.pipe_chunk_bytes = v;
  } else if (name == "pipe_min_bytes") {
    cfg_.pipe_min_bytes = v;
  } else if (name == "pipe_stage_bytes") {
    FR_CHECK(v >= 16 && v % 16 == 0 && pipeSharedBytes((int)v, cfg_.pipe_stages) <= (200u << 10), "stage too large");
    cfg_.pipe_stage_bytes = (int32_t)v;
  } else if (name == "pipe_stages") {
    FR_CHECK(v >= 2 && v <= 8 && pipeSharedBytes(cfg_.pipe_stage_bytes, (int)v) <= (200u << 10), "too many stages");
    cfg_.pipe_stages = (int32_t)v;
  } else if (name == "direct_blocks") {
    FR_CHECK(v >= 0 && v <= kMaxBlocks, "direct_blocks out of range");
    cfg_.direct_blocks = (int32_t)v;
  } else if (name == "direct_unroll") {
    cfg_.direct_unroll = (int32_t)v;
  } else if (name == "direct_max_slices") {
    cfg_.direct_max_slices = (int32_t)std::max<int64_t>(1, v);
  } else if (name == "direct_min_slice_bytes") {
    cfg_.direct_min_slice_bytes = std::max<int64_t>(kVecBytes * topo_.world, v);
  } else if (name == "ll_max_bytes") {
    FR_CHECK(ll_channels_ == 0 || (int64_t)kMaxRanks * roundUp(ceilDiv(v, 8), 64) * 16 <= ll_half_bytes_,
             "ll_max_bytes beyond the areas allocated at start-up");
    cfg_.ll_max_bytes = v;
  } else if (name == "ll2_max_bytes") {
    cfg_.ll2_max_bytes = v;  // messages that do not fit the areas are refused per message
  } else if (name == "oneshot_max_bytes") {
    cfg_.oneshot_max_bytes = v;
  } else if (name == "nvls_oneshot_max_bytes") {
    cfg_.nvls_oneshot_max_bytes = v;
  } else if (name == "nvls_min_bytes") {
    cfg_.nvls_min_bytes = v;
  } else if (name == "inline_small") {
    cfg_.inline_small = v != 0;
  } else if (name == "algo") {
    FR_CHECK(v >= 0 && v <= (int64_t)Algo::LL2, "algo out of range");
    cfg_.algo = (Algo)v;
  } else {
    FR_CHECK(false, "unknown engine option '", name, "'");
  }
}

void Engine::launch(Channel& ch, KernelId id, const OpArgs& a, int blocks) {
  cudaError_t e = launchCollective(id, channels_dev_ + (&ch - channels_.data()), a,
                                   blocks > 0 ? blocks : cfg_.blocks, ch.stream);
  FR_CHECK(e == cudaSuccess, "launch of ", kernelName(id), " failed: ", cudaGetErrorString(e));
  ++stats_.launches[(size_t)id];
  if (cur_.launches == 0) cur_.first_kernel = (int32_t)id;
  ++cur_.launches;
}

void Engine::runAllreduceSlice(Channel& ch, const CollectiveDesc& d, const void* in, void* out,
                               int64_t n, Algo algo) {
  OpArgs a{};
  a.in[0] = in;
  a.out[0] = out;
  a.seg = allreduceSeg(n, dtypeSize(d.wire), topo_.world);
  a.scale = d.scale;
  a.op = (int32_t)d.op;
  a.io_dtype = (int32_t)d.io;
  a.wire_dtype = (int32_t)d.wire;
  switch (algo) {
    case Algo::ONESHOT:
      a.flags = kAdvanceSeq;
      launch(ch, KernelId::ONESHOT, a);
      break;
    case Algo::TWOSHOT:
      a.flags = kAdvanceSeq;
      launch(ch, KernelId::TWOSHOT, a);
      break;
    case Algo::NVLS:
      a.flags = kAdvanceSeq;
      launch(ch, KernelId::NVLS_TWOSHOT, a);
      break;
    case Algo::NVLS_ONESHOT:
      a.flags = kAdvanceSeq;
      launch(ch, KernelId::NVLS_ONESHOT, a);
      break;
    case Algo::HIER:
    default:
      a.flags = 0;
      launch(ch, KernelId::RS_INTRAGROUP, a);
      if (topo_.M > 1) launch(ch, KernelId::SHARD_SERVER_REDUCE, a);
      a.flags = kAdvanceSeq;
      launch(ch, KernelId::AG_INTRAGROUP, a);
      break;
  }
}

cudaStream_t Engine::run(const CollectiveDesc& d, cudaEvent_t after,
                         std::vector<cudaStream_t>* used_streams) {
  std::lock_guard<std::mutex> lk(mu_);
  checkHealth();
  FR_CHECK(comboSupported(d.io, d.wire), "no kernel for this (tensor dtype, wire dtype) pair");
  const int W = topo_.world;
  const int ies = dtypeSize(d.io), wes = dtypeSize(d.wire);
  const int64_t V = kVecBytes / wes;
  std::vector<int> used;
  // take(-1): the next channel in turn; take(c): channel c.
  std::function<Channel&(int)> take = [&](int want) -> Channel& {
    const int c = want >= 0 ? want : (int)(next_channel_++ % channels_.size());
    if (std::find(used.begin(), used.end(), c) == used.end()) {
      Channel& ch = channels_[c];
      FR_CUDA(cudaStreamWaitEvent(ch.stream, after, 0));
      if (ch.last_stream != ch.stream) {  // its last kernel ran inline on a caller's stream
        FR_CUDA(cudaStreamWaitEvent(ch.stream, ch.last_done, 0));
        ch.last_stream = ch.stream;
      }
      used.push_back(c);
    }
    return channels_[c];
  };
  const char* in = static_cast<const char*>(d.in);
  char* out = static_cast<char*>(d.out);
  const auto t_begin = std::chrono::steady_clock::now();
  const uint64_t slices_before = stats_.slices;
  cur_ = TraceEntry{};
  cur_.seq = stats_.collectives;
  cur_.kind = (int32_t)d.kind;
  cur_.bytes = d.numel * wes * (d.kind == CollKind::ALLREDUCE ? 1 : W);
  if (nvtx_) {
    static const char* kNames[] = {"fairring.all_reduce", "fairring.reduce_scatter",
                                   "fairring.all_gather"};
    nvtxRangePushA(kNames[(int)d.kind]);
  }
  struct Finish {
    Engine* e;
    std::vector<int>* used;
    std::chrono::steady_clock::time_point t0;
    uint64_t slices0;
    ~Finish() {
      e->cur_.slices = (int32_t)(e->stats_.slices - slices0);
      e->cur_.channels = (int32_t)used->size();
      e->cur_.host_us =
          std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count();
      if (e->trace_.size() < kTraceLen) e->trace_.resize(kTraceLen);
      e->trace_[e->cur_.seq % kTraceLen] = e->cur_;
      ++e->stats_.collectives;
      if (e->nvtx_) nvtxRangePop();
    }
  } finish{this, &used, t_begin, slices_before};

  if (llKind(d) != 0) {
    Channel& ch = take((int)(next_ll_++ % (uint64_t)ll_channels_));
    launchLL(ch, d, ch.stream);
  } else if (runDirect(d, take) || runPipe(d, take)) {
    // nothing else to do
  } else if (d.kind == CollKind::ALLREDUCE) {
    const int64_t bytes = d.numel * wes;
    const Algo whole = chooseAllreduce(bytes, d.wire, d.op);
    if (whole == Algo::ONESHOT ||
        (whole == Algo::NVLS_ONESHOT && bytes <= plan_.max_slice_bytes)) {
      runAllreduceSlice(take(-1), d, in, out, d.numel, whole);
      ++stats_.slices;
    } else {
      // A big message is spread over all channels (more blocks in flight),
      // down to direct_min_slice_bytes per slice.
      int64_t cap = std::max<int64_t>(cfg_.direct_min_slice_bytes,
                                      ceilDiv(bytes, (int64_t)channels_.size()));
      if (cap > plan_.max_slice_bytes) cap = plan_.max_slice_bytes;
      const SlicePlan sp = planSlices(d.numel, wes, W, cap);
      for (int64_t k = 0; k < sp.num_slices; ++k) {
        const int64_t off = k * sp.slice_elems;
        const int64_t n = std::min(sp.slice_elems, d.numel - off);
        // Slices of a big message use the variant chosen for the whole message:
        // the one-shot variants move W times the data and only pay off for
        // messages that are small as a whole.
        Algo a = sp.num_slices > 1 ? whole : chooseAllreduce(n * wes, d.wire, d.op);
        if (a == Algo::ONESHOT || a == Algo::NVLS_ONESHOT) a = chooseAllreduce(n * wes, d.wire, d.op);
        if (sp.num_slices > 1 && a == Algo::ONESHOT) a = topo_.M > 1 ? Algo::HIER : Algo::TWOSHOT;
        if (sp.num_slices > 1 && a == Algo::NVLS_ONESHOT) a = Algo::NVLS;
        runAllreduceSlice(take(-1), d, in + off * ies, out + off * ies, n, a);
        ++stats_.slices;
      }
    }
    stats_.wire_bytes += (uint64_t)bytes;
  } else {
    int64_t max_len = roundDown(plan_.max_slice_bytes / wes / W, V);
    if (max_len < V) max_len = V;
    for (int64_t off = 0; off < d.numel; off += max_len) {
      const int64_t len = std::min(max_len, d.numel - off);
      OpArgs a{};
      a.in[0] = in + off * ies;
      a.out[0] = out + off * ies;
      a.seg = scatterSeg(len, d.numel, wes);
      a.scale = d.scale;
      a.op = (int32_t)d.op;
      a.io_dtype = (int32_t)d.io;
      a.wire_dtype = (int32_t)d.wire;
      Channel& ch = take(-1);
      if (d.kind == CollKind::REDUCE_SCATTER) {
        if (topo_.M == 1) {
          a.flags = kToUser | kAdvanceSeq;
          launch(ch, KernelId::RS_INTRAGROUP, a);
        } else {
          a.flags = 0;
          launch(ch, KernelId::RS_INTRAGROUP, a);
          a.flags = kToUser | kAdvanceSeq;
          launch(ch, KernelId::SHARD_SERVER_REDUCE, a);
        }
      } else {
        a.flags = 0;
        launch(ch, KernelId::DIFFUSE, a);
        a.flags = kAdvanceSeq;
        launch(ch, KernelId::AG_INTRAGROUP, a);
      }
      ++stats_.slices;
    }
    stats_.wire_bytes += (uint64_t)d.numel * wes * W;
  }

  if (used.empty()) {  // zero elements: still give the caller a stream ordered after `after`
    Channel& ch = take(-1);
    return ch.stream;
  }
  if (cfg_.inline_small)
    for (int c : used)
      if (c < ll_channels_) {  // an inline collective may come next on this channel
        FR_CUDA(cudaEventRecord(channels_[c].last_done, channels_[c].stream));
        channels_[c].last_stream = channels_[c].stream;
      }
  if (used_streams)
    for (int c : used) used_streams->push_back(channels_[c].stream);
  Channel& join = channels_[used[0]];
  for (size_t i = 1; i < used.size(); ++i) {
    Channel& ch = channels_[used[i]];
    FR_CUDA(cudaEventRecord(ch.done, ch.stream));
    FR_CUDA(cudaStreamWaitEvent(join.stream, ch.done, 0));
  }
  return join.stream;
}

}  // namespace fairring
