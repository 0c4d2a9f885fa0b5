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
    case Algo::BOUNCE: return "bounce";
  }
  return "?";
}

Algo parseAlgo(const std::string& s) {
  for (Algo a : {Algo::AUTO, Algo::ONESHOT, Algo::TWOSHOT, Algo::HIER, Algo::NVLS, Algo::NVLS_ONESHOT,
                 Algo::BOUNCE})
    if (s == algoName(a)) return a;
  FR_CHECK(false, "unknown FAIRRING_ALGO '", s,
           "' (auto, oneshot, twoshot, hier, nvls, nvls_oneshot, bounce)");
  return Algo::AUTO;
}

void CommandQueue::push(std::function<void()> fn) {
  {
    std::lock_guard<std::mutex> lk(mu_);
    q_.push_back(std::move(fn));
  }
  cv_.notify_one();
}

std::function<void()> CommandQueue::pop() {
  std::unique_lock<std::mutex> lk(mu_);
  cv_.wait(lk, [&] { return !q_.empty(); });
  auto fn = std::move(q_.front());
  q_.pop_front();
  return fn;
}

namespace {
constexpr size_t kFlagPadBytes = (size_t)kMaxRanks * kMaxBlocks * sizeof(uint32_t);
constexpr int kEventPool = 2048;
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
  // other GPU, and nobody would move.  So: (channels x blocks) never exceeds
  // the SM count.  The kernels are built for two resident blocks per SM
  // (__launch_bounds__(512, 2)), which leaves the other half of every SM to
  // the compute kernels the collectives overlap with, or to a second engine.
  int sms = 0;
  FR_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device_));
  // FAIRRING_SM_BUDGET further limits how many SMs the collectives may hold at
  // once, so that backward keeps most of the GPU while gradients are reduced.
  const int budget = std::max(cfg_.blocks, std::min(sms, cfg_.sm_budget));
  const int max_channels = std::max(1, budget / cfg_.blocks);
  if (cfg_.parallelism > max_channels) cfg_.parallelism = max_channels;
  const bool want_bounce = cfg_.bounce != "off" && topo_.world > 1 && topo_.M == 1;
  // With bounce buffers the budget is cut in three equal parts per channel:
  // the two staging halves and the bounce buffer.
  plan_ = planMemory(want_bounce ? cfg_.total_memory / 3 * 2 : cfg_.total_memory, cfg_.slice_bytes,
                     cfg_.parallelism, topo_.world, cfg_.min_half_bytes);

  alloc_.reset(new SymmAllocator(store_, topo_.rank, topo_.world, device_, cfg_.transport,
                                 cfg_.nvls, cfg_.bootstrap_timeout));
  flags_bytes_ = (size_t)roundUp((int64_t)(kFlagPadBytes * plan_.channels), 64 << 10);
  region_ = alloc_->allocate(flags_bytes_ + (size_t)plan_.slot_bytes * plan_.channels,
                             /*want_multicast=*/true);

  if (want_bounce)
    bounce_ = alloc_->allocate((size_t)plan_.half_bytes * plan_.channels, /*want_multicast=*/true);

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
    for (int r = 0; r < topo_.world; ++r) {
      char* base = static_cast<char*>(region_.ptrs[r]);
      ch.dev.flags[r] = reinterpret_cast<uint32_t*>(base + kFlagPadBytes * c);
      ch.dev.staging[r] = base + flags_bytes_ + (size_t)plan_.slot_bytes * c;
    }
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
  events_.resize(kEventPool);
  for (auto& e : events_) FR_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
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
    for (auto& r : user_regions_) alloc_->release(r);
    alloc_->release(bounce_);
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
  }
  for (auto& e : events_)
    if (e) cudaEventDestroy(e);
  if (seq_dev_) cudaFree(seq_dev_);
  if (channels_dev_) cudaFree(channels_dev_);
  if (status_host_) cudaFreeHost(status_host_);
}

cudaEvent_t Engine::nextEvent() {
  cudaEvent_t e = events_[next_event_];
  next_event_ = (next_event_ + 1) % events_.size();
  return e;
}

cudaEvent_t Engine::begin(cudaStream_t caller) {
  std::lock_guard<std::mutex> lk(mu_);
  cudaEvent_t e = nextEvent();
  FR_CUDA(cudaEventRecord(e, caller));
  return e;
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
           << " waiting for rank " << s[2] << " at barrier " << s[1] << " of collective " << s[3];
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
  FR_CUDA(cudaDeviceSynchronize());
  std::memset(status_host_, 0, ((size_t)plan_.channels * kStatusWords + 16) * sizeof(uint32_t));
  poisoned_ = false;
  // Ranks may have issued different numbers of collectives before the failure:
  // start the round-robin over channels from the same place everywhere.
  next_channel_ = 0;
  store_->barrier(pfx + "/clean", topo_.world, cfg_.bootstrap_timeout);
}

void* Engine::allocSymmetric(size_t bytes) {
  std::lock_guard<std::mutex> lk(mu_);
  FR_CUDA(cudaSetDevice(device_));
  user_regions_.push_back(alloc_->allocate(bytes, /*want_multicast=*/true));
  return user_regions_.back().ptrs[topo_.rank];
}

bool Engine::findSymmetric(const void* p, size_t bytes, const SymmRegion** reg, size_t* off) const {
  const char* q = static_cast<const char*>(p);
  for (const auto& r : user_regions_) {
    const char* base = static_cast<const char*>(r.ptrs[topo_.rank]);
    if (q >= base && q + bytes <= base + r.bytes) {
      *reg = &r;
      *off = (size_t)(q - base);
      return true;
    }
  }
  return false;
}

// All-reduce in place on symmetric memory.  Returns false if the tensor does
// not qualify (then the staged path is taken).
bool Engine::runDirect(const CollectiveDesc& d, const std::function<Channel&()>& take) {
  if (cfg_.direct == "off" || d.kind != CollKind::ALLREDUCE || topo_.M != 1 || topo_.world < 2)
    return false;
  if (d.in != d.out || d.io != d.wire) return false;
  const int es = dtypeSize(d.io);
  const size_t bytes = (size_t)d.numel * es;
  if ((reinterpret_cast<uintptr_t>(d.out) & 15u) != 0 || bytes % kVecBytes != 0) return false;
  if ((int64_t)bytes <= cfg_.oneshot_max_bytes) return false;  // one barrier beats two
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
    const size_t o = off + (size_t)start * es;
    for (int r = 0; r < W; ++r) a.peer[r] = static_cast<char*>(reg->ptrs[r]) + o;
    a.mc = nvls ? static_cast<char*>(reg->mc_ptr) + o : nullptr;
    a.in[0] = a.out[0] = a.peer[topo_.rank];
    launch(take(), nvls ? KernelId::NVLS_DIRECT : KernelId::P2P_DIRECT, a);
    ++stats_.slices;
  }
  stats_.wire_bytes += bytes;
  return true;
}

// Ordinary tensor, big message: copy kernel in -> in-place kernel on the
// symmetric bounce buffer -> copy kernel out, all on the channel's stream.  The
// copy kernels do not wait on anybody, so they may be wide without touching
// the residency bound.  The
// kernel's closing barrier means every peer is done with this rank's buffer
// before the copy-out (and the next copy-in) touches it, so one buffer per
// channel is enough.
bool Engine::runBounce(const CollectiveDesc& d, const std::function<Channel&()>& take) {
  if (bounce_.ptrs.empty() || d.kind != CollKind::ALLREDUCE) return false;
  if (d.io != d.wire || d.scale != 1.0f) return false;  // the fused kernels do scale and cast
  const bool forced = cfg_.algo == Algo::BOUNCE;
  if (!forced && cfg_.algo != Algo::AUTO) return false;
  const int es = dtypeSize(d.io);
  const int64_t bytes = d.numel * es;
  if (!forced && bytes < cfg_.bounce_min_bytes) return false;
  if (bytes <= cfg_.oneshot_max_bytes) return false;
  bool nvls = bounce_.mc_ptr != nullptr && nvlsSupported(d.wire, d.op) && cfg_.direct != "p2p";
  if (cfg_.direct == "auto" && topo_.world <= 2) nvls = false;
  const int W = topo_.world;
  const int64_t V = kVecBytes / es;
  int64_t cap = std::max<int64_t>(cfg_.direct_min_slice_bytes,
                                  ceilDiv(bytes, (int64_t)channels_.size()));
  if (cap > plan_.half_bytes) cap = plan_.half_bytes;
  int64_t slice_elems = roundDown(cap / es, V * W);
  if (slice_elems < V * W) slice_elems = V * W;
  const char* in = static_cast<const char*>(d.in);
  char* out = static_cast<char*>(d.out);
  for (int64_t start = 0; start < d.numel; start += slice_elems) {
    const int64_t n = std::min(slice_elems, d.numel - start);
    Channel& ch = take();
    const size_t o = (size_t)(&ch - channels_.data()) * (size_t)plan_.half_bytes;
    char* mine = static_cast<char*>(bounce_.ptrs[topo_.rank]) + o;
    FR_CUDA(launchCopy(mine, in + start * es, (size_t)n * es, cfg_.bounce_copy_blocks, ch.stream));
    OpArgs a{};
    a.seg = allreduceSeg(n, es, W);
    a.scale = 1.0f;
    a.op = (int32_t)d.op;
    a.io_dtype = a.wire_dtype = (int32_t)d.io;
    a.flags = kAdvanceSeq;
    for (int r = 0; r < W; ++r) a.peer[r] = static_cast<char*>(bounce_.ptrs[r]) + o;
    a.mc = nvls ? static_cast<char*>(bounce_.mc_ptr) + o : nullptr;
    a.in[0] = a.out[0] = mine;
    launch(ch, nvls ? KernelId::NVLS_DIRECT : KernelId::P2P_DIRECT, a);
    FR_CUDA(launchCopy(out + start * es, mine, (size_t)n * es, cfg_.bounce_copy_blocks, ch.stream));
    ++stats_.slices;
    ++stats_.bounce_slices;
  }
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
  os << "world=" << topo_.world << " grouping=" << topo_.M << "x" << topo_.D
     << (topo_.favorable ? " (device-major ranks)" : " (machine-major ranks)")
     << " transport=" << alloc_->describe() << " nvls=" << (nvlsAvailable() ? "yes" : "no")
     << " channels=" << plan_.channels << " half_slot=" << plan_.half_bytes
     << "B max_slice=" << plan_.max_slice_bytes << "B blocks=" << cfg_.blocks
     << " algo=" << algoName(cfg_.algo) << " bounce=" << (bounce_.ptrs.empty() ? "no" : "yes");
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
  if (a == Algo::BOUNCE) a = Algo::AUTO;  // this message did not qualify for the bounce path
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

void Engine::launch(Channel& ch, KernelId id, const OpArgs& a) {
  cudaError_t e = launchCollective(id, channels_dev_ + (&ch - channels_.data()), a, cfg_.blocks,
                                   ch.stream);
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
  std::function<Channel&()> take = [&]() -> Channel& {
    const int c = (int)(next_channel_++ % channels_.size());
    if (std::find(used.begin(), used.end(), c) == used.end()) {
      FR_CUDA(cudaStreamWaitEvent(channels_[c].stream, after, 0));
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

  if (runDirect(d, take) || runBounce(d, take)) {
    // nothing else to do
  } else if (d.kind == CollKind::ALLREDUCE) {
    const int64_t bytes = d.numel * wes;
    const Algo whole = chooseAllreduce(bytes, d.wire, d.op);
    if (whole == Algo::ONESHOT ||
        (whole == Algo::NVLS_ONESHOT && bytes <= plan_.max_slice_bytes)) {
      runAllreduceSlice(take(), d, in, out, d.numel, whole);
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
        runAllreduceSlice(take(), d, in + off * ies, out + off * ies, n, a);
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
      Channel& ch = take();
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
    Channel& ch = take();
    return ch.stream;
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
