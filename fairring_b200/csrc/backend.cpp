#include "backend.h"
#include "store_adapter.h"

#include <ATen/ATen.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAFunctions.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/csrc/distributed/c10d/PrefixStore.hpp>

#include <thread>

namespace fairring {

namespace {

bool toDType(at::ScalarType st, DType* out) {
  switch (st) {
    case at::kByte: *out = DType::U8; return true;
    case at::kChar: *out = DType::I8; return true;
    case at::kInt: *out = DType::I32; return true;
    case at::kLong: *out = DType::I64; return true;
    case at::kHalf: *out = DType::F16; return true;
    case at::kBFloat16: *out = DType::BF16; return true;
    case at::kFloat: *out = DType::F32; return true;
    case at::kDouble: *out = DType::F64; return true;
    default: return false;
  }
}

bool isFloating(DType d) {
  return d == DType::F16 || d == DType::BF16 || d == DType::F32 || d == DType::F64;
}

NvlsMode parseNvls(const std::string& s) {
  if (s == "on" || s == "1") return NvlsMode::ON;
  if (s == "off" || s == "0") return NvlsMode::OFF;
  return NvlsMode::AUTO;
}
SymmTransport parseTransport(const std::string& s) {
  if (s == "vmm") return SymmTransport::VMM;
  if (s == "ipc") return SymmTransport::IPC;
  return SymmTransport::AUTO;
}

void checkDense(const at::Tensor& t, const char* what) {
  TORCH_CHECK(t.layout() == at::kStrided, "fairring: ", what, " must be a strided tensor");
  TORCH_CHECK(t.is_non_overlapping_and_dense(), "fairring: ", what,
              " must be dense and non-overlapping (any permutation of a contiguous tensor)");
}

// Are these tensors back-to-back pieces of one allocation (so that the list is
// really one flat buffer)?  Counterpart of unUnbind, fairring/utils.h:363-386.
bool adjacent(const std::vector<at::Tensor>& ts) {
  if (ts.empty()) return false;
  const char* p = static_cast<const char*>(ts[0].data_ptr());
  const int64_t nb = ts[0].numel() * ts[0].element_size();
  for (size_t i = 0; i < ts.size(); ++i) {
    if (!ts[i].is_contiguous() || ts[i].numel() != ts[0].numel() ||
        ts[i].scalar_type() != ts[0].scalar_type() || ts[i].device() != ts[0].device())
      return false;
    if (static_cast<const char*>(ts[i].data_ptr()) != p + (int64_t)i * nb) return false;
  }
  return true;
}

}  // namespace

// ---------------------------------------------------------------------------
// Work
// ---------------------------------------------------------------------------
WorkFairring::WorkFairring(c10d::OpType op, std::shared_ptr<Engine> engine, int device,
                           std::vector<at::Tensor> result, bool blocking,
                           std::chrono::milliseconds default_timeout)
    : c10d::Work(-1, op), engine_(std::move(engine)), device_(device), result_(std::move(result)),
      blocking_(blocking), default_timeout_(default_timeout) {
  if (!engine_) enqueued_ = true;  // nothing to wait for (CPU path, world of one)
}

WorkFairring::~WorkFairring() {
  // The completion event goes back to the engine only now: nobody can wait on
  // this Work any more, so nobody can observe its next use.
  if (engine_ && done_) engine_->releaseEvent(done_);
}

void WorkFairring::markEnqueued(cudaEvent_t done, cudaStream_t join) {
  {
    std::lock_guard<std::mutex> lk(mu_);
    done_ = done;
    join_ = join;
    enqueued_ = true;
    if (future_) completeFuture();
  }
  cv_.notify_all();
}

void WorkFairring::markFailed(std::exception_ptr e) {
  {
    std::lock_guard<std::mutex> lk(mu_);
    error_ = e;
    enqueued_ = true;
    if (future_) future_->setError(e);
  }
  cv_.notify_all();
}

void WorkFairring::waitEnqueued() {
  std::unique_lock<std::mutex> lk(mu_);
  cv_.wait(lk, [&] { return enqueued_; });
  if (error_) std::rethrow_exception(error_);
}

void WorkFairring::completeFuture() {
  if (done_ == nullptr) {
    future_->markCompleted(c10::IValue(result_));
    return;
  }
  // The Future records its own event on the "current" stream: make that the
  // side stream the collective finished on.
  const c10::DeviceIndex di = static_cast<c10::DeviceIndex>(device_);
  c10::cuda::CUDAGuard g(di);
  c10::cuda::CUDAStreamGuard sg(c10::cuda::getStreamFromExternal(join_, di));
  future_->markCompleted(c10::IValue(result_));
}

c10::intrusive_ptr<c10::ivalue::Future> WorkFairring::getFuture() {
  std::lock_guard<std::mutex> lk(mu_);
  if (!future_) {
    std::vector<c10::Device> devs;
    if (engine_) devs.emplace_back(at::kCUDA, static_cast<c10::DeviceIndex>(device_));
    future_ = c10::make_intrusive<c10::ivalue::Future>(
        c10::ListType::create(c10::TensorType::get()), devs);
    if (enqueued_) {
      if (error_)
        future_->setError(error_);
      else
        completeFuture();
    }
  }
  return future_;
}

bool WorkFairring::isCompleted() {
  std::lock_guard<std::mutex> lk(mu_);
  if (!enqueued_) return false;
  if (done_ == nullptr) return true;
  cudaError_t q = cudaEventQuery(done_);
  if (q == cudaErrorNotReady) {
    (void)cudaGetLastError();
    return false;
  }
  return true;
}
bool WorkFairring::isSuccess() const { return enqueued_ && !error_; }
std::exception_ptr WorkFairring::exception() const { return error_; }
std::vector<at::Tensor> WorkFairring::result() { return result_; }
void WorkFairring::synchronize() { wait(kNoTimeout); }
void WorkFairring::abort() {
  if (engine_) engine_->abort();
}

bool WorkFairring::wait(std::chrono::milliseconds timeout) {
  // Host: until the kernels are enqueued (immediate unless a command thread is
  // used).  Device: the caller's current stream is made to wait for them.
  waitEnqueued();
  if (done_ == nullptr || !engine_) return true;
  const c10::DeviceIndex di = static_cast<c10::DeviceIndex>(device_);
  C10_CUDA_CHECK(cudaStreamWaitEvent(c10::cuda::getCurrentCUDAStream(di).stream(), done_, 0));
  if (blocking_ || timeout != kNoTimeout) {
    const auto limit = timeout != kNoTimeout ? timeout : default_timeout_;
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
      cudaError_t q = cudaEventQuery(done_);
      if (q == cudaSuccess) break;
      TORCH_CHECK(q == cudaErrorNotReady, "fairring: CUDA error while waiting: ",
                  cudaGetErrorString(q));
      (void)cudaGetLastError();
      if (std::chrono::steady_clock::now() - t0 > limit) {
        engine_->abort();
        TORCH_CHECK(false, "fairring: collective did not finish within ", limit.count(),
                    " ms; device-side waits were told to give up");
      }
      std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
    try {
      engine_->checkHealth();
    } catch (const Error& err) {
      TORCH_CHECK(false, err.what());
    }
  }
  return true;
}

// ---------------------------------------------------------------------------
// MultiWork
// ---------------------------------------------------------------------------
bool MultiWorkFairring::isCompleted() {
  for (auto& p : parts_)
    if (!p->isCompleted()) return false;
  return true;
}
bool MultiWorkFairring::isSuccess() const {
  for (auto& p : parts_)
    if (!p->isSuccess()) return false;
  return true;
}
std::exception_ptr MultiWorkFairring::exception() const {
  for (auto& p : parts_)
    if (p->exception()) return p->exception();
  return nullptr;
}
bool MultiWorkFairring::wait(std::chrono::milliseconds timeout) {
  for (auto& p : parts_) p->wait(timeout);
  return true;
}
void MultiWorkFairring::abort() {
  for (auto& p : parts_) p->abort();
}
c10::intrusive_ptr<c10::ivalue::Future> MultiWorkFairring::getFuture() {
  std::lock_guard<std::mutex> lk(mu_);
  if (!future_) {
    std::vector<c10::Device> devs;
    std::vector<c10::cuda::CUDAStream> streams;
    for (auto& p : parts_) {
      const c10::DeviceIndex di = static_cast<c10::DeviceIndex>(p->device());
      devs.emplace_back(at::kCUDA, di);
      streams.push_back(c10::cuda::getStreamFromExternal(p->joinStream(), di));
    }
    future_ = c10::make_intrusive<c10::ivalue::Future>(
        c10::ListType::create(c10::TensorType::get()), devs);
    // The Future records one event per device on that device's current
    // stream: make those the streams the collective finishes on.
    c10::cuda::CUDAMultiStreamGuard g(streams);
    future_->markCompleted(c10::IValue(result_));
  }
  return future_;
}

// ---------------------------------------------------------------------------
// Backend
// ---------------------------------------------------------------------------
BackendFairring::BackendFairring(c10::intrusive_ptr<c10d::Store> store, int rank, int size,
                                 c10::intrusive_ptr<OptionsFairring> options)
    : c10d::Backend(rank, size), store_(std::move(store)), options_(std::move(options)) {
  // Nothing is allocated and nobody is contacted here: like the reference
  // (fairring/process_group.cc:106-116) everything is set up on first use.
}

BackendFairring::~BackendFairring() {
  try {
    shutdown();
  } catch (...) {
  }
}

void BackendFairring::shutdown() {
  std::lock_guard<std::mutex> lk(mu_);
  if (!multi_engines_.empty()) {
    // Tearing an engine down is collective over all (rank, GPU) pairs: the
    // engines of this process must go down side by side.
    std::vector<std::thread> ts;
    for (auto& e : multi_engines_) ts.emplace_back([&e] { e.reset(); });
    for (auto& t : ts) t.join();
    multi_engines_.clear();
    multi_devices_.clear();
  }
  engine_.reset();
  cpu_engine_.reset();
  for (auto& kv : delegates_) {
    try {
      kv.second->shutdown();
    } catch (...) {
    }
  }
  delegates_.clear();
}

void BackendFairring::abort() {
  std::lock_guard<std::mutex> lk(mu_);
  if (engine_) engine_->abort();
}

c10d::ErrorType BackendFairring::getError() {
  std::lock_guard<std::mutex> lk(mu_);
  if (!engine_) return c10d::ErrorType::SUCCESS;
  const uint32_t h = engine_->health(nullptr);
  if (h == kStatusTimeout) return c10d::ErrorType::TIMEOUT;
  if (h != kStatusOk) return c10d::ErrorType::COMM_ERROR;
  return c10d::ErrorType::SUCCESS;
}

const Deployment& BackendFairring::ensureDeployment() {
  if (!have_deployment_) {
    StoreAdapter s(store_, "fairring/");
    deployment_ = detectDeployment(s, getRank(), getSize(), (int)options_->gpus_per_machine,
                                   options_->favorable_layout, options_->boot_id_override);
    have_deployment_ = true;
  }
  return deployment_;
}

std::shared_ptr<Engine> BackendFairring::ensureEngine(int device) {
  TORCH_CHECK(multi_engines_.empty(), "fairring: this process group serves several GPUs per process "
              "(one tensor per GPU in every call); single-tensor collectives are not available on it");
  if (engine_) {
    TORCH_CHECK(device == engine_device_, "fairring: this process group already serves cuda:",
                engine_device_, "; one GPU per process");
    return engine_;
  }
  const Deployment& dep = ensureDeployment();
  const EngineConfig cfg = engineConfig();
  c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
  engine_ = std::make_shared<Engine>(std::make_shared<StoreAdapter>(store_, "fairring/gpu/"),
                                     dep.topo, device, cfg);
  engine_device_ = device;
  if (getRank() == 0) LOG(WARNING) << "fairring: " << engine_->describe();
  return engine_;
}

EngineConfig BackendFairring::engineConfig() const {
  EngineConfig cfg;
  cfg.total_memory = options_->max_memory_allocated_in_bytes;
  cfg.slice_bytes = options_->slice_size_in_bytes;
  cfg.parallelism = (int32_t)options_->min_parallelism;
  cfg.blocks = (int32_t)options_->blocks;
  cfg.sm_budget = (int32_t)options_->sm_budget;
  cfg.oneshot_max_bytes = options_->oneshot_max_bytes;
  cfg.ll_max_bytes = options_->ll_max_bytes;
  cfg.ll2_max_bytes = options_->ll2_max_bytes;
  cfg.ll_channels = (int32_t)options_->ll_channels;
  cfg.inline_small = options_->inline_small;
  cfg.direct_blocks = (int32_t)options_->direct_blocks;
  cfg.direct_unroll = (int32_t)options_->direct_unroll;
  cfg.nvls_min_bytes = options_->nvls_min_bytes;
  cfg.nvls_oneshot_max_bytes = options_->nvls_oneshot_max_bytes;
  const int64_t wait_ms = options_->device_timeout_ms > 0 ? options_->device_timeout_ms
                                                          : (int64_t)options_->timeout.count();
  cfg.device_timeout_ns = (uint64_t)std::max<int64_t>(wait_ms, 1) * 1000000ull;
  cfg.algo = parseAlgo(options_->algo);
  cfg.high_priority = options_->is_high_priority_stream;
  cfg.command_thread = options_->command_thread;
  cfg.transport = parseTransport(options_->transport);
  cfg.nvls = parseNvls(options_->nvls);
  cfg.direct = options_->direct;
  cfg.pipe = options_->pipe;
  cfg.pipe_min_bytes = options_->pipe_min_bytes;
  cfg.pipe_blocks = (int32_t)options_->pipe_blocks;
  cfg.pipe_channels = (int32_t)options_->pipe_channels;
  cfg.pipe_slots = (int32_t)options_->pipe_slots;
  cfg.pipe_chunk_bytes = options_->pipe_chunk_bytes;
  cfg.pipe_stage_bytes = (int32_t)options_->pipe_stage_bytes;
  cfg.pipe_stages = (int32_t)options_->pipe_stages;
  cfg.direct_max_slices = (int32_t)options_->direct_max_slices;
  cfg.direct_min_slice_bytes = options_->direct_min_slice_bytes;
  cfg.bootstrap_timeout = options_->timeout;
  return cfg;
}

void BackendFairring::ensureEngines(const std::vector<int>& devices) {
  if (!multi_engines_.empty()) {
    TORCH_CHECK(devices == multi_devices_, "fairring: every call must name the same GPUs in the "
                "same order as the first one");
    return;
  }
  TORCH_CHECK(!engine_, "fairring: this process group already serves one GPU per process");
  const Deployment& dep = ensureDeployment();
  TORCH_CHECK(dep.single_host, "fairring: several GPUs per process need all ranks on one NVSwitch host");
  const int nd = (int)devices.size();
  const int world = getSize() * nd;
  TORCH_CHECK(world <= kMaxRanks, "fairring: ", getSize(), " processes x ", nd,
              " GPUs exceed the ", kMaxRanks, " ranks of the peer-memory path");
  int gpm = options_->gpus_per_machine > 0 ? (int)options_->gpus_per_machine : world;
  TORCH_CHECK(world % gpm == 0, "fairring: FAIRRING_GPUS_PER_MACHINE must divide ", world);
  EngineConfig cfg = engineConfig();
  cfg.command_thread = false;
  cfg.inline_small = false;
  // Every engine's constructor is a collective over all (rank, GPU) pairs, so
  // the engines of this process are built side by side, one thread each.
  std::vector<std::shared_ptr<Engine>> built(nd);
  std::vector<std::string> errors(nd);
  std::vector<std::thread> ts;
  for (int i = 0; i < nd; ++i) {
    ts.emplace_back([&, i] {
      try {
        c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(devices[i]));
        const Topo topo = makeTopo(world, gpm, options_->favorable_layout, getRank() * nd + i);
        built[i] = std::make_shared<Engine>(std::make_shared<StoreAdapter>(store_, "fairring/gpu/"),
                                            topo, devices[i], cfg);
      } catch (const std::exception& e) {
        errors[i] = e.what();
      }
    });
  }
  for (auto& t : ts) t.join();
  for (int i = 0; i < nd; ++i)
    TORCH_CHECK(errors[i].empty(), "fairring: engine for cuda:", devices[i], " failed: ", errors[i]);
  multi_engines_ = std::move(built);
  multi_devices_ = devices;
  if (getRank() == 0) LOG(WARNING) << "fairring: " << multi_engines_[0]->describe() << " (" << nd << " GPUs per process)";
}

// One tensor per GPU of this process (fairring/machine.cc:177-202 of the
// reference): the same all_reduce runs on every GPU's engine; the returned
// Work waits for all of them.
c10::intrusive_ptr<c10d::Work> BackendFairring::allreduceMulti(std::vector<at::Tensor>& tensors,
                                                               const c10d::AllreduceOptions& opts) {
  std::vector<int> devices;
  for (const auto& t : tensors) {
    TORCH_CHECK(t.is_cuda() && !t.is_sparse(), "fairring: a multi-GPU all_reduce takes dense CUDA tensors");
    TORCH_CHECK(t.numel() == tensors[0].numel() && t.scalar_type() == tensors[0].scalar_type(),
                "fairring: the tensors of a multi-GPU all_reduce must agree in size and dtype");
    checkDense(t, "the all_reduce tensor");
    for (int d : devices) TORCH_CHECK(d != t.get_device(), "fairring: one tensor per GPU");
    devices.push_back(t.get_device());
  }
  Mapped m = mapOp(tensors[0], opts.reduceOp);
  TORCH_CHECK(m.ok, "fairring: this reduction is not available for several GPUs per process");
  std::lock_guard<std::mutex> lk(mu_);
  ensureEngines(devices);
  if (m.scale != 1.0f) m.scale = 1.0f / (float)(getSize() * (int)devices.size());  // AVG over all GPUs
  std::vector<c10::intrusive_ptr<WorkFairring>> parts;
  for (size_t i = 0; i < tensors.size(); ++i) {
    auto& engine = multi_engines_[i];
    const c10::DeviceIndex di = static_cast<c10::DeviceIndex>(devices[i]);
    c10::cuda::CUDAGuard guard(di);
    CollectiveDesc d;
    d.kind = CollKind::ALLREDUCE;
    d.in = d.out = tensors[i].data_ptr();
    d.numel = tensors[i].numel();
    d.io = d.wire = m.dtype;
    d.op = m.op;
    d.scale = m.scale;
    auto work = c10::make_intrusive<WorkFairring>(c10d::OpType::ALLREDUCE, engine, (int)di,
                                                  std::vector<at::Tensor>{tensors[i]},
                                                  options_->blocking_wait, options_->timeout);
    cudaEvent_t after = engine->begin(c10::cuda::getCurrentCUDAStream(di).stream());
    try {
      std::vector<cudaStream_t> used;
      cudaStream_t s = engine->run(d, after, &used);
      engine->releaseEvent(after);
      for (cudaStream_t u : used)
        c10::cuda::CUDACachingAllocator::recordStream(tensors[i].storage().data_ptr(),
                                                      c10::cuda::getStreamFromExternal(u, di));
      work->markEnqueued(engine->begin(s), s);
    } catch (const Error& e) {
      engine->releaseEvent(after);
      TORCH_CHECK(false, e.what());
    }
    parts.push_back(std::move(work));
  }
  ++seq_;
  return c10::make_intrusive<MultiWorkFairring>(c10d::OpType::ALLREDUCE, std::move(parts), tensors);
}

CpuEngine& BackendFairring::ensureCpuEngine() {
  if (!cpu_engine_) {
    const Deployment& dep = ensureDeployment();
    // The host path runs one slice at a time: one channel.
    MemoryPlan plan = planMemory(options_->max_memory_allocated_in_bytes,
                                 options_->slice_size_in_bytes, 1, dep.topo.world, 4096);
    cpu_engine_.reset(new CpuEngine(std::make_shared<StoreAdapter>(store_, "fairring/cpu/"),
                                    dep.topo, plan,
                                    std::chrono::milliseconds(
                                        options_->device_timeout_ms > 0
                                            ? options_->device_timeout_ms
                                            : (int64_t)options_->timeout.count())));
    cpu_engine_->oneshotMaxBytes = std::min<int64_t>(options_->oneshot_max_bytes, 32 << 10);
  }
  return *cpu_engine_;
}

BackendFairring::Mapped BackendFairring::mapOp(const at::Tensor& t, const c10d::ReduceOp& op) const {
  Mapped m;
  if (!toDType(t.scalar_type(), &m.dtype)) return m;
  switch (op.op_) {
    case c10d::ReduceOp::SUM: m.op = RedOp::SUM; break;
    case c10d::ReduceOp::MAX: m.op = RedOp::MAX; break;
    case c10d::ReduceOp::MIN: m.op = RedOp::MIN; break;
    case c10d::ReduceOp::AVG:
      if (!isFloating(m.dtype)) return m;
      m.op = RedOp::SUM;
      m.scale = 1.0f / (float)getSize();
      break;
    default: return m;  // PRODUCT, bitwise, PREMUL_SUM: the delegate knows them
  }
  m.ok = true;
  return m;
}

BackendFairring::Route BackendFairring::routeFor(const at::Tensor& t, bool mapped_ok) {
  if (!mapped_ok) return Route::DELEGATE;
  const Deployment& dep = ensureDeployment();
  // Peer memory and POSIX shared memory both stop at the host boundary.
  if (!dep.single_host || dep.topo.world > kMaxRanks) return Route::DELEGATE;
  if (t.is_cuda()) return Route::OWN_GPU;
  if (t.is_cpu()) return Route::OWN_CPU;
  return Route::DELEGATE;
}

c10::intrusive_ptr<c10d::Backend> BackendFairring::delegate(const at::Device& dev) {
  const std::string key = dev.is_cuda() ? "cuda" : "cpu";
  auto it = delegates_.find(key);
  if (it != delegates_.end()) return it->second;
  TORCH_CHECK(factory_, "fairring: no delegate factory installed; the operation needs the ",
              key == "cuda" ? "NCCL" : "Gloo", " backend");
  auto b = factory_(key);
  TORCH_CHECK(b, "fairring: delegate factory returned nothing for ", key);
  delegates_[key] = b;
  return b;
}

c10::intrusive_ptr<c10d::Backend> BackendFairring::delegateFor(const std::vector<at::Tensor>& t) {
  TORCH_CHECK(!t.empty(), "fairring: empty tensor list");
  std::lock_guard<std::mutex> lk(mu_);
  ++delegated_;
  return delegate(t[0].device());
}

c10::intrusive_ptr<c10d::Work> BackendFairring::completedWork(c10d::OpType type,
                                                              std::vector<at::Tensor> result) {
  return c10::make_intrusive<WorkFairring>(type, nullptr, -1, std::move(result), false,
                                           options_->timeout);
}

c10::intrusive_ptr<c10d::Work> BackendFairring::runGpu(c10d::OpType type, const CollectiveDesc& d,
                                                       std::vector<at::Tensor> keep,
                                                       std::vector<at::Tensor> result,
                                                       std::function<void()> epilogue) {
  auto engine = engine_;
  const c10::DeviceIndex di = static_cast<c10::DeviceIndex>(engine_device_);
  c10::cuda::CUDAGuard guard(di);
  const auto cur = c10::cuda::getCurrentCUDAStream(di);
  cudaEvent_t after = engine->begin(cur.stream());
  auto work = c10::make_intrusive<WorkFairring>(type, engine, (int)di, std::move(result),
                                                options_->blocking_wait, options_->timeout);
  const bool async = engine->config().command_thread;
  auto job = [=]() {
    try {
      c10::cuda::CUDAGuard g2(di);
      std::vector<cudaStream_t> used;
      cudaStream_t s = nullptr;
      try {
        s = engine->run(d, after, &used);
      } catch (...) {
        engine->releaseEvent(after);
        throw;
      }
      engine->releaseEvent(after);  // the side streams' waits on it are enqueued
      // The tensors are used on side streams: tell the caching allocator, as
      // the reference does for its stage streams (device.cc:297-301).
      for (const auto& t : keep)
        for (cudaStream_t u : used)
          c10::cuda::CUDACachingAllocator::recordStream(t.storage().data_ptr(),
                                                        c10::cuda::getStreamFromExternal(u, di));
      if (epilogue) {
        c10::cuda::CUDAStreamGuard sg(c10::cuda::getStreamFromExternal(s, di));
        epilogue();
      }
      work->markEnqueued(engine->begin(s), s);
    } catch (...) {
      work->markFailed(std::current_exception());
      if (!async) throw;
    }
  };
  try {
    engine->submit(job);
  } catch (const Error& e) {
    TORCH_CHECK(false, e.what());
  }
  ++seq_;
  return work;
}

// ---- all_reduce ------------------------------------------------------------
c10::intrusive_ptr<c10d::Work> BackendFairring::allreduce(std::vector<at::Tensor>& tensors,
                                                          const c10d::AllreduceOptions& opts) {
  TORCH_CHECK(!tensors.empty(), "fairring: empty tensor list");
  if (tensors.size() > 1) return allreduceMulti(tensors, opts);
  at::Tensor& t = tensors[0];
  TORCH_CHECK(!t.is_sparse(), "fairring: sparse tensors are not supported");
  const Mapped m = mapOp(t, opts.reduceOp);
  Route route;
  {
    std::lock_guard<std::mutex> lk(mu_);
    route = routeFor(t, m.ok);
  }
  if (route == Route::DELEGATE) return delegateFor(tensors)->allreduce(tensors, opts);
  checkDense(t, "the all_reduce tensor");
  std::lock_guard<std::mutex> lk(mu_);
  if (route == Route::OWN_CPU) {
    try {
      ensureCpuEngine().allReduce(t.data_ptr(), t.data_ptr(), t.numel(), m.dtype, m.op, m.scale);
    } catch (const Error& e) {
      TORCH_CHECK(false, e.what());
    }
    ++seq_;
    return completedWork(c10d::OpType::ALLREDUCE, tensors);
  }
  ensureEngine(t.get_device());
  if (getSize() == 1 && m.scale == 1.0f) return completedWork(c10d::OpType::ALLREDUCE, tensors);
  CollectiveDesc d;
  d.kind = CollKind::ALLREDUCE;
  d.in = t.data_ptr();
  d.out = t.data_ptr();
  d.numel = t.numel();
  d.io = d.wire = m.dtype;
  d.op = m.op;
  d.scale = m.scale;
  if (!opts.asyncOp && engine_->fitsInline(d)) {
    // A small blocking all_reduce: the kernel goes on the caller's own stream,
    // which would wait for it anyway; nothing is handed to a side stream.
    const c10::DeviceIndex di = static_cast<c10::DeviceIndex>(engine_device_);
    c10::cuda::CUDAGuard guard(di);
    try {
      engine_->runInline(d, c10::cuda::getCurrentCUDAStream(di).stream());
    } catch (const Error& e) {
      TORCH_CHECK(false, e.what());
    }
    ++seq_;
    return completedWork(c10d::OpType::ALLREDUCE, tensors);
  }
  return runGpu(c10d::OpType::ALLREDUCE, d, {t}, tensors, nullptr);
}

c10::intrusive_ptr<c10d::Work> BackendFairring::allreduceFused(
    at::Tensor tensor, double scale, c10::optional<at::ScalarType> wire_dtype,
    const std::string& op) {
  TORCH_CHECK(tensor.is_cuda(), "fairring: allreduce_fused takes a CUDA tensor");
  checkDense(tensor, "the all_reduce tensor");
  DType io;
  TORCH_CHECK(toDType(tensor.scalar_type(), &io), "fairring: unsupported dtype");
  DType wire = io;
  if (wire_dtype.has_value()) TORCH_CHECK(toDType(*wire_dtype, &wire), "fairring: unsupported wire dtype");
  TORCH_CHECK(comboSupported(io, wire), "fairring: tensors of ", tensor.scalar_type(),
              " cannot be carried as ", *wire_dtype, " (fp32 -> bf16/fp16 or same type)");
  RedOp rop = RedOp::SUM;
  if (op == "max") rop = RedOp::MAX;
  else if (op == "min") rop = RedOp::MIN;
  else TORCH_CHECK(op == "sum", "fairring: op must be sum, max or min");
  std::lock_guard<std::mutex> lk(mu_);
  const Deployment& dep = ensureDeployment();
  TORCH_CHECK(dep.single_host && dep.topo.world <= kMaxRanks,
              "fairring: the fused all_reduce needs all ranks on one NVSwitch host");
  ensureEngine(tensor.get_device());
  CollectiveDesc d;
  d.kind = CollKind::ALLREDUCE;
  d.in = tensor.data_ptr();
  d.out = tensor.data_ptr();
  d.numel = tensor.numel();
  d.io = io;
  d.wire = wire;
  d.op = rop;
  d.scale = (float)scale;
  if (getSize() == 1 && d.scale == 1.0f) return completedWork(c10d::OpType::ALLREDUCE, {tensor});
  return runGpu(c10d::OpType::ALLREDUCE, d, {tensor}, {tensor}, nullptr);
}

// ---- reduce_scatter ---------------------------------------------------------
c10::intrusive_ptr<c10d::Work> BackendFairring::_reduce_scatter_base(
    at::Tensor& output, at::Tensor& input, const c10d::ReduceScatterOptions& opts) {
  TORCH_CHECK(input.scalar_type() == output.scalar_type() && input.device() == output.device(),
              "fairring: reduce_scatter input and output must agree in dtype and device");
  TORCH_CHECK(input.numel() == output.numel() * getSize(),
              "fairring: reduce_scatter input must hold world_size * output elements");
  const Mapped m = mapOp(input, opts.reduceOp);
  Route route;
  {
    std::lock_guard<std::mutex> lk(mu_);
    route = routeFor(input, m.ok && input.is_contiguous() && output.is_contiguous());
  }
  if (route == Route::DELEGATE) {
    std::vector<at::Tensor> v{input};
    return delegateFor(v)->_reduce_scatter_base(output, input, opts);
  }
  std::lock_guard<std::mutex> lk(mu_);
  if (route == Route::OWN_CPU) {
    try {
      ensureCpuEngine().reduceScatter(input.data_ptr(), output.data_ptr(), output.numel(), m.dtype,
                                      m.op, m.scale);
    } catch (const Error& e) {
      TORCH_CHECK(false, e.what());
    }
    ++seq_;
    return completedWork(c10d::OpType::_REDUCE_SCATTER_BASE, {output});
  }
  ensureEngine(input.get_device());
  CollectiveDesc d;
  d.kind = CollKind::REDUCE_SCATTER;
  d.in = input.data_ptr();
  d.out = output.data_ptr();
  d.numel = output.numel();
  d.io = d.wire = m.dtype;
  d.op = m.op;
  d.scale = m.scale;
  return runGpu(c10d::OpType::_REDUCE_SCATTER_BASE, d, {input, output}, {output}, nullptr);
}

c10::intrusive_ptr<c10d::Work> BackendFairring::reduce_scatter(
    std::vector<at::Tensor>& outputs, std::vector<std::vector<at::Tensor>>& inputs,
    const c10d::ReduceScatterOptions& opts) {
  TORCH_CHECK(outputs.size() == 1 && inputs.size() == 1,
              "fairring: one output tensor and one input list per call");
  TORCH_CHECK((int)inputs[0].size() == getSize(),
              "fairring: reduce_scatter needs one input tensor per rank");
  for (const auto& t : inputs[0])
    TORCH_CHECK(t.numel() == outputs[0].numel() && t.scalar_type() == outputs[0].scalar_type() &&
                    t.device() == outputs[0].device(),
                "fairring: reduce_scatter inputs must match the output in size, dtype and device");
  // Back-to-back views of one buffer are used in place; anything else is
  // flattened first (the reference insists on the former, utils.h:363-386).
  at::Tensor flat;
  if (adjacent(inputs[0])) {
    flat = at::from_blob(inputs[0][0].data_ptr(), {outputs[0].numel() * getSize()},
                         inputs[0][0].options());
  } else {
    std::vector<at::Tensor> parts;
    for (const auto& t : inputs[0]) parts.push_back(t.reshape({-1}));
    flat = at::cat(parts);
  }
  at::Tensor out = outputs[0];
  if (!out.is_contiguous()) {
    std::vector<at::Tensor> v{flat};
    return delegateFor(v)->reduce_scatter(outputs, inputs, opts);
  }
  auto work = _reduce_scatter_base(out, flat, opts);
  // `flat` may be a temporary: its storage was recorded on the side streams
  // by _reduce_scatter_base, and the inputs themselves outlive the call.
  return work;
}

// ---- all_gather ---------------------------------------------------------------
c10::intrusive_ptr<c10d::Work> BackendFairring::_allgather_base(at::Tensor& output,
                                                                at::Tensor& input,
                                                                const c10d::AllgatherOptions& opts) {
  TORCH_CHECK(input.scalar_type() == output.scalar_type() && input.device() == output.device(),
              "fairring: all_gather input and output must agree in dtype and device");
  TORCH_CHECK(output.numel() == input.numel() * getSize(),
              "fairring: all_gather output must hold world_size * input elements");
  DType dt;
  const bool ok = toDType(input.scalar_type(), &dt) && input.is_contiguous() && output.is_contiguous();
  Route route;
  {
    std::lock_guard<std::mutex> lk(mu_);
    route = routeFor(input, ok);
  }
  if (route == Route::DELEGATE) {
    std::vector<at::Tensor> v{input};
    return delegateFor(v)->_allgather_base(output, input, opts);
  }
  std::lock_guard<std::mutex> lk(mu_);
  if (route == Route::OWN_CPU) {
    try {
      ensureCpuEngine().allGather(input.data_ptr(), output.data_ptr(), input.numel(), dt);
    } catch (const Error& e) {
      TORCH_CHECK(false, e.what());
    }
    ++seq_;
    return completedWork(c10d::OpType::_ALLGATHER_BASE, {output});
  }
  ensureEngine(input.get_device());
  CollectiveDesc d;
  d.kind = CollKind::ALLGATHER;
  d.in = input.data_ptr();
  d.out = output.data_ptr();
  d.numel = input.numel();
  d.io = d.wire = dt;
  return runGpu(c10d::OpType::_ALLGATHER_BASE, d, {input, output}, {output}, nullptr);
}

c10::intrusive_ptr<c10d::Work> BackendFairring::allgather(
    std::vector<std::vector<at::Tensor>>& outputs, std::vector<at::Tensor>& inputs,
    const c10d::AllgatherOptions& opts) {
  TORCH_CHECK(outputs.size() == 1 && inputs.size() == 1,
              "fairring: one input tensor and one output list per call");
  TORCH_CHECK((int)outputs[0].size() == getSize(),
              "fairring: all_gather needs one output tensor per rank");
  at::Tensor in = inputs[0];
  for (const auto& t : outputs[0])
    TORCH_CHECK(t.numel() == in.numel() && t.scalar_type() == in.scalar_type() &&
                    t.device() == in.device(),
                "fairring: all_gather outputs must match the input in size, dtype and device");
  if (!in.is_contiguous()) in = in.contiguous();
  if (adjacent(outputs[0])) {
    at::Tensor flat = at::from_blob(outputs[0][0].data_ptr(), {in.numel() * getSize()}, in.options());
    return _allgather_base(flat, in, opts);
  }
  // Scattered outputs: gather into one buffer, then copy each piece out on the
  // stream the collective finishes on.
  at::Tensor flat = at::empty({in.numel() * getSize()}, in.options());
  DType dt;
  Route route;
  {
    std::lock_guard<std::mutex> lk(mu_);
    route = routeFor(in, toDType(in.scalar_type(), &dt));
  }
  if (route == Route::DELEGATE) return delegateFor(inputs)->allgather(outputs, inputs, opts);
  std::vector<at::Tensor> outs = outputs[0];
  const int64_t n = in.numel();
  auto scatter_out = [outs, flat, n]() {
    for (size_t i = 0; i < outs.size(); ++i)
      outs[i].copy_(flat.narrow(0, (int64_t)i * n, n).view_as(outs[i]), /*non_blocking=*/true);
  };
  if (route == Route::OWN_CPU) {
    auto w = _allgather_base(flat, in, opts);
    scatter_out();
    return completedWork(c10d::OpType::ALLGATHER, outs);
  }
  std::lock_guard<std::mutex> lk(mu_);
  ensureEngine(in.get_device());
  CollectiveDesc d;
  d.kind = CollKind::ALLGATHER;
  d.in = in.data_ptr();
  d.out = flat.data_ptr();
  d.numel = n;
  d.io = d.wire = dt;
  std::vector<at::Tensor> keep = outs;
  keep.push_back(in);
  keep.push_back(flat);
  return runGpu(c10d::OpType::ALLGATHER, d, keep, outs, scatter_out);
}

// ---- delegated -------------------------------------------------------------------
c10::intrusive_ptr<c10d::Work> BackendFairring::broadcast(std::vector<at::Tensor>& t,
                                                          const c10d::BroadcastOptions& o) {
  return delegateFor(t)->broadcast(t, o);
}
c10::intrusive_ptr<c10d::Work> BackendFairring::allreduce_coalesced(
    std::vector<at::Tensor>& t, const c10d::AllreduceCoalescedOptions& o) {
  return delegateFor(t)->allreduce_coalesced(t, o);
}
c10::intrusive_ptr<c10d::Work> BackendFairring::reduce(std::vector<at::Tensor>& t,
                                                       const c10d::ReduceOptions& o) {
  return delegateFor(t)->reduce(t, o);
}
c10::intrusive_ptr<c10d::Work> BackendFairring::allgather_coalesced(
    std::vector<std::vector<at::Tensor>>& o, std::vector<at::Tensor>& i,
    const c10d::AllgatherOptions& opts) {
  return delegateFor(i)->allgather_coalesced(o, i, opts);
}
c10::intrusive_ptr<c10d::Work> BackendFairring::allgather_into_tensor_coalesced(
    std::vector<at::Tensor>& o, std::vector<at::Tensor>& i, const c10d::AllgatherOptions& opts) {
  return delegateFor(i)->allgather_into_tensor_coalesced(o, i, opts);
}
c10::intrusive_ptr<c10d::Work> BackendFairring::reduce_scatter_tensor_coalesced(
    std::vector<at::Tensor>& o, std::vector<at::Tensor>& i, const c10d::ReduceScatterOptions& opts) {
  return delegateFor(i)->reduce_scatter_tensor_coalesced(o, i, opts);
}
c10::intrusive_ptr<c10d::Work> BackendFairring::gather(std::vector<std::vector<at::Tensor>>& o,
                                                       std::vector<at::Tensor>& i,
                                                       const c10d::GatherOptions& opts) {
  return delegateFor(i)->gather(o, i, opts);
}
c10::intrusive_ptr<c10d::Work> BackendFairring::scatter(std::vector<at::Tensor>& o,
                                                        std::vector<std::vector<at::Tensor>>& i,
                                                        const c10d::ScatterOptions& opts) {
  return delegateFor(o)->scatter(o, i, opts);
}
c10::intrusive_ptr<c10d::Work> BackendFairring::alltoall_base(at::Tensor& o, at::Tensor& i,
                                                              std::vector<int64_t>& os,
                                                              std::vector<int64_t>& is,
                                                              const c10d::AllToAllOptions& opts) {
  std::vector<at::Tensor> v{i};
  return delegateFor(v)->alltoall_base(o, i, os, is, opts);
}
c10::intrusive_ptr<c10d::Work> BackendFairring::alltoall(std::vector<at::Tensor>& o,
                                                         std::vector<at::Tensor>& i,
                                                         const c10d::AllToAllOptions& opts) {
  return delegateFor(i)->alltoall(o, i, opts);
}
c10::intrusive_ptr<c10d::Work> BackendFairring::send(std::vector<at::Tensor>& t, int dst, int tag) {
  return delegateFor(t)->send(t, dst, tag);
}
c10::intrusive_ptr<c10d::Work> BackendFairring::recv(std::vector<at::Tensor>& t, int src, int tag) {
  return delegateFor(t)->recv(t, src, tag);
}
c10::intrusive_ptr<c10d::Work> BackendFairring::recvAnysource(std::vector<at::Tensor>& t, int tag) {
  return delegateFor(t)->recvAnysource(t, tag);
}

namespace {
at::Device barrierDevice(const c10d::BarrierOptions& o, int engine_device) {
  if (o.device.has_value()) return *o.device;
  if (!o.device_ids.empty()) return at::Device(at::kCUDA, (c10::DeviceIndex)o.device_ids[0]);
  if (engine_device >= 0) return at::Device(at::kCUDA, (c10::DeviceIndex)engine_device);
  return at::Device(at::kCPU);
}
}  // namespace

c10::intrusive_ptr<c10d::Work> BackendFairring::barrier(const c10d::BarrierOptions& o) {
  c10::intrusive_ptr<c10d::Backend> b;
  {
    std::lock_guard<std::mutex> lk(mu_);
    ++delegated_;
    b = delegate(barrierDevice(o, engine_device_));
  }
  return b->barrier(o);
}

void BackendFairring::monitoredBarrier(const c10d::BarrierOptions& o, bool wait_all_ranks) {
  c10::intrusive_ptr<c10d::Backend> b;
  {
    std::lock_guard<std::mutex> lk(mu_);
    ++delegated_;
    b = delegate(at::Device(at::kCPU));  // only Gloo implements it
  }
  b->monitoredBarrier(o, wait_all_ranks);
}

// ---- introspection ------------------------------------------------------------------
std::string BackendFairring::describe() {
  std::lock_guard<std::mutex> lk(mu_);
  if (engine_) return engine_->describe();
  if (have_deployment_) {
    std::ostringstream os;
    os << "world=" << deployment_.topo.world << " grouping=" << deployment_.topo.M << "x"
       << deployment_.topo.D << " (no GPU engine yet)";
    return os.str();
  }
  return "uninitialised (nothing has been communicated yet)";
}

std::map<std::string, int64_t> BackendFairring::stats() {
  std::lock_guard<std::mutex> lk(mu_);
  std::map<std::string, int64_t> m;
  m["delegated"] = (int64_t)delegated_;
  m["sequence"] = (int64_t)seq_;
  m["kernel_launches_process"] = (int64_t)launchCount();
  if (engine_) {
    EngineStats s = engine_->stats();
    m["gpu_collectives"] = (int64_t)s.collectives;
    m["gpu_slices"] = (int64_t)s.slices;
    m["gpu_wire_bytes"] = (int64_t)s.wire_bytes;
    m["gpu_inline_collectives"] = (int64_t)s.inline_collectives;
    m["symmetric_regions"] = (int64_t)s.symmetric_regions;
    m["symmetric_bytes"] = (int64_t)s.symmetric_bytes;
    m["symmetric_pending_release"] = (int64_t)s.symmetric_pending;
    for (int k = 0; k < (int)KernelId::kCount; ++k)
      m[std::string("launch_") + kernelName((KernelId)k)] = (int64_t)s.launches[k];
    m["nvls"] = engine_->nvlsAvailable() ? 1 : 0;
    m["channels"] = engine_->plan().channels;
    m["half_bytes"] = engine_->plan().half_bytes;
    m["max_slice_bytes"] = engine_->plan().max_slice_bytes;
  }
  if (cpu_engine_) {
    const CpuStats& c = cpu_engine_->stats();
    m["cpu_collectives"] = (int64_t)c.collectives;
    m["cpu_slices"] = (int64_t)c.slices;
    m["cpu_oneshot"] = (int64_t)c.oneshot;
    m["cpu_twoshot"] = (int64_t)c.twoshot;
    m["cpu_hierarchical"] = (int64_t)c.hierarchical;
  }
  return m;
}

std::map<std::string, int64_t> BackendFairring::deployment() {
  std::lock_guard<std::mutex> lk(mu_);
  const Deployment& d = ensureDeployment();
  return {{"world", d.topo.world},       {"D", d.topo.D},
          {"M", d.topo.M},               {"favorable", d.topo.favorable},
          {"rank", d.topo.rank},         {"m", d.topo.m},
          {"d", d.topo.d},               {"num_hosts", d.num_hosts},
          {"ranks_per_host", d.ranks_per_host}, {"single_host", d.single_host ? 1 : 0}};
}

std::vector<std::map<std::string, std::string>> BackendFairring::trace() {
  std::lock_guard<std::mutex> lk(mu_);
  std::vector<std::map<std::string, std::string>> out;
  if (!engine_) return out;
  static const char* kKinds[] = {"all_reduce", "reduce_scatter", "all_gather"};
  for (const TraceEntry& t : engine_->trace()) {
    std::map<std::string, std::string> m;
    m["seq"] = std::to_string(t.seq);
    m["kind"] = kKinds[t.kind];
    m["bytes"] = std::to_string(t.bytes);
    m["first_kernel"] = t.first_kernel >= 0 ? kernelName((KernelId)t.first_kernel) : "none";
    m["launches"] = std::to_string(t.launches);
    m["slices"] = std::to_string(t.slices);
    m["channels"] = std::to_string(t.channels);
    m["host_us"] = std::to_string(t.host_us);
    out.push_back(std::move(m));
  }
  return out;
}

void BackendFairring::checkHealth() {
  std::shared_ptr<Engine> e;
  {
    std::lock_guard<std::mutex> lk(mu_);
    e = engine_;
  }
  if (!e) return;
  c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(engine_device_));
  for (cudaStream_t s : e->streams()) C10_CUDA_CHECK(cudaStreamSynchronize(s));
  try {
    e->checkHealth();
  } catch (const Error& err) {
    TORCH_CHECK(false, err.what());
  }
}

std::string BackendFairring::health() {
  std::shared_ptr<Engine> e;
  {
    std::lock_guard<std::mutex> lk(mu_);
    e = engine_;
  }
  std::string what;
  if (e && e->health(&what) != kStatusOk) return what.empty() ? "failed" : what;
  return "";
}

int64_t BackendFairring::releaseSymmetric() {
  std::shared_ptr<Engine> e;
  {
    std::lock_guard<std::mutex> lk(mu_);
    e = engine_;
  }
  if (!e) return 0;
  try {
    return e->releaseFreedSymmetric();
  } catch (const Error& err) {
    TORCH_CHECK(false, err.what());
  }
}

void BackendFairring::setOption(const std::string& name, int64_t value) {
  std::shared_ptr<Engine> e;
  {
    std::lock_guard<std::mutex> lk(mu_);
    e = engine_;
  }
  TORCH_CHECK(e, "fairring: no GPU engine yet (run a collective first)");
  try {
    e->setOption(name, value);
  } catch (const Error& err) {
    TORCH_CHECK(false, err.what());
  }
}

void BackendFairring::reset() {
  std::lock_guard<std::mutex> lk(mu_);
  if (engine_) engine_->reset();
}

at::Tensor BackendFairring::symmetricEmpty(int64_t numel, at::ScalarType dtype) {
  TORCH_CHECK(numel > 0, "fairring: symmetric_empty needs a positive size");
  std::lock_guard<std::mutex> lk(mu_);
  const Deployment& dep = ensureDeployment();
  TORCH_CHECK(dep.single_host && dep.topo.world <= kMaxRanks,
              "fairring: symmetric memory needs all ranks on one NVSwitch host");
  const int device = engine_ ? engine_device_ : (int)c10::cuda::current_device();
  auto engine = ensureEngine(device);
  const size_t bytes = (size_t)numel * c10::elementSize(dtype);
  void* p = nullptr;
  try {
    p = engine->allocSymmetric(bytes);
  } catch (const Error& e) {
    TORCH_CHECK(false, e.what());
  }
  // When the tensor dies the region is marked free; it is unmapped at the next
  // collective boundary at which every rank has let go of it (the next
  // symmetric_empty or release_symmetric), or with the process group.
  auto keep = engine;
  return at::from_blob(p, {numel}, [keep](void* q) { keep->freeSymmetric(q); },
                       at::TensorOptions().dtype(dtype).device(at::kCUDA, (c10::DeviceIndex)device));
}

bool BackendFairring::supportsTensorAlloc(c10::DeviceIndex) {
  std::lock_guard<std::mutex> lk(mu_);
  const Deployment& dep = ensureDeployment();
  return dep.single_host && dep.topo.world <= kMaxRanks;
}

at::Tensor BackendFairring::allocateTensor(long size, at::TensorOptions options) {
  return symmetricEmpty(size, c10::typeMetaToScalarType(options.dtype()));
}

void BackendFairring::skipCpuSignals(int n) {
  std::lock_guard<std::mutex> lk(mu_);
  ensureCpuEngine().skipSignals(n);
}

}  // namespace fairring
