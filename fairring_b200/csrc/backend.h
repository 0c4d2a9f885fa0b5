// The c10d backend: what `torch.distributed.init_process_group("fairring")`
// talks to.  Counterpart of ProcessGroupFairring / WorkFairring /
// OptionsFairring in the reference (fairring/process_group.{h,cc}), rebuilt on
// today's c10d::Backend / c10d::Work interfaces.
//
//   own algorithms : allreduce, reduce_scatter, _reduce_scatter_base,
//                    allgather, _allgather_base  (CUDA tensors -> Engine,
//                    CPU tensors -> CpuEngine)
//   delegated      : everything else, to a lazily created NCCL (CUDA) or Gloo
//                    (CPU) backend on a prefixed store; also any reduction op
//                    or dtype the kernels do not cover, instead of aborting
//                    the process as the reference does (fairring/utils.h:247-256).
#pragma once

#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/Store.hpp>
#include <torch/csrc/distributed/c10d/Work.hpp>

#include <condition_variable>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <string>

#include "cpu_path.h"
#include "engine.h"
#include "topology.h"

namespace fairring {

constexpr const char* kBackendName = "fairring";

struct OptionsFairring : c10d::Backend::Options {
  explicit OptionsFairring(std::chrono::milliseconds timeout = kBackendDefaultTimeout)
      : c10d::Backend::Options(kBackendName, timeout) {}

  // Same three knobs as the reference (fairring/process_group.h:52-77) ...
  int64_t max_memory_allocated_in_bytes = 50ll << 20;
  int64_t max_padding_allocated_in_bytes = 1 << 20;  // accepted; tails are predicated, no padding buffers exist
  int64_t min_parallelism = 16;
  bool is_high_priority_stream = true;
  // ... plus what the B200 design adds.
  int64_t slice_size_in_bytes = 25ll << 20;
  int64_t gpus_per_machine = 0;   // 0: one group per real host
  bool favorable_layout = false;  // numbering of virtual machines: d*M+m instead of m*D+d
  std::string algo = "auto";
  int64_t blocks = 16;
  int64_t sm_budget = 64;
  int64_t oneshot_max_bytes = 256 << 10;
  int64_t ll_max_bytes = 32 << 10;   // flag-in-data kernel up to this size; 0: off
  int64_t ll2_max_bytes = 1 << 20;   // ... and its two-shot form up to this size; 0: off
  int64_t ll_channels = 4;
  bool inline_small = true;          // blocking small all_reduce runs on the caller's stream
  int64_t direct_blocks = 0;
  int64_t direct_unroll = 8;
  int64_t nvls_min_bytes = 0;
  int64_t nvls_oneshot_max_bytes = 2 << 20;
  // Limit of one device-side wait on a peer.  0: the process group's timeout,
  // so that a rank that is merely late (checkpointing, evaluation, a data stall)
  // is waited for as long as the other collectives of the group would wait.
  int64_t device_timeout_ms = 0;
  std::string nvls = "auto";       // auto | on | off
  std::string transport = "auto";  // auto | vmm | ipc
  std::string direct = "auto";     // auto | p2p | nvls | off: in-place path for symmetric tensors
  std::string pipe = "auto";       // auto | on | off: pipelined kernel for ordinary tensors
  int64_t pipe_min_bytes = 64 << 20;
  int64_t pipe_blocks = 16;
  int64_t pipe_channels = 2;
  int64_t pipe_slots = 4;
  int64_t pipe_chunk_bytes = 0;
  int64_t pipe_stage_bytes = 16 << 10;
  int64_t pipe_stages = 6;
  int64_t direct_max_slices = 2;
  int64_t direct_min_slice_bytes = 2 << 20;
  bool command_thread = false;
  bool blocking_wait = false;
  std::string boot_id_override;    // tests: pretend to be on another host
};

class BackendFairring;

// Completion of a collective is a CUDA event on one of the engine's side
// streams: wait() makes the caller's current stream wait for it and returns
// without blocking the host (like NCCL's work objects).  A CUDA-aware Future is
// only built when somebody asks for one (DDP does); the reference always goes
// through a Future (fairring/process_group.cc:35-75).
class WorkFairring : public c10d::Work {
 public:
  WorkFairring(c10d::OpType op, std::shared_ptr<Engine> engine, int device,
               std::vector<at::Tensor> result, bool blocking,
               std::chrono::milliseconds default_timeout);
  ~WorkFairring() override;
  bool isCompleted() override;
  bool isSuccess() const override;
  std::exception_ptr exception() const override;
  std::vector<at::Tensor> result() override;
  void synchronize() override;
  bool wait(std::chrono::milliseconds timeout = kNoTimeout) override;
  void abort() override;
  c10::intrusive_ptr<c10::ivalue::Future> getFuture() override;

  // Called by the enqueueing code (caller's thread, or the command thread).
  void markEnqueued(cudaEvent_t done, cudaStream_t join);
  void markFailed(std::exception_ptr e);
  // Where the collective finishes (valid once enqueued).
  int device() const { return device_; }
  cudaStream_t joinStream() const { return join_; }

 private:
  void waitEnqueued();
  void completeFuture();  // mu_ held

  std::shared_ptr<Engine> engine_;
  int device_;
  std::vector<at::Tensor> result_;
  bool blocking_;
  std::chrono::milliseconds default_timeout_;
  std::mutex mu_;
  std::condition_variable cv_;
  bool enqueued_ = false;
  cudaEvent_t done_ = nullptr;
  cudaStream_t join_ = nullptr;
  std::exception_ptr error_;
  c10::intrusive_ptr<c10::ivalue::Future> future_;
};

// One collective over several GPUs of this process: one WorkFairring per GPU,
// waited for together.  Counterpart of mergeMultiDeviceFutures in the reference
// (fairring/machine.cc:251-288), which merges the per-device futures on a merge
// stream per device; here waiting is an event wait on each device's current
// stream and the merged Future is completed under all the finishing streams.
class MultiWorkFairring : public c10d::Work {
 public:
  MultiWorkFairring(c10d::OpType op, std::vector<c10::intrusive_ptr<WorkFairring>> parts,
                    std::vector<at::Tensor> result)
      : c10d::Work(-1, op), parts_(std::move(parts)), result_(std::move(result)) {}
  bool isCompleted() override;
  bool isSuccess() const override;
  std::exception_ptr exception() const override;
  std::vector<at::Tensor> result() override { return result_; }
  void synchronize() override { wait(kNoTimeout); }
  bool wait(std::chrono::milliseconds timeout = kNoTimeout) override;
  void abort() override;
  c10::intrusive_ptr<c10::ivalue::Future> getFuture() override;

 private:
  std::vector<c10::intrusive_ptr<WorkFairring>> parts_;
  std::vector<at::Tensor> result_;
  std::mutex mu_;
  c10::intrusive_ptr<c10::ivalue::Future> future_;
};

using DelegateFactory = std::function<c10::intrusive_ptr<c10d::Backend>(const std::string&)>;

class BackendFairring : public c10d::Backend {
 public:
  BackendFairring(c10::intrusive_ptr<c10d::Store> store, int rank, int size,
                  c10::intrusive_ptr<OptionsFairring> options);
  ~BackendFairring() override;

  const std::string getBackendName() const override { return kBackendName; }
  c10::intrusive_ptr<c10d::Backend::Options> getBackendOptions() override { return options_; }

  // --- own algorithms -------------------------------------------------------
  c10::intrusive_ptr<c10d::Work> allreduce(std::vector<at::Tensor>& tensors,
                                           const c10d::AllreduceOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> allgather(std::vector<std::vector<at::Tensor>>& outputs,
                                           std::vector<at::Tensor>& inputs,
                                           const c10d::AllgatherOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> _allgather_base(at::Tensor& output, at::Tensor& input,
                                                 const c10d::AllgatherOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> reduce_scatter(std::vector<at::Tensor>& outputs,
                                                std::vector<std::vector<at::Tensor>>& inputs,
                                                const c10d::ReduceScatterOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> _reduce_scatter_base(at::Tensor& output, at::Tensor& input,
                                                      const c10d::ReduceScatterOptions& opts) override;
  // all_reduce with the gradient scale and the wire-dtype cast fused into the
  // kernels (what the DDP communication hook calls).
  c10::intrusive_ptr<c10d::Work> allreduceFused(at::Tensor tensor, double scale,
                                                c10::optional<at::ScalarType> wire_dtype,
                                                const std::string& op);

  // --- delegated --------------------------------------------------------------
  c10::intrusive_ptr<c10d::Work> broadcast(std::vector<at::Tensor>& t,
                                           const c10d::BroadcastOptions& o) override;
  c10::intrusive_ptr<c10d::Work> allreduce_coalesced(std::vector<at::Tensor>& t,
                                                     const c10d::AllreduceCoalescedOptions& o) override;
  c10::intrusive_ptr<c10d::Work> reduce(std::vector<at::Tensor>& t,
                                        const c10d::ReduceOptions& o) override;
  c10::intrusive_ptr<c10d::Work> allgather_coalesced(std::vector<std::vector<at::Tensor>>& o,
                                                     std::vector<at::Tensor>& i,
                                                     const c10d::AllgatherOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> allgather_into_tensor_coalesced(
      std::vector<at::Tensor>& o, std::vector<at::Tensor>& i,
      const c10d::AllgatherOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> reduce_scatter_tensor_coalesced(
      std::vector<at::Tensor>& o, std::vector<at::Tensor>& i,
      const c10d::ReduceScatterOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> gather(std::vector<std::vector<at::Tensor>>& o,
                                        std::vector<at::Tensor>& i,
                                        const c10d::GatherOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> scatter(std::vector<at::Tensor>& o,
                                         std::vector<std::vector<at::Tensor>>& i,
                                         const c10d::ScatterOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> alltoall_base(at::Tensor& o, at::Tensor& i,
                                               std::vector<int64_t>& os, std::vector<int64_t>& is,
                                               const c10d::AllToAllOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> alltoall(std::vector<at::Tensor>& o, std::vector<at::Tensor>& i,
                                          const c10d::AllToAllOptions& opts) override;
  void monitoredBarrier(const c10d::BarrierOptions& o, bool wait_all_ranks) override;
  c10::intrusive_ptr<c10d::Work> send(std::vector<at::Tensor>& t, int dst, int tag) override;
  c10::intrusive_ptr<c10d::Work> recv(std::vector<at::Tensor>& t, int src, int tag) override;
  c10::intrusive_ptr<c10d::Work> recvAnysource(std::vector<at::Tensor>& t, int tag) override;
  c10::intrusive_ptr<c10d::Work> barrier(const c10d::BarrierOptions& o) override;

  void setSequenceNumberForGroup() override {}
  uint64_t getSequenceNumberForGroup() override { return seq_; }
  void setTimeout(std::chrono::milliseconds t) override { options_->timeout = t; }
  c10d::ErrorType getError() override;
  // Communication-optimised memory: tensors from here are symmetric (peer- and
  // multicast-mapped) and are all-reduced in place.
  bool supportsTensorAlloc(c10::DeviceIndex device) override;
  at::Tensor allocateTensor(long size, at::TensorOptions options = {}) override;
  void abort() override;
  void shutdown() override;

  // --- introspection and control (Python) ------------------------------------
  void setDelegateFactory(DelegateFactory f) { factory_ = std::move(f); }
  std::string describe();
  std::map<std::string, int64_t> stats();
  void checkHealth();
  // Host-side look at the kernels' status words, without synchronising: empty
  // when healthy, else what gave up waiting for whom.
  std::string health();
  // Collective in spirit: every rank changes the same engine tunable at the same
  // point between collectives (used by the tuning sweep).
  void setOption(const std::string& name, int64_t value);
  void reset();
  // Collective: unmap the symmetric tensors that have died on every rank.
  int64_t releaseSymmetric();
  void skipCpuSignals(int n);
  // Collective: a 1-D tensor in symmetric memory of the current CUDA device;
  // all_reduce on (slices of) it runs in place without staging copies.
  at::Tensor symmetricEmpty(int64_t numel, at::ScalarType dtype);
  std::map<std::string, int64_t> deployment();
  // The engine's record of the last collectives (kind, bytes, first kernel, launches, ...).
  std::vector<std::map<std::string, std::string>> trace();

 private:
  enum class Route { OWN_GPU, OWN_CPU, DELEGATE };
  struct Mapped {
    bool ok = false;
    DType dtype = DType::F32;
    RedOp op = RedOp::SUM;
    float scale = 1.0f;
  };
  Mapped mapOp(const at::Tensor& t, const c10d::ReduceOp& op) const;
  Route routeFor(const at::Tensor& t, bool mapped_ok);
  c10::intrusive_ptr<c10d::Backend> delegate(const at::Device& dev);
  c10::intrusive_ptr<c10d::Backend> delegateFor(const std::vector<at::Tensor>& t);
  const Deployment& ensureDeployment();
  std::shared_ptr<Engine> ensureEngine(int device);
  EngineConfig engineConfig() const;
  CpuEngine& ensureCpuEngine();
  c10::intrusive_ptr<c10d::Work> runGpu(c10d::OpType type, const CollectiveDesc& d,
                                        std::vector<at::Tensor> keep,
                                        std::vector<at::Tensor> result,
                                        std::function<void()> epilogue);
  c10::intrusive_ptr<c10d::Work> completedWork(c10d::OpType type, std::vector<at::Tensor> result);
  // Several GPUs in this process (one tensor per GPU in a call): one engine per
  // GPU, built together on first use; every (rank, GPU) pair is a rank of the
  // peer-memory world.
  void ensureEngines(const std::vector<int>& devices);
  c10::intrusive_ptr<c10d::Work> allreduceMulti(std::vector<at::Tensor>& tensors,
                                                const c10d::AllreduceOptions& opts);

  c10::intrusive_ptr<c10d::Store> store_;
  c10::intrusive_ptr<OptionsFairring> options_;
  DelegateFactory factory_;
  std::mutex mu_;
  bool have_deployment_ = false;
  Deployment deployment_;
  std::shared_ptr<Engine> engine_;
  int engine_device_ = -1;
  std::vector<std::shared_ptr<Engine>> multi_engines_;  // multi-GPU-per-process mode
  std::vector<int> multi_devices_;
  std::unique_ptr<CpuEngine> cpu_engine_;
  std::map<std::string, c10::intrusive_ptr<c10d::Backend>> delegates_;
  uint64_t seq_ = 0;
  uint64_t delegated_ = 0;
};

}  // namespace fairring
