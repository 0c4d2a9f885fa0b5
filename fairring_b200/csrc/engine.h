// Per-GPU engine: owns the symmetric staging memory, the channels (slot + flag
// pad + side stream each), picks a kernel variant per slice and enqueues the
// kernels.  Counterpart of DeviceFairring in the reference
// (fairring/device.{h,cc}): there, five stage streams run NCCL calls chained by
// events and a command thread does the enqueueing; here a slice is one to three
// kernel launches on one of `channels` side streams, consecutive slices go to
// different channels so they overlap, and the command thread is optional
// because a kernel launch never blocks.
#pragma once

#include <cuda_runtime.h>

#include <array>
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <deque>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "command_queue.h"
#include "kernels/kernels.h"
#include "kernels/pipe_allreduce.h"
#include "kvstore.h"
#include "layout.h"
#include "symmem.h"

namespace fairring {

enum class Algo : int32_t { AUTO = 0, ONESHOT, TWOSHOT, HIER, NVLS, NVLS_ONESHOT, PIPE, LL, LL2 };
const char* algoName(Algo a);
Algo parseAlgo(const std::string& s);

struct EngineConfig {
  int64_t total_memory = 50ll << 20;   // FAIRRING_TOTAL_MEMORY
  int64_t slice_bytes = 25ll << 20;    // FAIRRING_SLICE_SIZE
  int32_t parallelism = 16;            // FAIRRING_PARALLELISM: slices in flight
  int64_t min_half_bytes = 4ll << 20;  // channels are merged until a half-slot is at least this
  int32_t blocks = 16;                 // thread blocks per kernel
  int32_t sm_budget = 64;              // channels x blocks never exceeds this (nor the SM count)
  int64_t oneshot_max_bytes = 256 << 10;
  // Messages up to ll_max_bytes take the flag-in-data kernel (no barrier at
  // all); its areas (2 x 16 bytes per 8 bytes of message per rank, on up to
  // ll_channels channels) come off the top of the memory budget.  0: off.
  int64_t ll_max_bytes = 32 << 10;
  // ... and up to ll2_max_bytes its two-shot form (reduce-scatter + all-gather
  // in flag-in-data words), which needs 4 bytes of area per byte of message.
  int64_t ll2_max_bytes = 1 << 20;
  int32_t ll_channels = 4;
  // A blocking all_reduce (async_op=False) that fits the flag-in-data kernel is
  // launched on the caller's own stream: no hand-over to a side stream and back.
  bool inline_small = true;
  int32_t direct_blocks = 0;           // blocks of an in-place launch (0: `blocks`); the switch
                                       // saturates with few, and backward keeps the other SMs
  int32_t direct_unroll = 8;           // in-place NVLS kernel: 16-byte loads in flight per thread
  int64_t nvls_min_bytes = 0;          // below this the peer-load two-shot is used
  int64_t nvls_oneshot_max_bytes = 2 << 20;
  uint64_t device_timeout_ns = 30ull * 1000 * 1000 * 1000;
  Algo algo = Algo::AUTO;
  bool high_priority = true;
  bool command_thread = false;
  SymmTransport transport = SymmTransport::AUTO;
  NvlsMode nvls = NvlsMode::AUTO;
  // Tensors allocated with allocSymmetric() are all-reduced in place, without
  // staging: "auto" (NVLS when possible, else peer loads), "p2p", "nvls", "off".
  std::string direct = "auto";
  int64_t direct_min_slice_bytes = 2ll << 20;  // a message is split over channels down to this
  int32_t direct_max_slices = 2;               // ... but an in-place message into at most this many
  // Ordinary (non-symmetric) tensors of at least pipe_min_bytes take the
  // pipelined kernel (kernels/pipe_allreduce.h): one launch whatever the size.
  // "auto" | "on" | "off".  A third of the memory budget becomes its staging
  // rings when it is enabled.
  std::string pipe = "auto";
  int64_t pipe_min_bytes = 64 << 20;  // 8 GPUs: ahead of the staged kernels from 64 MiB on
  int32_t pipe_blocks = 16;        // thread blocks of one pipelined launch (fewer for small messages)
  int32_t pipe_channels = 2;       // rings, i.e. pipelined launches that may overlap
  int32_t pipe_slots = 4;          // ring length in chunks
  int64_t pipe_chunk_bytes = 0;    // 0: chosen from the message size
  int32_t pipe_stage_bytes = 16 << 10;  // one shared-memory stage of a copy role
  int32_t pipe_stages = 6;
  std::chrono::milliseconds bootstrap_timeout{120000};
};

enum class CollKind : int32_t { ALLREDUCE = 0, REDUCE_SCATTER, ALLGATHER };

struct CollectiveDesc {
  CollKind kind = CollKind::ALLREDUCE;
  const void* in = nullptr;
  void* out = nullptr;
  int64_t numel = 0;   // all_reduce: total elements; the others: elements per rank
  DType io = DType::F32;
  DType wire = DType::F32;
  RedOp op = RedOp::SUM;
  float scale = 1.0f;
};

struct EngineStats {
  uint64_t collectives = 0;
  uint64_t slices = 0;
  uint64_t wire_bytes = 0;
  uint64_t inline_collectives = 0;  // launched on the caller's stream
  uint64_t symmetric_regions = 0;   // live allocations handed out by allocSymmetric
  uint64_t symmetric_bytes = 0;     // ... and their size (outside the staging budget)
  uint64_t symmetric_pending = 0;   // freed by their tensor, not yet released by all ranks
  std::array<uint64_t, (size_t)KernelId::kCount> launches{};
};

// One line of the engine's trace: what a collective was turned into.
struct TraceEntry {
  uint64_t seq = 0;
  int32_t kind = 0;           // CollKind
  int64_t bytes = 0;          // wire bytes of the whole collective
  int32_t first_kernel = -1;  // KernelId of the first launch
  int32_t launches = 0;
  int32_t slices = 0;
  int32_t channels = 0;       // side streams used
  double host_us = 0;         // time spent enqueueing
};

class Engine {
 public:
  // Collective over the group.  `device` must be the current CUDA device.
  Engine(std::shared_ptr<KvStore> store, const Topo& topo, int device, const EngineConfig& cfg);
  ~Engine();

  // Record "the caller's work so far" so that a later run() can order itself
  // after it; cheap, called on the caller's thread.  The event belongs to the
  // caller until it hands it back with releaseEvent(): it is never re-recorded
  // behind a holder's back.
  cudaEvent_t begin(cudaStream_t caller);
  void releaseEvent(cudaEvent_t e);
  // Enqueue the whole collective.  Returns the side stream on which everything
  // it launched is ordered; the caller records its completion event there.
  // `used` (optional) receives every side stream the collective touched.
  cudaStream_t run(const CollectiveDesc& d, cudaEvent_t after,
                   std::vector<cudaStream_t>* used_streams = nullptr);
  // Would run() put this collective on the caller's stream if asked to?
  bool fitsInline(const CollectiveDesc& d) const;
  // The same collective launched on `caller` itself (see inline_small).  Only
  // for descriptors for which fitsInline() holds.
  void runInline(const CollectiveDesc& d, cudaStream_t caller);
  // Changes a tunable between collectives; every rank must make the same call
  // at the same point.  Throws for unknown names and values that would break
  // the residency bound.
  void setOption(const std::string& name, int64_t value);
  // Run `fn` now, or on the command thread when one is configured.
  void submit(std::function<void()> fn);

  // Throws if a kernel reported a timeout/abort since the last call.
  void checkHealth();
  // Non-throwing variant: code (StatusCode) and a description.
  uint32_t health(std::string* what) const;
  // Makes every device-side wait give up (host-visible flag).
  void abort();
  // Collective: after a failure, bring flags and sequence numbers back to zero.
  void reset();

  // Collective: symmetric device memory (peer-mapped everywhere, multicast
  // alias when available).  all_reduce on a tensor inside it runs in place with
  // no staging copies.  It is not part of the staging budget.
  void* allocSymmetric(size_t bytes);
  // Not collective, any thread: the holder of `p` (from allocSymmetric) is done
  // with it.  The memory is unmapped at the next allocSymmetric() or
  // releaseFreedSymmetric() on which every rank has let go of the same region.
  void freeSymmetric(void* p);
  // Collective: release the regions every rank has freed; returns how many.
  int releaseFreedSymmetric();

  const Topo& topo() const { return topo_; }
  const MemoryPlan& plan() const { return plan_; }
  const EngineConfig& config() const { return cfg_; }
  EngineStats stats() const;
  // The last collectives (newest last), at most 256.
  std::vector<TraceEntry> trace() const;
  bool nvlsAvailable() const { return region_.mc_ptr != nullptr; }
  std::string describe() const;
  Algo chooseAllreduce(int64_t wire_bytes, DType wire, RedOp op) const;
  std::vector<cudaStream_t> streams() const;

 private:
  struct Channel {
    cudaStream_t stream = nullptr;
    ChannelDev dev{};
    cudaEvent_t done = nullptr;
    // Where the channel's last kernel was launched (its own stream, or a
    // caller's for an inline collective) and an event recorded after it.
    cudaStream_t last_stream = nullptr;
    cudaEvent_t last_done = nullptr;
  };
  void launchLL(Channel& ch, const CollectiveDesc& d, cudaStream_t stream);
  // 0: not for the flag-in-data kernels; 1: one-shot; 2: two-shot.
  int llKind(const CollectiveDesc& d) const;
  void launch(Channel& ch, KernelId id, const OpArgs& a, int blocks = 0);
  bool directEligible(const CollectiveDesc& d) const;
  void runAllreduceSlice(Channel& ch, const CollectiveDesc& d, const void* in, void* out,
                         int64_t n, Algo algo);
  bool findSymmetric(const void* p, size_t bytes, const SymmRegion** reg, size_t* off) const;
  int releaseFreedLocked();
  bool runDirect(const CollectiveDesc& d, const std::function<Channel&(int)>& take);
  bool runPipe(const CollectiveDesc& d, const std::function<Channel&(int)>& take);

  std::shared_ptr<KvStore> store_;
  Topo topo_;
  int device_;
  EngineConfig cfg_;
  MemoryPlan plan_;
  std::unique_ptr<SymmAllocator> alloc_;
  SymmRegion region_;
  struct UserRegion {
    SymmRegion reg;
    uint64_t id = 0;    // allocation number: the same on every rank
    bool freed = false;
  };
  std::map<uintptr_t, UserRegion> user_regions_;  // by local base address
  uint64_t next_region_id_ = 0;
  int release_round_ = 0;
  // Pipelined kernel: flag pads of all its channels, then one ring per channel.
  SymmRegion pipe_region_;
  size_t pipe_flags_bytes_ = 0;
  int64_t pipe_slot_bytes_ = 0;
  int pipe_channels_ = 0;
  uint64_t next_pipe_ = 0;
  SymmRegion ll_region_;
  int64_t ll_half_bytes_ = 0;
  int ll_channels_ = 0;
  uint64_t next_ll_ = 0;
  int sm_count_ = 0;
  uint32_t* pipe_seq_dev_ = nullptr;
  PipeChannelDev* pipe_channels_dev_ = nullptr;
  size_t flags_bytes_ = 0;
  uint32_t* seq_dev_ = nullptr;
  uint32_t* status_host_ = nullptr;  // pinned + mapped: [channels][kStatusWords], then abort word
  uint32_t* status_dev_ = nullptr;
  std::vector<Channel> channels_;
  ChannelDev* channels_dev_ = nullptr;  // device copy of channels_[i].dev
  std::vector<cudaEvent_t> free_events_;  // created on demand, reused after releaseEvent()
  std::mutex events_mu_;
  uint64_t next_channel_ = 0;
  mutable std::mutex mu_;
  EngineStats stats_;
  std::vector<TraceEntry> trace_;  // ring of kTraceLen entries
  TraceEntry cur_;
  bool nvtx_ = false;
  bool poisoned_ = false;
  int reset_count_ = 0;

  CommandQueue queue_;
  std::thread worker_;
};

}  // namespace fairring
