// The same collectives on host memory, for CPU tensors.  The reference rejects
// CPU tensors outright (fairring/process_group.cc:136); here they run the very
// same algorithm as the GPU kernels -- push into symmetric staging, flag
// barriers with a time limit, local reduce, shard-server reduce across rails,
// gather -- with POSIX shared memory standing in for peer-mapped HBM.  That
// makes the slicing, the (machine, device) index maps, the double-buffered
// staging and the failure handling testable on a machine without a GPU.
#pragma once

#include <chrono>
#include <memory>
#include <string>
#include <vector>

#include "kvstore.h"
#include "layout.h"

namespace fairring {

struct CpuStats {
  uint64_t collectives = 0;
  uint64_t slices = 0;
  uint64_t oneshot = 0;
  uint64_t twoshot = 0;
  uint64_t hierarchical = 0;
};

class CpuEngine {
 public:
  // Collective over all ranks of the group (which must share one host).
  CpuEngine(std::shared_ptr<KvStore> store, const Topo& topo, const MemoryPlan& plan,
            std::chrono::milliseconds wait_timeout);
  ~CpuEngine();

  // In place when in == out.  scale is applied to floating types on first read.
  void allReduce(const void* in, void* out, int64_t numel, DType dt, RedOp op, float scale);
  // in: world * per_rank elements, chunk r belongs to rank r; out: per_rank elements.
  void reduceScatter(const void* in, void* out, int64_t per_rank, DType dt, RedOp op, float scale);
  // in: per_rank elements; out: world * per_rank elements.
  void allGather(const void* in, void* out, int64_t per_rank, DType dt);

  const CpuStats& stats() const { return stats_; }
  // Test hook: this rank stays away from the next `n` barriers it should signal,
  // so that its peers run into their time limit.
  void skipSignals(int n) { skip_signals_ = n; }
  int64_t oneshotMaxBytes = 32 * 1024;

 private:
  struct Shm;
  enum BarrierKind { kAll, kGroup, kRail };
  void barrier(BarrierKind kind, int idx);
  char* stage(int rank, int64_t vec) const;
  template <typename T> void pushPhase(const T* in, const Seg& s, float scale);
  template <typename T> void localReducePhase(const Seg& s, RedOp op, T* out_or_null);
  template <typename T> void serverReducePhase(const Seg& s, RedOp op, T* out_or_null);
  template <typename T> void gatherPhase(T* out, const Seg& s);
  template <typename T> void diffusePhase(const T* in, const Seg& s);
  template <typename T> void pushAllPhase(const T* in, const Seg& s, float scale);
  template <typename T> void reduceAllPhase(T* out, const Seg& s, RedOp op);
  template <typename T> void allReduceT(const T* in, T* out, int64_t numel, RedOp op, float scale);
  template <typename T> void reduceScatterT(const T* in, T* out, int64_t per_rank, RedOp op, float scale);
  template <typename T> void allGatherT(const T* in, T* out, int64_t per_rank);
  void finishOp();

  std::shared_ptr<KvStore> store_;
  Topo topo_;
  MemoryPlan plan_;
  std::chrono::milliseconds wait_timeout_;
  std::unique_ptr<Shm> shm_;
  uint32_t seq_ = 0;
  int skip_signals_ = 0;
  CpuStats stats_;
};

}  // namespace fairring
