// The collective kernels (sm_100a).  Each kernel is a short sequence of
// "phases" separated by flag barriers between the same-numbered blocks of the
// participating GPUs.  A phase moves 16-byte vectors between the user's tensor,
// this GPU's staging slot and the peers' staging slots (mapped peer memory over
// NVLink, or the NVSwitch multicast address for the NVLS variants).
//
// Work split: a chunk of qv vectors is cut into tiles of kTile vectors; block b
// owns tiles b, b+G, ...  The split is the same in every phase and on every
// rank, so the data block b reads after a barrier was written by block b of
// the peer before that barrier: block-to-block flags are enough and no
// grid-wide synchronisation is needed inside a kernel.  Between kernels of one
// channel the stream order of the peer does the rest (a peer's block can only
// signal from kernel k+1 once its kernel k has finished).
//
// Staging reuse: consecutive collectives of a channel use alternate halves of
// the slot and the first barrier of every collective spans all ranks; having
// passed it proves that every peer finished the collective before, so the half
// used two collectives ago is free again without a trailing barrier.
//
// Reference behaviour covered: fairring/device.cc:33-209 (the five stage
// primitives) and :444-753 (their per-slice composition).

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <atomic>

#include "device_prims.cuh"
#include "kernels.h"

namespace fairring {
namespace {

using namespace dev;

constexpr int kU = 1;                      // vectors per thread per tile
constexpr int kTile = kThreads * kU;       // vectors per tile

enum BarrierKind { kAll = 0, kGroup = 1, kRail = 2 };

struct BlockCtx {
  uint32_t seq;     // collectives this block has completed on this channel
  uint64_t half;    // byte offset of the half-slot in use
  int b;            // block index within the rank
  int G;            // blocks per rank
};

// Arrive at barrier `idx` of the current collective and wait for the peers of
// the given kind.  Returns false if a wait gave up; the reason is then in the
// status words and the caller must leave the kernel.
template <int KIND>
__device__ __forceinline__ bool barrier(const ChannelDev& c, const BlockCtx& bc, int idx) {
  const Topo& t = c.topo;
  const uint32_t epoch = bc.seq * (uint32_t)kBarriersPerOp + (uint32_t)idx + 1u;
  const int n = KIND == kAll ? t.world : (KIND == kGroup ? t.D : t.M);
  __syncthreads();
  uint32_t st = kStatusOk;
  int peer = -1;
  if ((int)threadIdx.x < n) {
    const int i = threadIdx.x;
    peer = KIND == kAll ? i : (KIND == kGroup ? rankOf(t, t.m, i) : rankOf(t, i, t.d));
    if (peer != t.rank) {
      __threadfence_system();
      stReleaseSys(c.flags[peer] + t.rank * kMaxBlocks + bc.b, epoch);
      st = waitFlag(c.flags[t.rank] + peer * kMaxBlocks + bc.b, epoch, c.timeout_ns,
                    c.abort_flag);
      if (st != kStatusOk) {
        volatile uint32_t* s = c.status;
        s[1] = (uint32_t)idx;
        s[2] = (uint32_t)peer;
        s[3] = bc.seq;
        __threadfence_system();
        s[0] = st;
      }
    }
  }
  return __syncthreads_or(st != kStatusOk) == 0;
}

__device__ __forceinline__ BlockCtx enter(const ChannelDev& c) {
  BlockCtx bc;
  bc.b = blockIdx.x;
  bc.G = gridDim.x;
  bc.seq = c.seq[bc.b];  // written only by this block, at the end of a kernel
  bc.half = (bc.seq & 1u) ? c.half_bytes : 0;
  return bc;
}

__device__ __forceinline__ void leave(const ChannelDev& c, const OpArgs& a, const BlockCtx& bc) {
  __syncthreads();
  if ((a.flags & kAdvanceSeq) && threadIdx.x == 0) c.seq[bc.b] = bc.seq + 1u;
}

__device__ __forceinline__ char* stageAt(char* slot, uint64_t half, int64_t vec) {
  return slot + half + (uint64_t)vec * kVecBytes;
}

template <typename IO>
__device__ __forceinline__ bool chunkAligned(const IO* base, const Seg& s, int c) {
  return ((reinterpret_cast<uintptr_t>(base + (int64_t)c * s.chunk_stride)) & 15u) == 0;
}

// Scale (floating accumulators only) while the data is first read.
template <typename A, int V>
__device__ __forceinline__ void applyScale(A (&a)[V], float scale) {
  if constexpr (std::is_floating_point<A>::value) {
    if (scale != 1.0f) {
#pragma unroll
      for (int i = 0; i < V; ++i) a[i] = a[i] * (A)scale;
    }
  }
}

// ---------------------------------------------------------------------------
// Phase: push.  Read the user's input once and store rail chunk j destined to
// group member d' into slot d of that member's staging (scaled, cast to the
// wire type).  With M == 1 this is "chunk p goes to rank p".
// ---------------------------------------------------------------------------
template <typename IO, typename WIRE>
__device__ __forceinline__ void phasePush(const ChannelDev& c, const OpArgs& a,
                                          const BlockCtx& bc) {
  constexpr int V = kVecBytes / sizeof(WIRE);
  using Acc = typename Tr<IO>::Acc;
  const Topo& t = c.topo;
  const Seg& s = a.seg;
  const IO* in = static_cast<const IO*>(a.in);
  const int64_t ntiles = ceilDiv(s.qv, kTile);
  for (int j = 0; j < t.M; ++j) {
    for (int64_t tile = bc.b; tile < ntiles; tile += bc.G) {
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int64_t v = tile * kTile + u * kThreads + threadIdx.x;
        if (v >= s.qv) continue;
#pragma unroll 4
        for (int k = 0; k < t.D; ++k) {
          const int dd = (t.d + 1 + k) % t.D;  // start at the neighbour: spreads the links
          const int chunk = rankOf(t, j, dd);
          const int nvalid = (int)validInVector(s, chunk, v, V);
          Acc x[V];
          loadUser<IO, V>(in + (int64_t)chunk * s.chunk_stride + v * V, nvalid,
                          chunkAligned(in, s, chunk), x);
          applyScale(x, a.scale);
          const int peer = rankOf(t, t.m, dd);
          stStage(stageAt(c.staging[peer], bc.half, stagingVec(t, s, t.d, j) + v),
                  pack<WIRE, V>(x));
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Phase: local reduce.  Sum (or max/min) the D source slots of this GPU's own
// staging, in slot order so that the result does not depend on timing; write
// the self slot, or the user's output for a flat reduce_scatter.
// ---------------------------------------------------------------------------
template <typename IO, typename WIRE>
__device__ __forceinline__ void phaseLocalReduce(const ChannelDev& c, const OpArgs& a,
                                                 const BlockCtx& bc) {
  constexpr int V = kVecBytes / sizeof(WIRE);
  using Acc = typename Tr<WIRE>::Acc;
  const Topo& t = c.topo;
  const Seg& s = a.seg;
  char* own = c.staging[t.rank];
  const bool to_user = (a.flags & kToUser) != 0;
  IO* out = static_cast<IO*>(a.out);
  const int64_t ntiles = ceilDiv(s.qv, kTile);
  for (int j = 0; j < t.M; ++j) {
    for (int64_t tile = bc.b; tile < ntiles; tile += bc.G) {
      uint4 raw[kU][kMaxRanks];
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int64_t v = tile * kTile + u * kThreads + threadIdx.x;
#pragma unroll
        for (int k = 0; k < kMaxRanks; ++k)
          if (k < t.D && v < s.qv)
            raw[u][k] = ldStage(stageAt(own, bc.half, stagingVec(t, s, k, j) + v));
      }
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int64_t v = tile * kTile + u * kThreads + threadIdx.x;
        if (v >= s.qv) continue;
        Acc acc[V];
        unpack<WIRE, V>(raw[u][0], acc);
#pragma unroll
        for (int k = 1; k < kMaxRanks; ++k) {
          if (k < t.D) {
            Acc x[V];
            unpack<WIRE, V>(raw[u][k], x);
#pragma unroll
            for (int i = 0; i < V; ++i) acc[i] = combine(acc[i], x[i], a.op);
          }
        }
        if (to_user) {
          // Flat reduce_scatter: this rank's chunk is its whole output.
          const int chunk = rankOf(t, j, t.d);
          const int nvalid = (int)validInVector(s, chunk, v, V);
          typename Tr<IO>::Acc y[V];
#pragma unroll
          for (int i = 0; i < V; ++i) y[i] = (typename Tr<IO>::Acc)acc[i];
          storeUser<IO, V>(out + v * V, nvalid, (reinterpret_cast<uintptr_t>(out) & 15u) == 0, y);
        } else {
          stStage(stageAt(own, bc.half, stagingVec(t, s, t.d, j) + v), pack<WIRE, V>(acc));
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Phase: shard-server reduce.  This GPU serves shard (d, m): pull the group
// partial sums of that shard from the self slot of each rail peer (machine
// order), reduce in registers, then either push the result back into every
// rail peer's self slot (all_reduce: collect + add + diffuse in one pass) or
// write the user's output (reduce_scatter).
// ---------------------------------------------------------------------------
template <typename IO, typename WIRE>
__device__ __forceinline__ void phaseServerReduce(const ChannelDev& c, const OpArgs& a,
                                                  const BlockCtx& bc) {
  constexpr int V = kVecBytes / sizeof(WIRE);
  using Acc = typename Tr<WIRE>::Acc;
  const Topo& t = c.topo;
  const Seg& s = a.seg;
  const bool to_user = (a.flags & kToUser) != 0;
  IO* out = static_cast<IO*>(a.out);
  const int64_t shard = stagingVec(t, s, t.d, t.m);
  const int64_t ntiles = ceilDiv(s.qv, kTile);
  for (int64_t tile = bc.b; tile < ntiles; tile += bc.G) {
    uint4 raw[kU][kMaxRanks];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int64_t v = tile * kTile + u * kThreads + threadIdx.x;
#pragma unroll
      for (int k = 0; k < kMaxRanks; ++k)
        if (k < t.M && v < s.qv)
          raw[u][k] = ldStage(stageAt(c.staging[rankOf(t, k, t.d)], bc.half, shard + v));
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int64_t v = tile * kTile + u * kThreads + threadIdx.x;
      if (v >= s.qv) continue;
      Acc acc[V];
      unpack<WIRE, V>(raw[u][0], acc);
#pragma unroll
      for (int k = 1; k < kMaxRanks; ++k) {
        if (k < t.M) {
          Acc x[V];
          unpack<WIRE, V>(raw[u][k], x);
#pragma unroll
          for (int i = 0; i < V; ++i) acc[i] = combine(acc[i], x[i], a.op);
        }
      }
      if (to_user) {
        const int nvalid = (int)validInVector(s, t.rank, v, V);
        typename Tr<IO>::Acc y[V];
#pragma unroll
        for (int i = 0; i < V; ++i) y[i] = (typename Tr<IO>::Acc)acc[i];
        storeUser<IO, V>(out + v * V, nvalid, (reinterpret_cast<uintptr_t>(out) & 15u) == 0, y);
      } else {
        const uint4 r = pack<WIRE, V>(acc);
#pragma unroll
        for (int k = 0; k < kMaxRanks; ++k)
          if (k < t.M) stStage(stageAt(c.staging[rankOf(t, k, t.d)], bc.half, shard + v), r);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Phase: gather.  Pull the reduced rail chunks from the self slot of every
// group member and write them (cast back) into the user's output.
// ---------------------------------------------------------------------------
template <typename IO, typename WIRE>
__device__ __forceinline__ void phaseGather(const ChannelDev& c, const OpArgs& a,
                                            const BlockCtx& bc) {
  constexpr int V = kVecBytes / sizeof(WIRE);
  const Topo& t = c.topo;
  const Seg& s = a.seg;
  IO* out = static_cast<IO*>(a.out);
  const int64_t ntiles = ceilDiv(s.qv, kTile);
  for (int j = 0; j < t.M; ++j) {
    for (int64_t tile = bc.b; tile < ntiles; tile += bc.G) {
      uint4 raw[kU][kMaxRanks];
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int64_t v = tile * kTile + u * kThreads + threadIdx.x;
#pragma unroll
        for (int k = 0; k < kMaxRanks; ++k) {
          if (k < t.D && v < s.qv) {
            const int dd = (t.d + k) % t.D;
            raw[u][k] = ldStage(stageAt(c.staging[rankOf(t, t.m, dd)], bc.half,
                                        stagingVec(t, s, dd, j) + v));
          }
        }
      }
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int64_t v = tile * kTile + u * kThreads + threadIdx.x;
        if (v >= s.qv) continue;
#pragma unroll
        for (int k = 0; k < kMaxRanks; ++k) {
          if (k < t.D) {
            const int dd = (t.d + k) % t.D;
            const int chunk = rankOf(t, j, dd);
            const int nvalid = (int)validInVector(s, chunk, v, V);
            typename Tr<WIRE>::Acc x[V];
            unpack<WIRE, V>(raw[u][k], x);
            typename Tr<IO>::Acc y[V];
#pragma unroll
            for (int i = 0; i < V; ++i) y[i] = (typename Tr<IO>::Acc)x[i];
            storeUser<IO, V>(out + (int64_t)chunk * s.chunk_stride + v * V, nvalid,
                             chunkAligned(out, s, chunk), y);
          }
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Phase: diffuse (all_gather stage 1).  The user's input is this rank's chunk;
// store it into the self slot, rail position m, of every rail peer (self
// included).  Afterwards every GPU's self slot holds its whole rail.
// ---------------------------------------------------------------------------
template <typename IO, typename WIRE>
__device__ __forceinline__ void phaseDiffuse(const ChannelDev& c, const OpArgs& a,
                                             const BlockCtx& bc) {
  constexpr int V = kVecBytes / sizeof(WIRE);
  using Acc = typename Tr<IO>::Acc;
  const Topo& t = c.topo;
  const Seg& s = a.seg;
  const IO* in = static_cast<const IO*>(a.in);
  const bool aligned = (reinterpret_cast<uintptr_t>(in) & 15u) == 0;
  const int64_t shard = stagingVec(t, s, t.d, t.m);
  const int64_t ntiles = ceilDiv(s.qv, kTile);
  for (int64_t tile = bc.b; tile < ntiles; tile += bc.G) {
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int64_t v = tile * kTile + u * kThreads + threadIdx.x;
      if (v >= s.qv) continue;
      int64_t nv = s.chunk_len - v * V;
      const int nvalid = nv > V ? V : (nv < 0 ? 0 : (int)nv);
      Acc x[V];
      loadUser<IO, V>(in + v * V, nvalid, aligned, x);
      applyScale(x, a.scale);
      const uint4 r = pack<WIRE, V>(x);
#pragma unroll
      for (int k = 0; k < kMaxRanks; ++k)
        if (k < t.M) stStage(stageAt(c.staging[rankOf(t, k, t.d)], bc.half, shard + v), r);
    }
  }
}

// ---------------------------------------------------------------------------
// One-shot phases.  Staging layout of a half: [source rank][chunk][qv].
// ---------------------------------------------------------------------------
template <typename IO, typename WIRE>
__device__ __forceinline__ void phasePushAll(const ChannelDev& c, const OpArgs& a,
                                             const BlockCtx& bc) {
  constexpr int V = kVecBytes / sizeof(WIRE);
  using Acc = typename Tr<IO>::Acc;
  const Topo& t = c.topo;
  const Seg& s = a.seg;
  const IO* in = static_cast<const IO*>(a.in);
  const int W = t.world;
  const int64_t ntiles = ceilDiv(s.qv, kTile);
  for (int chunk = 0; chunk < W; ++chunk) {
    const bool aligned = chunkAligned(in, s, chunk);
    for (int64_t tile = bc.b; tile < ntiles; tile += bc.G) {
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int64_t v = tile * kTile + u * kThreads + threadIdx.x;
        if (v >= s.qv) continue;
        const int nvalid = (int)validInVector(s, chunk, v, V);
        Acc x[V];
        loadUser<IO, V>(in + (int64_t)chunk * s.chunk_stride + v * V, nvalid, aligned, x);
        applyScale(x, a.scale);
        const uint4 r = pack<WIRE, V>(x);
        const int64_t pos = ((int64_t)t.rank * W + chunk) * s.qv + v;
#pragma unroll
        for (int k = 0; k < kMaxRanks; ++k)
          if (k < W) stStage(stageAt(c.staging[(t.rank + k) % W], bc.half, pos), r);
      }
    }
  }
}

template <typename IO, typename WIRE>
__device__ __forceinline__ void phaseReduceAll(const ChannelDev& c, const OpArgs& a,
                                               const BlockCtx& bc) {
  constexpr int V = kVecBytes / sizeof(WIRE);
  using Acc = typename Tr<WIRE>::Acc;
  const Topo& t = c.topo;
  const Seg& s = a.seg;
  IO* out = static_cast<IO*>(a.out);
  char* own = c.staging[t.rank];
  const int W = t.world;
  const int64_t ntiles = ceilDiv(s.qv, kTile);
  for (int chunk = 0; chunk < W; ++chunk) {
    const bool aligned = chunkAligned(out, s, chunk);
    for (int64_t tile = bc.b; tile < ntiles; tile += bc.G) {
      uint4 raw[kU][kMaxRanks];
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int64_t v = tile * kTile + u * kThreads + threadIdx.x;
#pragma unroll
        for (int k = 0; k < kMaxRanks; ++k)
          if (k < W && v < s.qv)
            raw[u][k] = ldStage(stageAt(own, bc.half, ((int64_t)k * W + chunk) * s.qv + v));
      }
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int64_t v = tile * kTile + u * kThreads + threadIdx.x;
        if (v >= s.qv) continue;
        Acc acc[V];
        unpack<WIRE, V>(raw[u][0], acc);
#pragma unroll
        for (int k = 1; k < kMaxRanks; ++k) {
          if (k < W) {
            Acc x[V];
            unpack<WIRE, V>(raw[u][k], x);
#pragma unroll
            for (int i = 0; i < V; ++i) acc[i] = combine(acc[i], x[i], a.op);
          }
        }
        const int nvalid = (int)validInVector(s, chunk, v, V);
        typename Tr<IO>::Acc y[V];
#pragma unroll
        for (int i = 0; i < V; ++i) y[i] = (typename Tr<IO>::Acc)acc[i];
        storeUser<IO, V>(out + (int64_t)chunk * s.chunk_stride + v * V, nvalid, aligned, y);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// NVLS phases.  Staging layout of a half: [chunk][qv], one copy per GPU, all
// copies bound to one multicast object.
// ---------------------------------------------------------------------------
template <typename IO, typename WIRE>
__device__ __forceinline__ void phaseCopyIn(const ChannelDev& c, const OpArgs& a,
                                            const BlockCtx& bc) {
  constexpr int V = kVecBytes / sizeof(WIRE);
  using Acc = typename Tr<IO>::Acc;
  const Topo& t = c.topo;
  const Seg& s = a.seg;
  const IO* in = static_cast<const IO*>(a.in);
  char* own = c.staging[t.rank];
  const int64_t ntiles = ceilDiv(s.qv, kTile);
  for (int chunk = 0; chunk < t.world; ++chunk) {
    const bool aligned = chunkAligned(in, s, chunk);
    for (int64_t tile = bc.b; tile < ntiles; tile += bc.G) {
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int64_t v = tile * kTile + u * kThreads + threadIdx.x;
        if (v >= s.qv) continue;
        const int nvalid = (int)validInVector(s, chunk, v, V);
        Acc x[V];
        loadUser<IO, V>(in + (int64_t)chunk * s.chunk_stride + v * V, nvalid, aligned, x);
        applyScale(x, a.scale);
        stStage(stageAt(own, bc.half, (int64_t)chunk * s.qv + v), pack<WIRE, V>(x));
      }
    }
  }
}

template <typename IO, typename WIRE>
__device__ __forceinline__ void phaseCopyOut(const ChannelDev& c, const OpArgs& a,
                                             const BlockCtx& bc) {
  constexpr int V = kVecBytes / sizeof(WIRE);
  const Topo& t = c.topo;
  const Seg& s = a.seg;
  IO* out = static_cast<IO*>(a.out);
  char* own = c.staging[t.rank];
  const int64_t ntiles = ceilDiv(s.qv, kTile);
  for (int chunk = 0; chunk < t.world; ++chunk) {
    const bool aligned = chunkAligned(out, s, chunk);
    for (int64_t tile = bc.b; tile < ntiles; tile += bc.G) {
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int64_t v = tile * kTile + u * kThreads + threadIdx.x;
        if (v >= s.qv) continue;
        const int nvalid = (int)validInVector(s, chunk, v, V);
        typename Tr<WIRE>::Acc x[V];
        unpack<WIRE, V>(ldStage(stageAt(own, bc.half, (int64_t)chunk * s.qv + v)), x);
        typename Tr<IO>::Acc y[V];
#pragma unroll
        for (int i = 0; i < V; ++i) y[i] = (typename Tr<IO>::Acc)x[i];
        storeUser<IO, V>(out + (int64_t)chunk * s.chunk_stride + v * V, nvalid, aligned, y);
      }
    }
  }
}

// The switch reduces this rank's chunk over all GPUs; the result is multicast
// back into every GPU's staging, in place.
template <typename WIRE>
__device__ __forceinline__ void phaseNvlsReduceBroadcast(const ChannelDev& c, const OpArgs& a,
                                                         const BlockCtx& bc) {
  const Topo& t = c.topo;
  const Seg& s = a.seg;
  const int64_t ntiles = ceilDiv(s.qv, kTile);
  for (int64_t tile = bc.b; tile < ntiles; tile += bc.G) {
    uint4 r[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int64_t v = tile * kTile + u * kThreads + threadIdx.x;
      if (v < s.qv)
        r[u] = multimemLdReduce<WIRE>(stageAt(c.mc_staging, bc.half, (int64_t)t.rank * s.qv + v),
                                      a.op);
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int64_t v = tile * kTile + u * kThreads + threadIdx.x;
      if (v < s.qv) multimemSt(stageAt(c.mc_staging, bc.half, (int64_t)t.rank * s.qv + v), r[u]);
    }
  }
}

// The switch reduces the whole message for this GPU, straight into the output.
template <typename IO, typename WIRE>
__device__ __forceinline__ void phaseNvlsReduceAll(const ChannelDev& c, const OpArgs& a,
                                                   const BlockCtx& bc) {
  constexpr int V = kVecBytes / sizeof(WIRE);
  const Topo& t = c.topo;
  const Seg& s = a.seg;
  IO* out = static_cast<IO*>(a.out);
  const int64_t ntiles = ceilDiv(s.qv, kTile);
  for (int chunk = 0; chunk < t.world; ++chunk) {
    const bool aligned = chunkAligned(out, s, chunk);
    for (int64_t tile = bc.b; tile < ntiles; tile += bc.G) {
      uint4 r[kU];
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int64_t v = tile * kTile + u * kThreads + threadIdx.x;
        if (v < s.qv)
          r[u] = multimemLdReduce<WIRE>(stageAt(c.mc_staging, bc.half, (int64_t)chunk * s.qv + v),
                                        a.op);
      }
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int64_t v = tile * kTile + u * kThreads + threadIdx.x;
        if (v >= s.qv) continue;
        const int nvalid = (int)validInVector(s, chunk, v, V);
        typename Tr<WIRE>::Acc x[V];
        unpack<WIRE, V>(r[u], x);
        typename Tr<IO>::Acc y[V];
#pragma unroll
        for (int i = 0; i < V; ++i) y[i] = (typename Tr<IO>::Acc)x[i];
        storeUser<IO, V>(out + (int64_t)chunk * s.chunk_stride + v * V, nvalid, aligned, y);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Kernel bodies: phase programs.  Barrier indices are fixed per collective so
// that the three hierarchical kernels of one all_reduce share a numbering.
//   0: after the first push / copy-in   (always all ranks)
//   1: shard server start (rail)        2: shard server end (rail)
//   3: gather start (group)
// ---------------------------------------------------------------------------
template <typename IO, typename WIRE, KernelId K>
__device__ __forceinline__ void body(const ChannelDev& c, const OpArgs& a) {
  const BlockCtx bc = enter(c);
  if constexpr (K == KernelId::ONESHOT) {
    phasePushAll<IO, WIRE>(c, a, bc);
    if (barrier<kAll>(c, bc, 0)) phaseReduceAll<IO, WIRE>(c, a, bc);
  } else if constexpr (K == KernelId::TWOSHOT) {
    phasePush<IO, WIRE>(c, a, bc);
    if (barrier<kAll>(c, bc, 0)) {
      phaseLocalReduce<IO, WIRE>(c, a, bc);
      if (barrier<kGroup>(c, bc, 3)) phaseGather<IO, WIRE>(c, a, bc);
    }
  } else if constexpr (K == KernelId::RS_INTRAGROUP) {
    phasePush<IO, WIRE>(c, a, bc);
    if (barrier<kAll>(c, bc, 0)) phaseLocalReduce<IO, WIRE>(c, a, bc);
  } else if constexpr (K == KernelId::SHARD_SERVER_REDUCE) {
    if (barrier<kRail>(c, bc, 1)) {
      phaseServerReduce<IO, WIRE>(c, a, bc);
      if (!(a.flags & kToUser)) barrier<kRail>(c, bc, 2);
    }
  } else if constexpr (K == KernelId::AG_INTRAGROUP) {
    if (barrier<kGroup>(c, bc, 3)) phaseGather<IO, WIRE>(c, a, bc);
  } else if constexpr (K == KernelId::DIFFUSE) {
    phaseDiffuse<IO, WIRE>(c, a, bc);
    barrier<kAll>(c, bc, 0);
  } else if constexpr (K == KernelId::NVLS_TWOSHOT) {
    phaseCopyIn<IO, WIRE>(c, a, bc);
    if (barrier<kAll>(c, bc, 0)) {
      phaseNvlsReduceBroadcast<WIRE>(c, a, bc);
      if (barrier<kAll>(c, bc, 3)) phaseCopyOut<IO, WIRE>(c, a, bc);
    }
  } else if constexpr (K == KernelId::NVLS_ONESHOT) {
    phaseCopyIn<IO, WIRE>(c, a, bc);
    if (barrier<kAll>(c, bc, 0)) phaseNvlsReduceAll<IO, WIRE>(c, a, bc);
  }
  leave(c, a, bc);
}

// One __global__ per kernel id so that profiles show the stage by name.
#define FR_DEFINE_KERNEL(NAME, KID)                                                         \
  template <typename IO, typename WIRE>                                                     \
  __global__ void __launch_bounds__(kThreads, 2)                                            \
      NAME(const __grid_constant__ ChannelDev c, const __grid_constant__ OpArgs a) {        \
    body<IO, WIRE, KID>(c, a);                                                              \
  }                                                                                         \
  template <typename IO, typename WIRE>                                                     \
  __global__ void __launch_bounds__(kThreads, 2)                                            \
      NAME##_emulated(const ChannelDev* cs, const OpArgs* as) {                             \
    body<IO, WIRE, KID>(cs[blockIdx.y], as[blockIdx.y]);                                    \
  }

FR_DEFINE_KERNEL(oneshot_allreduce, KernelId::ONESHOT)
FR_DEFINE_KERNEL(twoshot_allreduce, KernelId::TWOSHOT)
FR_DEFINE_KERNEL(rs_intragroup, KernelId::RS_INTRAGROUP)
FR_DEFINE_KERNEL(shard_server_reduce, KernelId::SHARD_SERVER_REDUCE)
FR_DEFINE_KERNEL(ag_intragroup, KernelId::AG_INTRAGROUP)
FR_DEFINE_KERNEL(diffuse_rail, KernelId::DIFFUSE)
FR_DEFINE_KERNEL(nvls_allreduce, KernelId::NVLS_TWOSHOT)
FR_DEFINE_KERNEL(nvls_oneshot_allreduce, KernelId::NVLS_ONESHOT)

using RealFn = void (*)(const ChannelDev, const OpArgs);
using EmulFn = void (*)(const ChannelDev*, const OpArgs*);

template <typename IO, typename WIRE>
RealFn realFn(KernelId id) {
  switch (id) {
    case KernelId::ONESHOT: return oneshot_allreduce<IO, WIRE>;
    case KernelId::TWOSHOT: return twoshot_allreduce<IO, WIRE>;
    case KernelId::RS_INTRAGROUP: return rs_intragroup<IO, WIRE>;
    case KernelId::SHARD_SERVER_REDUCE: return shard_server_reduce<IO, WIRE>;
    case KernelId::AG_INTRAGROUP: return ag_intragroup<IO, WIRE>;
    case KernelId::DIFFUSE: return diffuse_rail<IO, WIRE>;
    case KernelId::NVLS_TWOSHOT:
      if constexpr (std::is_floating_point<typename Tr<WIRE>::Acc>::value && sizeof(WIRE) <= 4)
        return nvls_allreduce<IO, WIRE>;
      return nullptr;
    case KernelId::NVLS_ONESHOT:
      if constexpr (std::is_floating_point<typename Tr<WIRE>::Acc>::value && sizeof(WIRE) <= 4)
        return nvls_oneshot_allreduce<IO, WIRE>;
      return nullptr;
    default: return nullptr;
  }
}
template <typename IO, typename WIRE>
EmulFn emulFn(KernelId id) {
  switch (id) {
    case KernelId::ONESHOT: return oneshot_allreduce_emulated<IO, WIRE>;
    case KernelId::TWOSHOT: return twoshot_allreduce_emulated<IO, WIRE>;
    case KernelId::RS_INTRAGROUP: return rs_intragroup_emulated<IO, WIRE>;
    case KernelId::SHARD_SERVER_REDUCE: return shard_server_reduce_emulated<IO, WIRE>;
    case KernelId::AG_INTRAGROUP: return ag_intragroup_emulated<IO, WIRE>;
    case KernelId::DIFFUSE: return diffuse_rail_emulated<IO, WIRE>;
    default: return nullptr;  // multicast needs one GPU per rank
  }
}

#define FR_COMBO(IO_E, WIRE_E, IO_T, WIRE_T) \
  if (io == DType::IO_E && wire == DType::WIRE_E) return FN<IO_T, WIRE_T>(id);

#define FR_ALL_COMBOS                                   \
  FR_COMBO(U8, U8, uint8_t, uint8_t)                    \
  FR_COMBO(I8, I8, int8_t, int8_t)                      \
  FR_COMBO(I32, I32, int32_t, int32_t)                  \
  FR_COMBO(I64, I64, int64_t, int64_t)                  \
  FR_COMBO(F16, F16, __half, __half)                    \
  FR_COMBO(BF16, BF16, __nv_bfloat16, __nv_bfloat16)    \
  FR_COMBO(F32, F32, float, float)                      \
  FR_COMBO(F64, F64, double, double)                    \
  FR_COMBO(F32, BF16, float, __nv_bfloat16)             \
  FR_COMBO(F32, F16, float, __half)

RealFn lookupReal(DType io, DType wire, KernelId id) {
#define FN realFn
  FR_ALL_COMBOS
#undef FN
  return nullptr;
}
EmulFn lookupEmul(DType io, DType wire, KernelId id) {
#define FN emulFn
  FR_ALL_COMBOS
#undef FN
  return nullptr;
}

std::atomic<uint64_t> g_launches{0};

}  // namespace

const char* kernelName(KernelId id) {
  switch (id) {
    case KernelId::ONESHOT: return "oneshot_allreduce";
    case KernelId::TWOSHOT: return "twoshot_allreduce";
    case KernelId::RS_INTRAGROUP: return "rs_intragroup";
    case KernelId::SHARD_SERVER_REDUCE: return "shard_server_reduce";
    case KernelId::AG_INTRAGROUP: return "ag_intragroup";
    case KernelId::DIFFUSE: return "diffuse_rail";
    case KernelId::NVLS_TWOSHOT: return "nvls_allreduce";
    case KernelId::NVLS_ONESHOT: return "nvls_oneshot_allreduce";
    default: return "?";
  }
}

bool comboSupported(DType io, DType wire) {
  if (io == wire) return (int)io >= 0 && (int)io < (int)DType::kCount;
  return io == DType::F32 && (wire == DType::BF16 || wire == DType::F16);
}

bool nvlsSupported(DType wire, RedOp op) {
  if (wire == DType::F32) return op == RedOp::SUM;
  return wire == DType::BF16 || wire == DType::F16;
}

cudaError_t launchCollective(KernelId id, const ChannelDev& ch, const OpArgs& args, int blocks,
                             cudaStream_t stream) {
  if (blocks < 1 || blocks > kMaxBlocks) return cudaErrorInvalidValue;
  RealFn fn = lookupReal((DType)args.io_dtype, (DType)args.wire_dtype, id);
  if (fn == nullptr) return cudaErrorInvalidDeviceFunction;
  if ((id == KernelId::NVLS_TWOSHOT || id == KernelId::NVLS_ONESHOT) &&
      (ch.mc_staging == nullptr ||
       !nvlsSupported((DType)args.wire_dtype, (RedOp)args.op)))
    return cudaErrorInvalidValue;
  fn<<<dim3(blocks), dim3(kThreads), 0, stream>>>(ch, args);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError();
}

cudaError_t launchEmulated(KernelId id, const ChannelDev* chs, const OpArgs* args, int world,
                           int blocks, cudaStream_t stream) {
  if (blocks < 1 || blocks > kMaxBlocks || world < 1 || world > kMaxRanks)
    return cudaErrorInvalidValue;
  // The host mirrors are only needed to pick the instantiation.
  OpArgs a0;
  cudaError_t e = cudaMemcpyAsync(&a0, args, sizeof(OpArgs), cudaMemcpyDeviceToHost, stream);
  if (e != cudaSuccess) return e;
  e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return e;
  EmulFn fn = lookupEmul((DType)a0.io_dtype, (DType)a0.wire_dtype, id);
  if (fn == nullptr) return cudaErrorInvalidDeviceFunction;
  void* params[] = {(void*)&chs, (void*)&args};
  // Cooperative: all blocks of all emulated ranks must be resident at once,
  // because they wait on one another.
  e = cudaLaunchCooperativeKernel((const void*)fn, dim3(blocks, world), dim3(kThreads), params, 0,
                                  stream);
  if (e == cudaSuccess) g_launches.fetch_add(1, std::memory_order_relaxed);
  return e;
}

uint64_t launchCount() { return g_launches.load(std::memory_order_relaxed); }

}  // namespace fairring
