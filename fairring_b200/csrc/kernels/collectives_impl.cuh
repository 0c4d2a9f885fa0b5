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

#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "device_prims.cuh"
#include "kernels.h"

namespace fairring {
namespace impl {

using namespace dev;


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
  // Arrive: ONE system-scope fence for the whole block (its writes reached
  // thread 0 through the __syncthreads above), then a relaxed store per peer
  // by that same thread.  A fence and a release-store in each of n threads is
  // 2n system-scope membars that an SM works off one after the other.
  if (threadIdx.x == 0) {
    __threadfence_system();
    for (int i = 0; i < n; ++i) {
      const int q = KIND == kAll ? i : (KIND == kGroup ? rankOf(t, t.m, i) : rankOf(t, i, t.d));
      if (q != t.rank) stRelaxedSys(c.flags[q] + t.rank * kMaxBlocks + bc.b, epoch);
    }
  }
  uint32_t st = kStatusOk;
  int peer = -1;
  if ((int)threadIdx.x < n) {
    const int i = threadIdx.x;
    peer = KIND == kAll ? i : (KIND == kGroup ? rankOf(t, t.m, i) : rankOf(t, i, t.d));
    if (peer != t.rank) {
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
  if (a.flags & kAdvanceSeq) {
    if (threadIdx.x == 0) c.seq[bc.b] = bc.seq + 1u;
    // A launch narrower than the channel's grid: block 0 keeps the counts of the
    // blocks that did not run in step (all counts of a channel are equal between
    // kernels, and nothing else runs on the channel's stream meanwhile).
    if (bc.b == 0)
      for (int b = bc.G + (int)threadIdx.x; b < a.full_blocks; b += (int)blockDim.x) c.seq[b] = bc.seq + 1u;
  }
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
// Work split.  A chunk of qv vectors is cut into tiles of kThreads vectors;
// block b owns tiles b, b+G, b+2G, ...  A thread works on U of its block's
// tiles at a time so that U (times the number of peers) 16-byte accesses are
// in flight per thread; U differs between phases, ownership never does.
// ---------------------------------------------------------------------------
template <int U>
struct Batch {
  int64_t v[U];
  bool ok[U];
};
template <int U>
__device__ __forceinline__ Batch<U> batchAt(int64_t tile0, const BlockCtx& bc, int64_t ntiles,
                                            int64_t qv) {
  Batch<U> t;
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const int64_t tile = tile0 + (int64_t)u * bc.G;
    t.v[u] = tile * kThreads + threadIdx.x;
    t.ok[u] = tile < ntiles && t.v[u] < qv;
  }
  return t;
}

// Pick the unroll U and the static bound KP on the number of peers so that a
// batch keeps at most 16 sixteen-byte words live: `peers` accesses per vector,
// `nv` words per access.
#define FR_WITH_UNROLL(peers, nv, ...)          \
  do {                                          \
    if ((peers) * (nv) <= 4) {                  \
      constexpr int U = 4;                      \
      constexpr int KP = 4 / (nv);              \
      __VA_ARGS__;                              \
    } else if ((peers) * (nv) <= 8) {           \
      constexpr int U = 2;                      \
      constexpr int KP = 8 / (nv);              \
      __VA_ARGS__;                              \
    } else {                                    \
      constexpr int U = 1;                      \
      constexpr int KP = kMaxRanks;             \
      __VA_ARGS__;                              \
    }                                           \
  } while (0)

// V elements of the user's tensor.  When the vector is whole and 16-byte
// aligned ("fast") its raw words are loaded first and converted after all
// loads of the batch have been issued; otherwise it is read element by element
// at conversion time.  Only the raw words stay live across the batch.
template <typename IO, int V>
struct UserRaw {
  uint4 w[V * sizeof(IO) / 16];
};
template <typename IO, int V>
__device__ __forceinline__ void userIssue(UserRaw<IO, V>& r, const IO* p, bool fast) {
  if (fast) {
#pragma unroll
    for (int k = 0; k < (int)(V * sizeof(IO) / 16); ++k) r.w[k] = reinterpret_cast<const uint4*>(p)[k];
  }
}
template <typename IO, int V>
__device__ __forceinline__ void userFinish(const UserRaw<IO, V>& r, const IO* p, int nvalid,
                                           bool fast, typename Tr<IO>::Acc (&x)[V]) {
  if (fast) {
    const IO* e = reinterpret_cast<const IO*>(r.w);
#pragma unroll
    for (int i = 0; i < V; ++i) x[i] = Tr<IO>::up(e[i]);
  } else {
#pragma unroll
    for (int i = 0; i < V; ++i) x[i] = i < nvalid ? Tr<IO>::up(p[i]) : typename Tr<IO>::Acc(0);
  }
}

template <typename IO, typename WIRE, int V>
__device__ __forceinline__ void storeUserFromWire(IO* p, int nvalid, bool aligned, const uint4& w) {
  typename Tr<WIRE>::Acc x[V];
  unpack<WIRE, V>(w, x);
  typename Tr<IO>::Acc y[V];
#pragma unroll
  for (int i = 0; i < V; ++i) y[i] = (typename Tr<IO>::Acc)x[i];
  storeUser<IO, V>(p, nvalid, aligned, y);
}

// ---------------------------------------------------------------------------
// Phase: push.  Read the user's input once and store rail chunk j destined to
// group member d' into slot d of that member's staging (scaled, cast to the
// wire type).  With M == 1 this is "chunk p goes to rank p".
// ---------------------------------------------------------------------------
template <typename IO, typename WIRE, int U, int KP>
__device__ __forceinline__ void phasePushU(const ChannelDev& c, const OpArgs& a,
                                           const BlockCtx& bc) {
  constexpr int V = kVecBytes / sizeof(WIRE);
  using Acc = typename Tr<IO>::Acc;
  const Topo& t = c.topo;
  const Seg& s = a.seg;
  const IO* in = static_cast<const IO*>(a.in[blockIdx.y]);
  const int64_t ntiles = ceilDiv(s.qv, kThreads);
  for (int j = 0; j < t.M; ++j) {
    for (int64_t tile0 = bc.b; tile0 < ntiles; tile0 += (int64_t)bc.G * U) {
      const Batch<U> tb = batchAt<U>(tile0, bc, ntiles, s.qv);
      UserRaw<IO, V> raw[U][KP];
#pragma unroll
      for (int u = 0; u < U; ++u) {
#pragma unroll
        for (int k = 0; k < KP; ++k) {
          if (k < t.D && tb.ok[u]) {
            const int dd = (t.d + 1 + k) % t.D;  // start at the neighbour: spreads the links
            const int chunk = rankOf(t, j, dd);
            const bool fast = chunkAligned(in, s, chunk) && validInVector(s, chunk, tb.v[u], V) == V;
            userIssue<IO, V>(raw[u][k], in + (int64_t)chunk * s.chunk_stride + tb.v[u] * V, fast);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
#pragma unroll
        for (int k = 0; k < KP; ++k) {
          if (k < t.D && tb.ok[u]) {
            const int dd = (t.d + 1 + k) % t.D;
            const int chunk = rankOf(t, j, dd);
            const int nvalid = (int)validInVector(s, chunk, tb.v[u], V);
            const bool fast = chunkAligned(in, s, chunk) && nvalid == V;
            Acc x[V];
            userFinish<IO, V>(raw[u][k], in + (int64_t)chunk * s.chunk_stride + tb.v[u] * V, nvalid,
                              fast, x);
            applyScale(x, a.scale);
            stStage(stageAt(c.staging[rankOf(t, t.m, dd)], bc.half,
                            stagingVec(t, s, t.d, j) + tb.v[u]),
                    pack<WIRE, V>(x));
          }
        }
      }
    }
  }
}
template <typename IO, typename WIRE>
__device__ __forceinline__ void phasePush(const ChannelDev& c, const OpArgs& a,
                                          const BlockCtx& bc) {
  constexpr int NV = sizeof(IO) / sizeof(WIRE);  // 16-byte loads per vector
  FR_WITH_UNROLL(c.topo.D, NV, phasePushU<IO, WIRE, U, KP>(c, a, bc));
}

// ---------------------------------------------------------------------------
// Phase: local reduce.  Sum (or max/min) the D source slots of this GPU's own
// staging, in slot order so that the result does not depend on timing; write
// the self slot, or the user's output for a flat reduce_scatter.
// ---------------------------------------------------------------------------
template <typename IO, typename WIRE, int U, int KP>
__device__ __forceinline__ void phaseLocalReduceU(const ChannelDev& c, const OpArgs& a,
                                                  const BlockCtx& bc) {
  constexpr int V = kVecBytes / sizeof(WIRE);
  using Acc = typename Tr<WIRE>::Acc;
  const Topo& t = c.topo;
  const Seg& s = a.seg;
  char* own = c.staging[t.rank];
  const bool to_user = (a.flags & kToUser) != 0;
  IO* out = static_cast<IO*>(a.out[blockIdx.y]);
  const int64_t ntiles = ceilDiv(s.qv, kThreads);
  for (int j = 0; j < t.M; ++j) {
    for (int64_t tile0 = bc.b; tile0 < ntiles; tile0 += (int64_t)bc.G * U) {
      const Batch<U> tb = batchAt<U>(tile0, bc, ntiles, s.qv);
      uint4 raw[U][KP];
#pragma unroll
      for (int u = 0; u < U; ++u) {
#pragma unroll
        for (int k = 0; k < KP; ++k)
          if (k < t.D && tb.ok[u])
            raw[u][k] = ldStage(stageAt(own, bc.half, stagingVec(t, s, k, j) + tb.v[u]));
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (!tb.ok[u]) continue;
        Acc acc[V];
        unpack<WIRE, V>(raw[u][0], acc);
#pragma unroll
        for (int k = 1; k < KP; ++k) {
          if (k < t.D) {
            Acc x[V];
            unpack<WIRE, V>(raw[u][k], x);
#pragma unroll
            for (int i = 0; i < V; ++i) acc[i] = combine(acc[i], x[i], a.op);
          }
        }
        const uint4 r = pack<WIRE, V>(acc);
        if (to_user) {
          // Flat reduce_scatter: this rank's chunk is its whole output.
          const int chunk = rankOf(t, j, t.d);
          storeUserFromWire<IO, WIRE, V>(out + tb.v[u] * V, (int)validInVector(s, chunk, tb.v[u], V),
                                         (reinterpret_cast<uintptr_t>(out) & 15u) == 0, r);
        } else {
          stStage(stageAt(own, bc.half, stagingVec(t, s, t.d, j) + tb.v[u]), r);
        }
      }
    }
  }
}
template <typename IO, typename WIRE>
__device__ __forceinline__ void phaseLocalReduce(const ChannelDev& c, const OpArgs& a,
                                                 const BlockCtx& bc) {
  FR_WITH_UNROLL(c.topo.D, 1, phaseLocalReduceU<IO, WIRE, U, KP>(c, a, bc));
}

// ---------------------------------------------------------------------------
// Phase: shard-server reduce.  This GPU serves shard (d, m): pull the group
// partial sums of that shard from the self slot of each rail peer (machine
// order), reduce in registers, then either push the result back into every
// rail peer's self slot (all_reduce: collect + add + diffuse in one pass) or
// write the user's output (reduce_scatter).
// ---------------------------------------------------------------------------
template <typename IO, typename WIRE, int U, int KP>
__device__ __forceinline__ void phaseServerReduceU(const ChannelDev& c, const OpArgs& a,
                                                   const BlockCtx& bc) {
  constexpr int V = kVecBytes / sizeof(WIRE);
  using Acc = typename Tr<WIRE>::Acc;
  const Topo& t = c.topo;
  const Seg& s = a.seg;
  const bool to_user = (a.flags & kToUser) != 0;
  IO* out = static_cast<IO*>(a.out[blockIdx.y]);
  const int64_t shard = stagingVec(t, s, t.d, t.m);
  const int64_t ntiles = ceilDiv(s.qv, kThreads);
  for (int64_t tile0 = bc.b; tile0 < ntiles; tile0 += (int64_t)bc.G * U) {
    const Batch<U> tb = batchAt<U>(tile0, bc, ntiles, s.qv);
    uint4 raw[U][KP];
#pragma unroll
    for (int u = 0; u < U; ++u) {
#pragma unroll
      for (int k = 0; k < KP; ++k)
        if (k < t.M && tb.ok[u])
          raw[u][k] = ldStage(stageAt(c.staging[rankOf(t, k, t.d)], bc.half, shard + tb.v[u]));
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (!tb.ok[u]) continue;
      Acc acc[V];
      unpack<WIRE, V>(raw[u][0], acc);
#pragma unroll
      for (int k = 1; k < KP; ++k) {
        if (k < t.M) {
          Acc x[V];
          unpack<WIRE, V>(raw[u][k], x);
#pragma unroll
          for (int i = 0; i < V; ++i) acc[i] = combine(acc[i], x[i], a.op);
        }
      }
      const uint4 r = pack<WIRE, V>(acc);
      if (to_user) {
        storeUserFromWire<IO, WIRE, V>(out + tb.v[u] * V, (int)validInVector(s, t.rank, tb.v[u], V),
                                       (reinterpret_cast<uintptr_t>(out) & 15u) == 0, r);
      } else {
#pragma unroll
        for (int k = 0; k < KP; ++k)
          if (k < t.M) stStage(stageAt(c.staging[rankOf(t, k, t.d)], bc.half, shard + tb.v[u]), r);
      }
    }
  }
}
template <typename IO, typename WIRE>
__device__ __forceinline__ void phaseServerReduce(const ChannelDev& c, const OpArgs& a,
                                                  const BlockCtx& bc) {
  FR_WITH_UNROLL(c.topo.M, 1, phaseServerReduceU<IO, WIRE, U, KP>(c, a, bc));
}

// ---------------------------------------------------------------------------
// Phase: gather.  Pull the reduced rail chunks from the self slot of every
// group member and write them (cast back) into the user's output.
// ---------------------------------------------------------------------------
template <typename IO, typename WIRE, int U, int KP>
__device__ __forceinline__ void phaseGatherU(const ChannelDev& c, const OpArgs& a,
                                             const BlockCtx& bc) {
  constexpr int V = kVecBytes / sizeof(WIRE);
  const Topo& t = c.topo;
  const Seg& s = a.seg;
  IO* out = static_cast<IO*>(a.out[blockIdx.y]);
  const int64_t ntiles = ceilDiv(s.qv, kThreads);
  for (int j = 0; j < t.M; ++j) {
    for (int64_t tile0 = bc.b; tile0 < ntiles; tile0 += (int64_t)bc.G * U) {
      const Batch<U> tb = batchAt<U>(tile0, bc, ntiles, s.qv);
      uint4 raw[U][KP];
#pragma unroll
      for (int u = 0; u < U; ++u) {
#pragma unroll
        for (int k = 0; k < KP; ++k) {
          if (k < t.D && tb.ok[u]) {
            const int dd = (t.d + k) % t.D;
            raw[u][k] = ldStage(stageAt(c.staging[rankOf(t, t.m, dd)], bc.half,
                                        stagingVec(t, s, dd, j) + tb.v[u]));
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
#pragma unroll
        for (int k = 0; k < KP; ++k) {
          if (k < t.D && tb.ok[u]) {
            const int dd = (t.d + k) % t.D;
            const int chunk = rankOf(t, j, dd);
            storeUserFromWire<IO, WIRE, V>(out + (int64_t)chunk * s.chunk_stride + tb.v[u] * V,
                                           (int)validInVector(s, chunk, tb.v[u], V),
                                           chunkAligned(out, s, chunk), raw[u][k]);
          }
        }
      }
    }
  }
}
template <typename IO, typename WIRE>
__device__ __forceinline__ void phaseGather(const ChannelDev& c, const OpArgs& a,
                                            const BlockCtx& bc) {
  FR_WITH_UNROLL(c.topo.D, 1, phaseGatherU<IO, WIRE, U, KP>(c, a, bc));
}

// ---------------------------------------------------------------------------
// Phase: diffuse (all_gather stage 1).  The user's input is this rank's chunk;
// store it into the self slot, rail position m, of every rail peer (self
// included).  Afterwards every GPU's self slot holds its whole rail.
// ---------------------------------------------------------------------------
template <typename IO, typename WIRE, int U>
__device__ __forceinline__ void phaseDiffuseU(const ChannelDev& c, const OpArgs& a,
                                              const BlockCtx& bc) {
  constexpr int V = kVecBytes / sizeof(WIRE);
  using Acc = typename Tr<IO>::Acc;
  const Topo& t = c.topo;
  const Seg& s = a.seg;
  const IO* in = static_cast<const IO*>(a.in[blockIdx.y]);
  const bool aligned = (reinterpret_cast<uintptr_t>(in) & 15u) == 0;
  const int64_t shard = stagingVec(t, s, t.d, t.m);
  const int64_t ntiles = ceilDiv(s.qv, kThreads);
  for (int64_t tile0 = bc.b; tile0 < ntiles; tile0 += (int64_t)bc.G * U) {
    const Batch<U> tb = batchAt<U>(tile0, bc, ntiles, s.qv);
    UserRaw<IO, V> raw[U];
    auto validAt = [&](int64_t v) {
      const int64_t nv = s.chunk_len - v * V;
      return nv > V ? V : (nv < 0 ? 0 : (int)nv);
    };
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (tb.ok[u]) userIssue<IO, V>(raw[u], in + tb.v[u] * V, aligned && validAt(tb.v[u]) == V);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (!tb.ok[u]) continue;
      const int nvalid = validAt(tb.v[u]);
      Acc x[V];
      userFinish<IO, V>(raw[u], in + tb.v[u] * V, nvalid, aligned && nvalid == V, x);
      applyScale(x, a.scale);
      const uint4 r = pack<WIRE, V>(x);
#pragma unroll
      for (int k = 0; k < kMaxRanks; ++k)
        if (k < t.M) stStage(stageAt(c.staging[rankOf(t, k, t.d)], bc.half, shard + tb.v[u]), r);
    }
  }
}
template <typename IO, typename WIRE>
__device__ __forceinline__ void phaseDiffuse(const ChannelDev& c, const OpArgs& a,
                                             const BlockCtx& bc) {
  constexpr int NV = sizeof(IO) / sizeof(WIRE);
  phaseDiffuseU<IO, WIRE, 4 / NV>(c, a, bc);
}

// ---------------------------------------------------------------------------
// One-shot phases.  Staging layout of a half: [source rank][chunk][qv].
// ---------------------------------------------------------------------------
template <typename IO, typename WIRE, int U>
__device__ __forceinline__ void phasePushAllU(const ChannelDev& c, const OpArgs& a,
                                              const BlockCtx& bc) {
  constexpr int V = kVecBytes / sizeof(WIRE);
  using Acc = typename Tr<IO>::Acc;
  const Topo& t = c.topo;
  const Seg& s = a.seg;
  const IO* in = static_cast<const IO*>(a.in[blockIdx.y]);
  const int W = t.world;
  const int64_t ntiles = ceilDiv(s.qv, kThreads);
  for (int chunk = 0; chunk < W; ++chunk) {
    const bool aligned = chunkAligned(in, s, chunk);
    for (int64_t tile0 = bc.b; tile0 < ntiles; tile0 += (int64_t)bc.G * U) {
      const Batch<U> tb = batchAt<U>(tile0, bc, ntiles, s.qv);
      UserRaw<IO, V> raw[U];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (tb.ok[u])
          userIssue<IO, V>(raw[u], in + (int64_t)chunk * s.chunk_stride + tb.v[u] * V,
                           aligned && validInVector(s, chunk, tb.v[u], V) == V);
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (!tb.ok[u]) continue;
        const int nvalid = (int)validInVector(s, chunk, tb.v[u], V);
        Acc x[V];
        userFinish<IO, V>(raw[u], in + (int64_t)chunk * s.chunk_stride + tb.v[u] * V, nvalid,
                          aligned && nvalid == V, x);
        applyScale(x, a.scale);
        const uint4 r = pack<WIRE, V>(x);
        const int64_t pos = ((int64_t)t.rank * W + chunk) * s.qv + tb.v[u];
#pragma unroll
        for (int k = 0; k < kMaxRanks; ++k)
          if (k < W) stStage(stageAt(c.staging[(t.rank + k) % W], bc.half, pos), r);
      }
    }
  }
}
template <typename IO, typename WIRE>
__device__ __forceinline__ void phasePushAll(const ChannelDev& c, const OpArgs& a,
                                             const BlockCtx& bc) {
  constexpr int NV = sizeof(IO) / sizeof(WIRE);
  phasePushAllU<IO, WIRE, 4 / NV>(c, a, bc);
}

template <typename IO, typename WIRE, int U, int KP>
__device__ __forceinline__ void phaseReduceAllU(const ChannelDev& c, const OpArgs& a,
                                                const BlockCtx& bc) {
  constexpr int V = kVecBytes / sizeof(WIRE);
  using Acc = typename Tr<WIRE>::Acc;
  const Topo& t = c.topo;
  const Seg& s = a.seg;
  IO* out = static_cast<IO*>(a.out[blockIdx.y]);
  char* own = c.staging[t.rank];
  const int W = t.world;
  const int64_t ntiles = ceilDiv(s.qv, kThreads);
  for (int chunk = 0; chunk < W; ++chunk) {
    const bool aligned = chunkAligned(out, s, chunk);
    for (int64_t tile0 = bc.b; tile0 < ntiles; tile0 += (int64_t)bc.G * U) {
      const Batch<U> tb = batchAt<U>(tile0, bc, ntiles, s.qv);
      uint4 raw[U][KP];
#pragma unroll
      for (int u = 0; u < U; ++u) {
#pragma unroll
        for (int k = 0; k < KP; ++k)
          if (k < W && tb.ok[u])
            raw[u][k] = ldStage(stageAt(own, bc.half, ((int64_t)k * W + chunk) * s.qv + tb.v[u]));
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (!tb.ok[u]) continue;
        Acc acc[V];
        unpack<WIRE, V>(raw[u][0], acc);
#pragma unroll
        for (int k = 1; k < KP; ++k) {
          if (k < W) {
            Acc x[V];
            unpack<WIRE, V>(raw[u][k], x);
#pragma unroll
            for (int i = 0; i < V; ++i) acc[i] = combine(acc[i], x[i], a.op);
          }
        }
        storeUserFromWire<IO, WIRE, V>(out + (int64_t)chunk * s.chunk_stride + tb.v[u] * V,
                                       (int)validInVector(s, chunk, tb.v[u], V), aligned,
                                       pack<WIRE, V>(acc));
      }
    }
  }
}
template <typename IO, typename WIRE>
__device__ __forceinline__ void phaseReduceAll(const ChannelDev& c, const OpArgs& a,
                                               const BlockCtx& bc) {
  FR_WITH_UNROLL(c.topo.world, 1, phaseReduceAllU<IO, WIRE, U, KP>(c, a, bc));
}

// ---------------------------------------------------------------------------
// NVLS phases.  Staging layout of a half: [chunk][qv], one copy per GPU, all
// copies bound to one multicast object.
// ---------------------------------------------------------------------------
template <typename IO, typename WIRE, int U>
__device__ __forceinline__ void phaseCopyInU(const ChannelDev& c, const OpArgs& a,
                                             const BlockCtx& bc) {
  constexpr int V = kVecBytes / sizeof(WIRE);
  using Acc = typename Tr<IO>::Acc;
  const Topo& t = c.topo;
  const Seg& s = a.seg;
  const IO* in = static_cast<const IO*>(a.in[blockIdx.y]);
  char* own = c.staging[t.rank];
  const int64_t ntiles = ceilDiv(s.qv, kThreads);
  for (int chunk = 0; chunk < t.world; ++chunk) {
    const bool aligned = chunkAligned(in, s, chunk);
    for (int64_t tile0 = bc.b; tile0 < ntiles; tile0 += (int64_t)bc.G * U) {
      const Batch<U> tb = batchAt<U>(tile0, bc, ntiles, s.qv);
      UserRaw<IO, V> raw[U];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (tb.ok[u])
          userIssue<IO, V>(raw[u], in + (int64_t)chunk * s.chunk_stride + tb.v[u] * V,
                           aligned && validInVector(s, chunk, tb.v[u], V) == V);
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (!tb.ok[u]) continue;
        const int nvalid = (int)validInVector(s, chunk, tb.v[u], V);
        Acc x[V];
        userFinish<IO, V>(raw[u], in + (int64_t)chunk * s.chunk_stride + tb.v[u] * V, nvalid,
                          aligned && nvalid == V, x);
        applyScale(x, a.scale);
        stStage(stageAt(own, bc.half, (int64_t)chunk * s.qv + tb.v[u]), pack<WIRE, V>(x));
      }
    }
  }
}
template <typename IO, typename WIRE>
__device__ __forceinline__ void phaseCopyIn(const ChannelDev& c, const OpArgs& a,
                                            const BlockCtx& bc) {
  constexpr int NV = sizeof(IO) / sizeof(WIRE);
  phaseCopyInU<IO, WIRE, 4 / NV>(c, a, bc);
}

template <typename IO, typename WIRE>
__device__ __forceinline__ void phaseCopyOut(const ChannelDev& c, const OpArgs& a,
                                             const BlockCtx& bc) {
  constexpr int V = kVecBytes / sizeof(WIRE);
  constexpr int U = 4;
  const Topo& t = c.topo;
  const Seg& s = a.seg;
  IO* out = static_cast<IO*>(a.out[blockIdx.y]);
  char* own = c.staging[t.rank];
  const int64_t ntiles = ceilDiv(s.qv, kThreads);
  for (int chunk = 0; chunk < t.world; ++chunk) {
    const bool aligned = chunkAligned(out, s, chunk);
    for (int64_t tile0 = bc.b; tile0 < ntiles; tile0 += (int64_t)bc.G * U) {
      const Batch<U> tb = batchAt<U>(tile0, bc, ntiles, s.qv);
      uint4 raw[U];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (tb.ok[u]) raw[u] = ldStage(stageAt(own, bc.half, (int64_t)chunk * s.qv + tb.v[u]));
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (tb.ok[u])
          storeUserFromWire<IO, WIRE, V>(out + (int64_t)chunk * s.chunk_stride + tb.v[u] * V,
                                         (int)validInVector(s, chunk, tb.v[u], V), aligned, raw[u]);
    }
  }
}

// The switch reduces this rank's chunk over all GPUs; the result is multicast
// back into every GPU's staging, in place.
template <typename WIRE>
__device__ __forceinline__ void phaseNvlsReduceBroadcast(const ChannelDev& c, const OpArgs& a,
                                                         const BlockCtx& bc) {
  constexpr int U = 4;
  const Topo& t = c.topo;
  const Seg& s = a.seg;
  const int64_t ntiles = ceilDiv(s.qv, kThreads);
  for (int64_t tile0 = bc.b; tile0 < ntiles; tile0 += (int64_t)bc.G * U) {
    const Batch<U> tb = batchAt<U>(tile0, bc, ntiles, s.qv);
    uint4 r[U];
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (tb.ok[u])
        r[u] = multimemLdReduce<WIRE>(
            stageAt(c.mc_staging, bc.half, (int64_t)t.rank * s.qv + tb.v[u]), a.op);
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (tb.ok[u])
        multimemSt(stageAt(c.mc_staging, bc.half, (int64_t)t.rank * s.qv + tb.v[u]), r[u]);
  }
}

// The switch reduces the whole message for this GPU, straight into the output.
template <typename IO, typename WIRE>
__device__ __forceinline__ void phaseNvlsReduceAll(const ChannelDev& c, const OpArgs& a,
                                                   const BlockCtx& bc) {
  constexpr int V = kVecBytes / sizeof(WIRE);
  constexpr int U = 4;
  const Topo& t = c.topo;
  const Seg& s = a.seg;
  IO* out = static_cast<IO*>(a.out[blockIdx.y]);
  const int64_t ntiles = ceilDiv(s.qv, kThreads);
  for (int chunk = 0; chunk < t.world; ++chunk) {
    const bool aligned = chunkAligned(out, s, chunk);
    for (int64_t tile0 = bc.b; tile0 < ntiles; tile0 += (int64_t)bc.G * U) {
      const Batch<U> tb = batchAt<U>(tile0, bc, ntiles, s.qv);
      uint4 r[U];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (tb.ok[u])
          r[u] = multimemLdReduce<WIRE>(
              stageAt(c.mc_staging, bc.half, (int64_t)chunk * s.qv + tb.v[u]), a.op);
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (tb.ok[u])
          storeUserFromWire<IO, WIRE, V>(out + (int64_t)chunk * s.chunk_stride + tb.v[u] * V,
                                         (int)validInVector(s, chunk, tb.v[u], V), aligned, r[u]);
    }
  }
}

// ---------------------------------------------------------------------------
// Direct phases: the tensor itself is symmetric memory, nothing is staged.
// The slice is W chunks of qv vectors (whole vectors only: the engine takes
// this path for 16-byte aligned slices whose length is a multiple of 16 bytes).
// Rank r owns chunk r: it reads chunk r of every rank's tensor, reduces, scales
// and writes the result into chunk r of every rank's tensor.  Vector v of chunk
// r is read and then written by the same thread, and no other rank touches
// chunk r, so the update is safe in place.
// ---------------------------------------------------------------------------
template <typename WIRE, int U, int KP>
__device__ __forceinline__ void phaseDirectPeerU(const ChannelDev& c, const OpArgs& a,
                                                 const BlockCtx& bc) {
  constexpr int V = kVecBytes / sizeof(WIRE);
  using Acc = typename Tr<WIRE>::Acc;
  const Topo& t = c.topo;
  const Seg& s = a.seg;
  const int W = t.world;
  const int64_t nvec = ceilDiv(s.limit, V);
  const int64_t base = (int64_t)t.rank * s.qv;
  int64_t mine = nvec - base;
  if (mine > s.qv) mine = s.qv;
  if (mine < 0) mine = 0;
  const int64_t ntiles = ceilDiv(mine, kThreads);
  for (int64_t tile0 = bc.b; tile0 < ntiles; tile0 += (int64_t)bc.G * U) {
    const Batch<U> tb = batchAt<U>(tile0, bc, ntiles, mine);
    uint4 raw[U][KP];
#pragma unroll
    for (int u = 0; u < U; ++u) {
#pragma unroll
      for (int k = 0; k < KP; ++k)
        if (k < W && tb.ok[u])
          raw[u][k] = ldStage(static_cast<char*>(a.peer[k]) + (base + tb.v[u]) * kVecBytes);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (!tb.ok[u]) continue;
      Acc acc[V];
      unpack<WIRE, V>(raw[u][0], acc);
#pragma unroll
      for (int k = 1; k < KP; ++k) {
        if (k < W) {
          Acc x[V];
          unpack<WIRE, V>(raw[u][k], x);
#pragma unroll
          for (int i = 0; i < V; ++i) acc[i] = combine(acc[i], x[i], a.op);
        }
      }
      applyScale(acc, a.scale);
      const uint4 r = pack<WIRE, V>(acc);
#pragma unroll
      for (int k = 0; k < KP; ++k)
        if (k < W)
          stStage(static_cast<char*>(a.peer[(t.rank + k) % W]) + (base + tb.v[u]) * kVecBytes, r);
    }
  }
}
template <typename WIRE>
__device__ __forceinline__ void phaseDirectPeer(const ChannelDev& c, const OpArgs& a,
                                                const BlockCtx& bc) {
  FR_WITH_UNROLL(c.topo.world, 1, phaseDirectPeerU<WIRE, U, KP>(c, a, bc));
}

template <typename WIRE, int U>
__device__ __forceinline__ void phaseDirectNvlsU(const ChannelDev& c, const OpArgs& a,
                                                 const BlockCtx& bc) {
  constexpr int V = kVecBytes / sizeof(WIRE);
  using Acc = typename Tr<WIRE>::Acc;
  const Topo& t = c.topo;
  const Seg& s = a.seg;
  const int64_t nvec = ceilDiv(s.limit, V);
  const int64_t base = (int64_t)t.rank * s.qv;
  int64_t mine = nvec - base;
  if (mine > s.qv) mine = s.qv;
  if (mine < 0) mine = 0;
  char* mc = static_cast<char*>(a.mc);
  const int64_t ntiles = ceilDiv(mine, kThreads);
  for (int64_t tile0 = bc.b; tile0 < ntiles; tile0 += (int64_t)bc.G * U) {
    const Batch<U> tb = batchAt<U>(tile0, bc, ntiles, mine);
    uint4 r[U];
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (tb.ok[u]) r[u] = multimemLdReduce<WIRE>(mc + (base + tb.v[u]) * kVecBytes, a.op);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (!tb.ok[u]) continue;
      if (a.scale != 1.0f) {
        Acc x[V];
        unpack<WIRE, V>(r[u], x);
        applyScale(x, a.scale);
        r[u] = pack<WIRE, V>(x);
      }
      multimemSt(mc + (base + tb.v[u]) * kVecBytes, r[u]);
    }
  }
}
// a.unroll picks how many 16-byte multimem loads a thread keeps in flight.
template <typename WIRE>
__device__ __forceinline__ void phaseDirectNvls(const ChannelDev& c, const OpArgs& a,
                                                const BlockCtx& bc) {
  if (a.unroll >= 16)
    phaseDirectNvlsU<WIRE, 16>(c, a, bc);
  else if (a.unroll >= 8)
    phaseDirectNvlsU<WIRE, 8>(c, a, bc);
  else
    phaseDirectNvlsU<WIRE, 4>(c, a, bc);
}

// ---------------------------------------------------------------------------
// Phase: flag-in-data one-shot (small messages).  A unit is 8 bytes of the
// message.  Every rank stores its units, scaled, into the area of every peer as
// 16-byte words {data.lo, n, data.hi, n}, n = number of this collective on the
// channel (never 0).  A receiver spins on the word itself until both copies of
// n are there -- a 16-byte store may arrive as two 8-byte halves, each half then
// carries its own copy -- and reduces in rank order, so every rank gets the same
// bits.  No barrier and no separate flag: one trip over NVLink.
// The area holds LL words of earlier collectives only, so an old word can never
// be taken for a new one.  Halves alternate like the staging halves; a rank can
// be at most one collective ahead of the slowest peer (it needs everybody's
// words to finish), so the half written now was read two collectives ago.
// ---------------------------------------------------------------------------
// User-tensor access in 8-byte units and the spin on a flag-in-data word.
template <typename T>
struct LLIo {
  static constexpr int E = 8 / sizeof(T);
  using Acc = typename Tr<T>::Acc;
  const T* in;
  T* out;
  int64_t n;
  float scale;
  bool in_al, out_al;
  __device__ __forceinline__ LLIo(const void* i, void* o, int64_t n_, float s)
      : in(static_cast<const T*>(i)), out(static_cast<T*>(o)), n(n_), scale(s),
        in_al((reinterpret_cast<uintptr_t>(i) & 7u) == 0),
        out_al((reinterpret_cast<uintptr_t>(o) & 7u) == 0) {}
  // Unit u of the input, scaled, as it travels (rounded to T).
  __device__ __forceinline__ uint2 load(int64_t u) const {
    Acc x[E];
    const int64_t e0 = u * E;
    if (in_al && e0 + E <= n) {
      const uint2 raw = *reinterpret_cast<const uint2*>(in + e0);
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int i = 0; i < E; ++i) x[i] = Tr<T>::up(e[i]);
    } else {
#pragma unroll
      for (int i = 0; i < E; ++i) x[i] = e0 + i < n ? Tr<T>::up(in[e0 + i]) : Acc(0);
    }
    applyScale(x, scale);
    return pack(x);
  }
  static __device__ __forceinline__ uint2 pack(const Acc (&x)[E]) {
    uint2 raw;
    T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int i = 0; i < E; ++i) e[i] = Tr<T>::down(x[i]);
    return raw;
  }
  static __device__ __forceinline__ void unpack(const uint2& d, Acc (&x)[E]) {
    const T* e = reinterpret_cast<const T*>(&d);
#pragma unroll
    for (int i = 0; i < E; ++i) x[i] = Tr<T>::up(e[i]);
  }
  __device__ __forceinline__ void store(int64_t u, const uint2& d) const {
    const int64_t e0 = u * E;
    if (out_al && e0 + E <= n) {
      *reinterpret_cast<uint2*>(out + e0) = d;
    } else {
      const T* e = reinterpret_cast<const T*>(&d);
#pragma unroll
      for (int i = 0; i < E; ++i)
        if (e0 + i < n) out[e0 + i] = e[i];
    }
  }
};

// Spins until the 16-byte word at p carries `tag` in both flag positions.
// Bounded: on expiry records (timeout | aborted, peer q) and returns false.
__device__ __forceinline__ bool llWait(const ChannelDev& c, const BlockCtx& bc, const char* p,
                                       uint32_t tag, int q, uint2* data) {
  uint4 w = ldStage(p);
  if (w.y != tag || w.w != tag) {
    uint64_t t0 = 0;
    const uint64_t iter_cap = c.timeout_ns / 32 + (1ull << 20);
    for (uint64_t it = 1;; ++it) {
      w = ldStage(p);
      if (w.y == tag && w.w == tag) break;
      if ((it & 63) == 0) {
        const uint64_t now = globalTimerNs();
        if (t0 == 0) t0 = now;
        const bool aborted =
            (it & 1023) == 0 && c.abort_flag != nullptr && ldVolatile(c.abort_flag) != 0;
        if (now - t0 > c.timeout_ns || it > iter_cap || aborted) {
          volatile uint32_t* st = c.status;
          st[1] = 0;
          st[2] = (uint32_t)q;
          st[3] = bc.seq;
          __threadfence_system();
          st[0] = aborted ? kStatusAborted : kStatusTimeout;
          return false;
        }
      }
    }
  }
  *data = make_uint2(w.x, w.z);
  return true;
}

template <typename T>
__device__ __forceinline__ bool phaseLL(const ChannelDev& c, const OpArgs& a, const BlockCtx& bc) {
  constexpr int E = 8 / sizeof(T);
  using Acc = typename Tr<T>::Acc;
  const Topo& t = c.topo;
  const int W = t.world;
  const LLIo<T> io(a.in[blockIdx.y], a.out[blockIdx.y], a.seg.limit, a.scale);
  const int64_t units = ceilDiv(io.n, E);
  const int64_t cap = (int64_t)(c.ll_half_bytes / 16 / kMaxRanks);  // units per source rank
  const uint32_t tag = bc.seq + 1u == 0u ? 1u : bc.seq + 1u;
  const uint64_t half = (bc.seq & 1u) ? c.ll_half_bytes : 0;
  char* own = c.ll[t.rank] + half;

  const int64_t stride = (int64_t)bc.G * kThreads;
  for (int64_t u = (int64_t)bc.b * kThreads + threadIdx.x; u < units; u += stride) {
    const uint2 d = io.load(u);
    const uint4 word = make_uint4(d.x, tag, d.y, tag);
#pragma unroll
    for (int k = 1; k < kMaxRanks; ++k)
      if (k < W)
        stStage(c.ll[(t.rank + k) % W] + half + ((int64_t)t.rank * cap + u) * 16, word);
  }
  for (int64_t u = (int64_t)bc.b * kThreads + threadIdx.x; u < units; u += stride) {
    Acc acc[E];
#pragma unroll
    for (int q = 0; q < kMaxRanks; ++q) {
      if (q >= W) break;
      uint2 d;
      if (q == t.rank)
        d = io.load(u);  // what the peers got: the value after the round trip through T
      else if (!llWait(c, bc, own + ((int64_t)q * cap + u) * 16, tag, q, &d))
        return false;
      Acc x[E];
      LLIo<T>::unpack(d, x);
      if (q == 0) {
#pragma unroll
        for (int i = 0; i < E; ++i) acc[i] = x[i];
      } else {
#pragma unroll
        for (int i = 0; i < E; ++i) acc[i] = combine(acc[i], x[i], a.op);
      }
    }
    io.store(u, LLIo<T>::pack(acc));
  }
  return true;
}

// ---------------------------------------------------------------------------
// Phase: flag-in-data two-shot (a few hundred KiB to a MiB or two).  Same words
// as above, but the message is reduce-scattered and all-gathered: rank r
// receives everybody's units of chunk r (area A: [source rank][unit]), reduces
// them in rank order and sends the result to everybody (area B: [chunk][unit]).
// Every unit crosses NVLink twice as 16 bytes instead of W times: for a 1 MiB
// message 3.5 MiB leave each GPU, as for a 256 KiB one-shot.  Still no barrier.
// A half of the area holds A and B: 2 x W x (units per chunk) words.
// ---------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ bool phaseLL2(const ChannelDev& c, const OpArgs& a, const BlockCtx& bc) {
  constexpr int E = 8 / sizeof(T);
  using Acc = typename Tr<T>::Acc;
  const Topo& t = c.topo;
  const int W = t.world;
  const LLIo<T> io(a.in[blockIdx.y], a.out[blockIdx.y], a.seg.limit, a.scale);
  const int64_t units = ceilDiv(io.n, E);
  const int64_t cu = ceilDiv(units, W);  // units per chunk
  const uint32_t tag = bc.seq + 1u == 0u ? 1u : bc.seq + 1u;
  const uint64_t half = (bc.seq & 1u) ? c.ll_half_bytes : 0;
  const uint64_t areaB = (uint64_t)W * cu * 16;
  const int64_t stride = (int64_t)bc.G * kThreads;
  const int64_t first = (int64_t)bc.b * kThreads + threadIdx.x;

  // 1. My units of every other rank's chunk go to that rank.
  for (int k = 1; k < W; ++k) {
    const int p = (t.rank + k) % W;
    char* dst = c.ll[p] + half + (int64_t)t.rank * cu * 16;
    for (int64_t u = first; u < cu; u += stride) {
      const int64_t g = (int64_t)p * cu + u;
      if (g >= units) break;
      const uint2 d = io.load(g);
      stStage(dst + u * 16, make_uint4(d.x, tag, d.y, tag));
    }
  }
  // 2. Reduce my chunk in rank order; the result goes to everybody.
  char* ownA = c.ll[t.rank] + half;
  for (int64_t u = first; u < cu; u += stride) {
    const int64_t g = (int64_t)t.rank * cu + u;
    if (g >= units) break;
    Acc acc[E];
#pragma unroll
    for (int q = 0; q < kMaxRanks; ++q) {
      if (q >= W) break;
      uint2 d;
      if (q == t.rank)
        d = io.load(g);
      else if (!llWait(c, bc, ownA + ((int64_t)q * cu + u) * 16, tag, q, &d))
        return false;
      Acc x[E];
      LLIo<T>::unpack(d, x);
      if (q == 0) {
#pragma unroll
        for (int i = 0; i < E; ++i) acc[i] = x[i];
      } else {
#pragma unroll
        for (int i = 0; i < E; ++i) acc[i] = combine(acc[i], x[i], a.op);
      }
    }
    const uint2 r = LLIo<T>::pack(acc);
    const uint4 word = make_uint4(r.x, tag, r.y, tag);
#pragma unroll
    for (int k = 1; k < kMaxRanks; ++k)
      if (k < W)
        stStage(c.ll[(t.rank + k) % W] + half + areaB + ((int64_t)t.rank * cu + u) * 16, word);
    io.store(g, r);
  }
  // 3. The other chunks, reduced by their owners.
  char* ownB = c.ll[t.rank] + half + areaB;
  for (int k = 1; k < W; ++k) {
    const int p = (t.rank + k) % W;
    for (int64_t u = first; u < cu; u += stride) {
      const int64_t g = (int64_t)p * cu + u;
      if (g >= units) break;
      uint2 d;
      if (!llWait(c, bc, ownB + ((int64_t)p * cu + u) * 16, tag, p, &d)) return false;
      io.store(g, d);
    }
  }
  return true;
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
  } else if constexpr (K == KernelId::P2P_DIRECT) {
    // Barrier 0: every rank's tensor is ready (a rank signals from this kernel,
    // which its stream runs after the producer).  Barrier 3: all results have
    // landed everywhere, the tensor may be used again.
    if (barrier<kAll>(c, bc, 0)) {
      phaseDirectPeer<WIRE>(c, a, bc);
      barrier<kAll>(c, bc, 3);
    }
  } else if constexpr (K == KernelId::NVLS_DIRECT) {
    if (barrier<kAll>(c, bc, 0)) {
      phaseDirectNvls<WIRE>(c, a, bc);
      barrier<kAll>(c, bc, 3);
    }
  } else if constexpr (K == KernelId::LL_ONESHOT) {
    phaseLL<WIRE>(c, a, bc);
  } else if constexpr (K == KernelId::LL_TWOSHOT) {
    phaseLL2<WIRE>(c, a, bc);
  }
  leave(c, a, bc);
}

// One __global__ per kernel id so that profiles show the stage by name.
// grid.x = blocks of one rank; grid.y = 1 in a real job, = world when all ranks
// are emulated on one GPU (then chs[] and the in/out arrays hold one entry per
// rank).  The channel description lives in device memory: it never changes.
#define FR_DEFINE_KERNEL(NAME, KID)                                                         \
  template <typename IO, typename WIRE>                                                     \
  __global__ void __launch_bounds__(kThreads, 1)                                            \
      NAME(const ChannelDev* __restrict__ chs, const __grid_constant__ OpArgs a) {          \
    body<IO, WIRE, KID>(chs[blockIdx.y], a);                                                \
  }

FR_DEFINE_KERNEL(oneshot_allreduce, KernelId::ONESHOT)
FR_DEFINE_KERNEL(twoshot_allreduce, KernelId::TWOSHOT)
FR_DEFINE_KERNEL(rs_intragroup, KernelId::RS_INTRAGROUP)
FR_DEFINE_KERNEL(shard_server_reduce, KernelId::SHARD_SERVER_REDUCE)
FR_DEFINE_KERNEL(ag_intragroup, KernelId::AG_INTRAGROUP)
FR_DEFINE_KERNEL(diffuse_rail, KernelId::DIFFUSE)
FR_DEFINE_KERNEL(nvls_allreduce, KernelId::NVLS_TWOSHOT)
FR_DEFINE_KERNEL(nvls_oneshot_allreduce, KernelId::NVLS_ONESHOT)
FR_DEFINE_KERNEL(direct_allreduce, KernelId::P2P_DIRECT)
FR_DEFINE_KERNEL(nvls_direct_allreduce, KernelId::NVLS_DIRECT)
FR_DEFINE_KERNEL(ll_allreduce, KernelId::LL_ONESHOT)
FR_DEFINE_KERNEL(ll2_allreduce, KernelId::LL_TWOSHOT)


using KernelFn = void (*)(const ChannelDev*, const OpArgs);

template <typename IO, typename WIRE>
KernelFn kernelFor(KernelId id) {
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
    case KernelId::P2P_DIRECT:
      if constexpr (std::is_same<IO, WIRE>::value) return direct_allreduce<IO, WIRE>;
      return nullptr;
    case KernelId::NVLS_DIRECT:
      if constexpr (std::is_same<IO, WIRE>::value &&
                    std::is_floating_point<typename Tr<WIRE>::Acc>::value && sizeof(WIRE) <= 4)
        return nvls_direct_allreduce<IO, WIRE>;
      return nullptr;
    case KernelId::LL_ONESHOT:
      if constexpr (std::is_same<IO, WIRE>::value) return ll_allreduce<IO, WIRE>;
      return nullptr;
    case KernelId::LL_TWOSHOT:
      if constexpr (std::is_same<IO, WIRE>::value) return ll2_allreduce<IO, WIRE>;
      return nullptr;
    default: return nullptr;
  }
}

}  // namespace impl
}  // namespace fairring

// One translation unit per (tensor dtype, wire dtype) pair instantiates the
// kernels and exports a lookup function; they compile in parallel.
#define FR_INSTANTIATE_COMBO(TAG, IO_T, WIRE_T)                                  \
  namespace fairring {                                                           \
  impl::KernelFn lookupKernel_##TAG(KernelId id) { return impl::kernelFor<IO_T, WIRE_T>(id); } \
  }
