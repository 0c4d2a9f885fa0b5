// Index math shared by the host planner, the CPU path and the CUDA kernels.
//
// Vocabulary (same letters as the reference's README, README.md:82-98):
//   W  world size, D GPUs per "machine" (group), M machines, W = D*M.
//   A rank is the pair (m, d).  Two rank numberings are accepted, as in
//   fairring/machine.cc:91-117 of the reference:
//     standard  : rank = m*D + d   (what torchrun produces)
//     favorable : rank = d*M + m
//   A collective moves W "chunks"; chunk c is owned by rank c.  Inside the
//   staging memory every chunk is padded to `qv` 16-byte vectors so that every
//   remote access is a full, aligned 16-byte transaction; the ragged tail is
//   predicated where the user tensor is touched (the reference instead copies
//   the tail into padding buffers, fairring/device.cc:468-475,511-521).
//
// Staging layout of one half-slot on rank (m, d):
//     [ source slot s : 0..D ) [ rail chunk j : 0..M ) [ qv vectors ]
//   slot s holds what group member s pushed; rail chunk j is user chunk
//   rankOf(j, d).  Slot d ("self slot") is where reduced data lives.
//   With M == 1 this degenerates to the flat layout [ source rank ][ qv ].
#pragma once

#include <cstdint>

#if defined(__CUDACC__)
#define FR_HD __host__ __device__ __forceinline__
#else
#define FR_HD inline
#endif

namespace fairring {

constexpr int kMaxRanks = 8;        // one NVSwitch domain
constexpr int kVecBytes = 16;       // unit of every staging access
constexpr int kMaxBlocks = 64;      // upper bound on the grid of a channel
constexpr int kBarriersPerOp = 4;   // barrier epochs reserved per collective

enum class DType : int32_t { U8 = 0, I8, I32, I64, F16, BF16, F32, F64, kCount };
enum class RedOp : int32_t { SUM = 0, MAX, MIN };

FR_HD int dtypeSize(DType t) {
  switch (t) {
    case DType::U8: case DType::I8: return 1;
    case DType::F16: case DType::BF16: return 2;
    case DType::I32: case DType::F32: return 4;
    default: return 8;
  }
}

FR_HD int64_t ceilDiv(int64_t a, int64_t b) { return (a + b - 1) / b; }
FR_HD int64_t roundUp(int64_t a, int64_t b) { return ceilDiv(a, b) * b; }
FR_HD int64_t roundDown(int64_t a, int64_t b) { return (a / b) * b; }

struct Topo {
  int32_t world;      // W
  int32_t D;          // ranks per group ("GPUs per machine")
  int32_t M;          // groups ("machines")
  int32_t favorable;  // 1: rank = d*M+m, 0: rank = m*D+d
  int32_t rank;
  int32_t m;
  int32_t d;
  int32_t pad_;
};

FR_HD int rankOf(const Topo& t, int m, int d) {
  return t.favorable ? d * t.M + m : m * t.D + d;
}
FR_HD int machineOf(const Topo& t, int rank) {
  return t.favorable ? rank % t.M : rank / t.D;
}
FR_HD int deviceOf(const Topo& t, int rank) {
  return t.favorable ? rank / t.M : rank % t.D;
}

inline Topo makeTopo(int world, int D, bool favorable, int rank) {
  Topo t{};
  t.world = world;
  t.D = D;
  t.M = world / D;
  t.favorable = favorable ? 1 : 0;
  t.rank = rank;
  t.m = machineOf(t, rank);
  t.d = deviceOf(t, rank);
  return t;
}

// How the W chunks of one slice sit in the user's memory.
//   element (c, i) lives at user index  c*chunk_stride + i
//   and exists iff  i < chunk_len  and  c*chunk_stride + i < limit.
// all-reduce of a flat slice: chunk_len = chunk_stride = qv*V, limit = numel.
// reduce-scatter / all-gather: chunk_stride = per-rank numel, limit = INT64_MAX.
struct Seg {
  int64_t chunk_len;
  int64_t chunk_stride;
  int64_t limit;
  int64_t qv;  // staging vectors per chunk
};

FR_HD int64_t validInVector(const Seg& s, int c, int64_t v, int V) {
  // Number of real elements (0..V) in vector v of chunk c.
  int64_t i0 = v * V;
  int64_t n = s.chunk_len - i0;
  int64_t lim = s.limit - ((int64_t)c * s.chunk_stride + i0);
  if (lim < n) n = lim;
  if (n > V) n = V;
  return n < 0 ? 0 : n;
}

// Vector offset, inside a half-slot, of rail chunk j in source slot s.
FR_HD int64_t stagingVec(const Topo& t, const Seg& s, int slot, int j) {
  return ((int64_t)slot * t.M + j) * s.qv;
}

// ---------------------------------------------------------------------------
// Host-side planning: memory budget -> channels and half-slots -> slices.
// Counterpart of computeLayout in the reference (fairring/utils.h:288-327),
// with the documented-but-unimplemented FAIRRING_SLICE_SIZE honoured.
// ---------------------------------------------------------------------------
struct MemoryPlan {
  int64_t total_bytes;      // FAIRRING_TOTAL_MEMORY (staging only; flags are extra)
  int32_t channels;         // slices in flight (FAIRRING_PARALLELISM, clamped)
  int64_t slot_bytes;       // per channel
  int64_t half_bytes;       // slot_bytes / 2 : the unit one slice may use
  int64_t max_slice_bytes;  // min(FAIRRING_SLICE_SIZE, what a half can stage)
};

inline MemoryPlan planMemory(int64_t total_bytes, int64_t slice_bytes,
                             int32_t parallelism, int world,
                             int64_t min_half_bytes = 1 << 20) {
  MemoryPlan p{};
  if (parallelism < 1) parallelism = 1;
  const int64_t align = (int64_t)kVecBytes * world * 2;
  if (total_bytes < align) total_bytes = align;
  // Never let a half shrink below min_half_bytes: many tiny slices cost more
  // in barriers than they win in overlap.
  int64_t ch = parallelism;
  while (ch > 1 && total_bytes / ch / 2 < min_half_bytes) --ch;
  p.total_bytes = total_bytes;
  p.channels = (int32_t)ch;
  p.half_bytes = roundDown(total_bytes / ch / 2, (int64_t)kVecBytes * world);
  p.slot_bytes = p.half_bytes * 2;
  int64_t cap = p.half_bytes;
  if (slice_bytes > 0 && slice_bytes < cap) cap = slice_bytes;
  p.max_slice_bytes = roundDown(cap, (int64_t)kVecBytes * world);
  if (p.max_slice_bytes < (int64_t)kVecBytes * world)
    p.max_slice_bytes = (int64_t)kVecBytes * world;
  return p;
}

struct SlicePlan {
  int64_t num_slices;
  int64_t slice_elems;  // elements per slice (last one may be shorter)
};

// Split `numel` elements of `wire_esize` bytes into balanced slices of at most
// `max_slice_bytes` staged bytes, each a multiple of W vectors.
inline SlicePlan planSlices(int64_t numel, int wire_esize, int world,
                            int64_t max_slice_bytes) {
  const int64_t V = kVecBytes / wire_esize;
  const int64_t quantum = V * world;
  int64_t max_elems = roundDown(max_slice_bytes / wire_esize, quantum);
  if (max_elems < quantum) max_elems = quantum;
  SlicePlan s{};
  if (numel <= 0) { s.num_slices = 0; s.slice_elems = 0; return s; }
  s.num_slices = ceilDiv(numel, max_elems);
  s.slice_elems = roundUp(ceilDiv(numel, s.num_slices), quantum);
  if (s.slice_elems > max_elems) s.slice_elems = max_elems;
  s.num_slices = ceilDiv(numel, s.slice_elems);
  return s;
}

inline Seg allreduceSeg(int64_t slice_numel, int wire_esize, int world) {
  const int64_t V = kVecBytes / wire_esize;
  Seg s{};
  s.qv = ceilDiv(ceilDiv(slice_numel, V), world);
  if (s.qv < 1) s.qv = 1;
  s.chunk_len = s.qv * V;
  s.chunk_stride = s.chunk_len;
  s.limit = slice_numel;
  return s;
}

inline Seg scatterSeg(int64_t slice_len, int64_t per_rank_numel, int wire_esize) {
  const int64_t V = kVecBytes / wire_esize;
  Seg s{};
  s.qv = ceilDiv(slice_len, V);
  if (s.qv < 1) s.qv = 1;
  s.chunk_len = slice_len;
  s.chunk_stride = per_rank_numel;
  s.limit = INT64_MAX;
  return s;
}

}  // namespace fairring
