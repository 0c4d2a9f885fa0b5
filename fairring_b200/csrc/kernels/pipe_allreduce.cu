// Pipelined all-reduce for ordinary tensors (sm_100a): bulk copies through
// shared memory (cp.async.bulk + mbarrier) for the two local copy stages,
// multimem.ld_reduce / multimem.st (or peer loads / stores) for the reduction,
// all three overlapping chunk by chunk inside one launch.  See
// pipe_allreduce.h for the protocol.
#include "pipe_allreduce.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "device_prims.cuh"
#include "kernels.h"

namespace fairring {
namespace pipe {

using namespace dev;

constexpr int kMaxStages = 8;
constexpr int kNR = kPipeRedGroups;
constexpr int kFirstRedWarp = 2;  // warps 0, 1: copy-in, copy-out
constexpr int kRedWarps = (kPipeThreads / 32 - kFirstRedWarp) / kNR;  // warps per reduce group
constexpr int kRedThreads = kRedWarps * 32;

enum Where : uint32_t {  // second status word: which wait gave up
  kWaitCopyIn = 100,     // reduce waiting for a peer's copy-in counter
  kWaitReduce = 101,     // copy-out waiting for a peer's reduce counter
  kWaitSlot = 102,       // copy-in waiting for this block's copy-out (ring slot reuse)
  kWaitBulk = 103,       // a bulk copy into shared memory did not complete
  kWaitCopyInLocal = 104,  // the publisher waiting for this block's own copy-in
};

struct Ctl {  // block-shared control words
  unsigned long long full[2][kMaxStages];  // mbarriers: data of stage s has landed ([role][stage])
  volatile uint32_t cout_done;             // chunks (numbered across launches) copied out by this block
  volatile uint32_t cin_done;              // chunks whose copy-in stores are complete (not yet published)
  volatile uint32_t failed;                // some wait of this block gave up
};

struct Geo {
  int64_t nvec;  // 16-byte vectors in the message (the last one may be partial)
  int64_t cv;    // vectors per chunk
  int64_t sv;    // vectors per sub-chunk (what one rank reduces of a full chunk)
  int64_t pv;    // vectors per piece (one block's part of a sub-chunk)
  int32_t nchunks;
  int32_t tail;  // bytes in the partial last vector, 0 if the message is whole vectors
  int32_t W, G, b, slots;
};

struct Piece {
  int64_t lo, hi;  // message vectors [lo, hi)
};

// Block b's part of sub-chunk j of the chunk that starts at vector c_lo.
// Sub-chunk j is what rank j reduces.  The cut is the same for every chunk of a
// launch (it is made on the full chunk length and clipped to the message), so a
// position of a ring slot is always owned by the same block: a block that waits
// for its own copy-out of the slot's previous chunk has waited for all readers
// of what it overwrites.  (No division here: the copy warps run this per piece.)
__device__ __forceinline__ Piece pieceAt(const Geo& g, int64_t c_lo, int j, int b) {
  const int64_t c_hi = c_lo + g.cv < g.nvec ? c_lo + g.cv : g.nvec;
  const int64_t s_lo = c_lo + (int64_t)j * g.sv;
  const int64_t s_hi = s_lo + g.sv < c_hi ? s_lo + g.sv : c_hi;
  Piece p;
  p.lo = s_lo + (int64_t)b * g.pv;
  p.hi = p.lo + g.pv < s_hi ? p.lo + g.pv : s_hi;
  if (p.hi < p.lo) p.hi = p.lo;
  return p;
}

// Walks the items of this block in order: for every chunk k the non-empty
// pieces of sub-chunks 0..W-1 (partial tail vector left out), then an
// end-of-chunk marker (j == W).  Keeps the chunk's first vector and ring slot
// up to date by increments.
struct Cursor {
  int32_t k, j;
  int32_t slot;   // ring slot of chunk k
  int32_t pad_;
  int64_t c_lo;   // first vector of chunk k
  int64_t lo, hi;
};
__device__ __forceinline__ void cursorNext(Cursor& c, const Geo& g, int64_t took) {
  if (c.j == g.W) {
    ++c.k;
    c.j = -1;
    c.lo = c.hi = 0;
    c.c_lo += g.cv;
    if (++c.slot == g.slots) c.slot = 0;
  } else {
    c.lo += took;
  }
  while (c.k < g.nchunks && c.lo >= c.hi) {
    ++c.j;
    if (c.j == g.W) return;
    Piece p = pieceAt(g, c.c_lo, c.j, g.b);
    if (g.tail != 0 && p.hi == g.nvec && p.hi > p.lo) --p.hi;
    c.lo = p.lo;
    c.hi = p.hi;
  }
}
__device__ __forceinline__ void cursorInit(Cursor& c, const Geo& g, uint32_t g0) {
  c.k = 0;
  c.j = -1;
  c.slot = (int32_t)(g0 % (uint32_t)g.slots);
  c.c_lo = 0;
  c.lo = c.hi = 0;
  cursorNext(c, g, 0);
}

// Does this block own the (partial) last vector of the message, and is that
// vector in the chunk (number k) that starts at c_lo?
__device__ __forceinline__ bool ownsTail(const Geo& g, int k, int64_t c_lo) {
  if (g.tail == 0 || k != g.nchunks - 1) return false;
  for (int j = 0; j < g.W; ++j) {
    const Piece p = pieceAt(g, c_lo, j, g.b);
    if (p.hi == g.nvec && p.hi > p.lo) return true;
  }
  return false;
}

// ---- PTX wrappers ------------------------------------------------------------
__device__ __forceinline__ uint32_t smemAddr(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbarInit(unsigned long long* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smemAddr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbarExpectTx(unsigned long long* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smemAddr(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbarTryWait(unsigned long long* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
      : "=r"(ok)
      : "r"(smemAddr(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// global -> shared, completion counted on an mbarrier
__device__ __forceinline__ void bulkLoad(void* smem_dst, const void* gsrc, uint32_t bytes,
                                         unsigned long long* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smemAddr(smem_dst)),
      "l"(gsrc), "r"(bytes), "r"(smemAddr(bar))
      : "memory");
}
// shared -> global, completion tracked by this thread's bulk async-groups
__device__ __forceinline__ void bulkStore(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst),
               "r"(smemAddr(smem_src)), "r"(bytes)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void bulkWaitAll() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void fenceProxyAsync() {
  asm volatile("fence.proxy.async;" ::: "memory");
}
// Barrier among `count` threads (a whole number of warps) with an OR over a predicate.
__device__ __forceinline__ bool namedBarrierOr(int id, int count, bool pred) {
  uint32_t r;
  asm volatile(
      "{ .reg .pred p, q; setp.ne.u32 q, %3, 0; bar.red.or.pred p, %1, %2, q; selp.u32 %0, 1, 0, p; }"
      : "=r"(r)
      : "r"(id), "r"(count), "r"((uint32_t)pred)
      : "memory");
  return r != 0;
}

// ---- bounded waits -------------------------------------------------------------
__device__ __forceinline__ void recordFailure(const PipeChannelDev& c, Ctl* ctl, uint32_t code,
                                              uint32_t where, uint32_t peer, uint32_t chunk) {
  // The first failure of a block is the one worth reporting: the waits that
  // give up after it do so because of it.
  if (atomicExch(const_cast<uint32_t*>(&ctl->failed), 1u) != 0u) return;
  volatile uint32_t* s = c.status;
  s[1] = where;
  s[2] = peer;
  s[3] = chunk;
  __threadfence_system();
  s[0] = code;
}

// Waits until *flag (written by a peer with a release store) has reached
// `want`.  Gives up after the time limit, when the host raises the abort word
// or when another role of this block has failed.
__device__ __forceinline__ bool waitCounter(const PipeChannelDev& c, Ctl* ctl, const uint32_t* flag,
                                            uint32_t want, uint32_t where, uint32_t peer) {
  uint64_t t0 = 0;
  // A wait on this rank's own counter only fails because something upstream of
  // it did: give the waits on peers the time to report first.
  const uint64_t limit = peer == (uint32_t)c.rank ? 2 * c.timeout_ns : c.timeout_ns;
  const uint64_t iter_cap = limit / 32 + (1ull << 20);
  for (uint64_t n = 1;; ++n) {
    const uint32_t v = ldAcquireSys(flag);
    if ((int32_t)(v - want) >= 0) return true;
    if ((n & 63) == 0) {
      if (ctl->failed) return false;
      const uint64_t now = globalTimerNs();
      if (t0 == 0) t0 = now;
      if (now - t0 > limit || n > iter_cap) {
        recordFailure(c, ctl, kStatusTimeout, where, peer, want - 1);
        return false;
      }
      if ((n & 1023) == 0 && c.abort_flag != nullptr && ldVolatile(c.abort_flag) != 0) {
        recordFailure(c, ctl, kStatusAborted, where, peer, want - 1);
        return false;
      }
    }
  }
}

// All lanes of the warp call this; true once the bulk copy has landed.
__device__ __forceinline__ bool mbarWait(const PipeChannelDev& c, Ctl* ctl, unsigned long long* bar,
                                         uint32_t parity, uint32_t chunk, bool heed_failed = true) {
  uint64_t t0 = 0;
  for (uint64_t n = 1;; ++n) {
    if (mbarTryWait(bar, parity)) return true;
    if ((n & 255) == 0) {
      if (heed_failed && ctl->failed) return false;
      const uint64_t now = globalTimerNs();
      if (t0 == 0) t0 = now;
      if (now - t0 > 2 * c.timeout_ns || n > (1ull << 34)) {
        recordFailure(c, ctl, kStatusTimeout, kWaitBulk, (uint32_t)c.rank, chunk);
        return false;
      }
    }
  }
}

// Copy-in may write ring slot (g mod slots) once this block has copied out
// chunk g - slots.
__device__ __forceinline__ bool waitSlotFree(const PipeChannelDev& c, Ctl* ctl, uint32_t g) {
  const uint32_t need = g + 1u - (uint32_t)c.slots;
  uint64_t t0 = 0;
  for (uint64_t n = 1;; ++n) {
    if ((int32_t)(ctl->cout_done - need) >= 0) return true;
    if ((n & 255) == 0) {
      if (ctl->failed) return false;
      const uint64_t now = globalTimerNs();
      if (t0 == 0) t0 = now;
      if (now - t0 > 2 * c.timeout_ns || n > (1ull << 34)) {
        recordFailure(c, ctl, kStatusTimeout, kWaitSlot, (uint32_t)c.rank, g);
        return false;
      }
    }
  }
}

__device__ __forceinline__ uint32_t* counterAt(uint32_t* pad, int lane_idx, int src, int b) {
  return pad + ((size_t)lane_idx * kMaxRanks + src) * kMaxBlocks + b;
}

__device__ __forceinline__ uint64_t slotOffset(const PipeChannelDev& c, int slot) {
  return (uint64_t)slot * c.slot_bytes;
}

// ---- the two copy roles ------------------------------------------------------
// wait_group takes an immediate operand.
__device__ __forceinline__ void bulkWaitReadN(int n) {
  switch (n) {
    case 0: asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); break;
    case 1: asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); break;
    case 2: asm volatile("cp.async.bulk.wait_group.read 2;" ::: "memory"); break;
    default: asm volatile("cp.async.bulk.wait_group.read 3;" ::: "memory"); break;
  }
}
__device__ __forceinline__ void bulkWaitN(int n) {
  switch (n) {
    case 0: asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); break;
    case 1: asm volatile("cp.async.bulk.wait_group 1;" ::: "memory"); break;
    case 2: asm volatile("cp.async.bulk.wait_group 2;" ::: "memory"); break;
    default: asm volatile("cp.async.bulk.wait_group 3;" ::: "memory"); break;
  }
}

// CIN: user tensor -> own ring slot.  !CIN: own ring slot -> user tensor.
// One warp; lane 0 issues the bulk copies and owns their bulk async-groups.
// Half of the stages are being filled by loads while the other half is being
// drained by stores.  Copy-in does not stop at the end of a chunk: the chunk's
// counter is published a few stores later, once wait_group says that its
// stores are complete.
// The warp is alone with its instruction stream, so the per-copy path is kept
// to a pointer, a byte count and two stage indices; the cursor arithmetic runs
// once per piece.
template <bool CIN>
__device__ __forceinline__ void copyRole(const PipeChannelDev& c, const PipeArgs& a, const Geo& g,
                                         Ctl* ctl, unsigned char* stage_base, uint32_t g0,
                                         const char* user_in, char* user_out) {
  const int lane = threadIdx.x & 31;
  const int role = CIN ? 0 : 1;
  const uint32_t NS = (uint32_t)a.stages;
  const uint32_t stage_bytes = (uint32_t)a.stage_bytes;
  int keep = (int)NS / 2 - 1;  // stores that may still be reading their stage after a wait
  if (keep > 3) keep = 3;
  if (keep < 0) keep = 0;
  char* own = c.ring[c.rank];
  uint32_t* my_pad = c.flags[c.rank];
  Cursor ld, st;
  cursorInit(ld, g, g0);
  cursorInit(st, g, g0);
  uint32_t nld = 0, nst = 0, freed = 0;  // loads issued, stores issued, stages released by stores
  uint32_t ls = 0, ss = 0, sph = 0;      // stage of the next load, of the next store, its phase
  const char* l_src = nullptr;           // rest of the piece being loaded
  uint32_t l_left = 0;
  char* s_dst = nullptr;                 // rest of the piece being stored
  uint32_t s_left = 0;
  int ld_open = -1;      // copy-out: last chunk whose reduce counters were seen complete
  int st_started = -1;   // copy-in: last chunk whose ring slot was seen free
  int pend_k = -1;       // copy-in: chunk whose counter is not yet published
  uint32_t pend_at = 0;  // ... and the number of stores issued when it ended
  bool ok = true;

  // Copy-in: chunk k of this block is in the ring (its bulk stores are complete
  // and so are the tail bytes).  The publisher warp tells the peers.
  auto publish = [&](int k) {
    __syncwarp();
    if (lane == 0) {
      __threadfence_block();
      ctl->cin_done = g0 + (uint32_t)k + 1u;
    }
  };
  auto waitReduced = [&](int k, bool block) -> int {  // copy-out: 1 ready, 0 not yet, -1 failed
    const uint32_t gg = g0 + (uint32_t)k;
    const uint32_t* f = counterAt(my_pad, kNR + (int)(gg % kNR), lane < g.W ? lane : 0, g.b);
    bool mine = true;
    if (block) {
      if (lane < g.W) mine = waitCounter(c, ctl, f, gg + 1u, kWaitReduce, (uint32_t)lane);
      if (!__all_sync(0xffffffffu, mine)) return -1;
    } else {
      mine = lane >= g.W || (int32_t)(ldAcquireSys(f) - (gg + 1u)) >= 0;
      if (!__all_sync(0xffffffffu, mine)) return 0;
    }
    fenceProxyAsync();  // peers' generic-proxy writes before this thread's bulk reads
    return 1;
  };
  // Moves the load side to its next piece.  1: l_src/l_left are set; 0: nothing
  // to load right now (message done, or the next chunk is not reduced yet);
  // -1: a wait failed.
  auto nextLoadPiece = [&]() -> int {
    while (ld.k < g.nchunks && ld.j == g.W) cursorNext(ld, g, 0);
    if (ld.k >= g.nchunks) return 0;
    if (!CIN && ld.k > ld_open) {
      // Only block when nothing is loaded ahead of the stores.
      const int r = waitReduced(ld.k, nld == nst);
      if (r <= 0) return r;
      ld_open = ld.k;
    }
    l_src = CIN ? user_in + ld.lo * kVecBytes
                : own + slotOffset(c, ld.slot) + (ld.lo - ld.c_lo) * kVecBytes;
    l_left = (uint32_t)((ld.hi - ld.lo) * kVecBytes);
    cursorNext(ld, g, ld.hi - ld.lo);
    return 1;
  };
  // End of chunk st.k on the store side.
  auto endOfChunk = [&]() -> bool {
    const uint32_t gg = g0 + (uint32_t)st.k;
    const bool tail_here = ownsTail(g, st.k, st.c_lo);
    const int64_t tv = g.nvec - 1;  // the partial vector
    char* ring_tail = own + slotOffset(c, st.slot) + (tv - st.c_lo) * kVecBytes;
    if (CIN) {
      if (tail_here) {
        if (st.k > st_started) {
          if (!__all_sync(0xffffffffu, waitSlotFree(c, ctl, gg))) return false;
          st_started = st.k;
        }
        if (lane < kVecBytes) {
          const unsigned char v = lane < g.tail ? (unsigned char)user_in[tv * kVecBytes + lane] : 0;
          *reinterpret_cast<volatile unsigned char*>(ring_tail + lane) = v;
        }
      }
      if (pend_k >= 0 || st.k == g.nchunks - 1) {
        // An earlier chunk is still unpublished, or nothing follows: drain.
        if (lane == 0) bulkWaitAll();
        freed = nst;
        if (pend_k >= 0) publish(pend_k);
        publish(st.k);
        pend_k = -1;
      } else {
        pend_k = st.k;
        pend_at = nst;
      }
    } else {
      if (tail_here && st.k > ld_open) {
        // No whole vector of this chunk came through the loads, so its reduce
        // counters have not been waited for yet.
        if (waitReduced(st.k, true) < 0) return false;
        ld_open = st.k;
      }
      if (tail_here && lane < g.tail)
        user_out[tv * kVecBytes + lane] = *reinterpret_cast<volatile unsigned char*>(ring_tail + lane);
      __syncwarp();
      if (lane == 0) {
        __threadfence_block();
        ctl->cout_done = gg + 1u;  // every bulk load of the chunk has been waited for
      }
    }
    return true;
  };

  for (;;) {
    // Store side: find the next piece, closing chunks on the way.
    if (s_left == 0) {
      while (st.k < g.nchunks && st.j == g.W) {
        if (!endOfChunk()) {
          ok = false;
          break;
        }
        cursorNext(st, g, 0);
      }
      if (!ok || st.k >= g.nchunks) break;
      if (CIN && st.k > st_started) {
        if (!__all_sync(0xffffffffu, waitSlotFree(c, ctl, g0 + (uint32_t)st.k))) {
          ok = false;
          break;
        }
        st_started = st.k;
      }
      s_dst = CIN ? own + slotOffset(c, st.slot) + (st.lo - st.c_lo) * kVecBytes
                  : user_out + st.lo * kVecBytes;
      s_left = (uint32_t)((st.hi - st.lo) * kVecBytes);
      cursorNext(st, g, st.hi - st.lo);
    }
    // Loads run ahead of the stores while shared-memory stages are free.
    while (nld < freed + NS) {
      if (l_left == 0) {
        const int r = nextLoadPiece();
        if (r < 0) ok = false;
        if (r <= 0) break;
      }
      const uint32_t take = l_left < stage_bytes ? l_left : stage_bytes;
      if (lane == 0) {
        mbarExpectTx(&ctl->full[role][ls], take);
        bulkLoad(stage_base + (size_t)ls * stage_bytes, l_src, take, &ctl->full[role][ls]);
      }
      l_src += take;
      l_left -= take;
      ++nld;
      if (++ls == NS) ls = 0;
    }
    if (!ok) break;
    // The next copy of the store side: its load was issued above (nld > nst).
    if (!__all_sync(0xffffffffu, mbarWait(c, ctl, &ctl->full[role][ss], sph, g0 + (uint32_t)st.k))) {
      ok = false;
      break;
    }
    const uint32_t take = s_left < stage_bytes ? s_left : stage_bytes;
    ++nst;
    const bool settle = CIN && pend_k >= 0 && nst - pend_at >= (uint32_t)keep;
    if (lane == 0) {
      bulkStore(s_dst, stage_base + (size_t)ss * stage_bytes, take);
      // All but the newest `keep` stores have finished reading their stage --
      // or, when a chunk waits to be published, have been written altogether.
      if (settle)
        bulkWaitN(keep);
      else
        bulkWaitReadN(keep);
    }
    s_dst += take;
    s_left -= take;
    if (++ss == NS) {
      ss = 0;
      sph ^= 1u;
    }
    freed = nst > (uint32_t)keep ? nst - (uint32_t)keep : 0;
    if (settle) {
      publish(pend_k);
      pend_k = -1;
    }
    __syncwarp();
  }
  // Leave nothing in flight: stores first, then loads that were never consumed.
  if (lane == 0) bulkWaitAll();
  if (CIN && ok && pend_k >= 0) publish(pend_k);
  for (uint32_t i = nst; i < nld; ++i) {
    mbarWait(c, ctl, &ctl->full[role][ss], sph, 0, /*heed_failed=*/false);
    if (++ss == NS) {
      ss = 0;
      sph ^= 1u;
    }
  }
  __syncwarp();
}

// ---- the reduce role ----------------------------------------------------------
// Peer-load flavour: read the vector from every rank's ring, reduce in rank
// order (the same bits on every GPU), write the result into every rank's ring.
// U vectors per thread and step, at most KW ranks.
template <typename T, int U, int KW>
__device__ __forceinline__ void reducePeers(const PipeChannelDev& c, const PipeArgs& a, uint64_t base,
                                            int64_t n, int gtid) {
  constexpr int V = kVecBytes / sizeof(T);
  using Acc = typename Tr<T>::Acc;
  const int W = c.world;
  for (int64_t i0 = gtid; i0 < n; i0 += (int64_t)kRedThreads * U) {
    uint4 raw[U][KW];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t i = i0 + (int64_t)u * kRedThreads;
#pragma unroll
      for (int q = 0; q < KW; ++q)
        if (q < W && i < n) raw[u][q] = ldStage(c.ring[q] + base + i * kVecBytes);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t i = i0 + (int64_t)u * kRedThreads;
      if (i >= n) continue;
      Acc acc[V];
      unpack<T, V>(raw[u][0], acc);
#pragma unroll
      for (int q = 1; q < KW; ++q) {
        if (q < W) {
          Acc x[V];
          unpack<T, V>(raw[u][q], x);
#pragma unroll
          for (int e = 0; e < V; ++e) acc[e] = combine(acc[e], x[e], a.op);
        }
      }
      if constexpr (std::is_floating_point<Acc>::value) {
        if (a.scale != 1.0f) {
#pragma unroll
          for (int e = 0; e < V; ++e) acc[e] = acc[e] * (Acc)a.scale;
        }
      }
      const uint4 r = pack<T, V>(acc);
#pragma unroll
      for (int q = 0; q < KW; ++q)
        if (q < W) stStage(c.ring[(c.rank + q) % W] + base + i * kVecBytes, r);
    }
  }
}

template <typename T, bool NVLS>
__device__ __forceinline__ void reducePiece(const PipeChannelDev& c, const PipeArgs& a,
                                            uint64_t slot_off, int64_t first_vec, int64_t n,
                                            int gtid) {
  constexpr int V = kVecBytes / sizeof(T);
  using Acc = typename Tr<T>::Acc;
  const uint64_t base = slot_off + (uint64_t)first_vec * kVecBytes;
  if constexpr (NVLS) {
    constexpr int U = 8;
    char* mc = c.ring_mc + base;
    for (int64_t i0 = gtid; i0 < n; i0 += (int64_t)kRedThreads * U) {
      uint4 r[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int64_t i = i0 + (int64_t)u * kRedThreads;
        if (i < n) r[u] = multimemLdReduce<T>(mc + i * kVecBytes, a.op);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int64_t i = i0 + (int64_t)u * kRedThreads;
        if (i >= n) continue;
        if constexpr (std::is_floating_point<Acc>::value) {
          if (a.scale != 1.0f) {
            Acc x[V];
            unpack<T, V>(r[u], x);
#pragma unroll
            for (int e = 0; e < V; ++e) x[e] = x[e] * (Acc)a.scale;
            r[u] = pack<T, V>(x);
          }
        }
        multimemSt(mc + i * kVecBytes, r[u]);
      }
    }
  } else {
    // Eight 16-byte peer loads in flight per thread whatever the number of ranks.
    if (c.world <= 2)
      reducePeers<T, 4, 2>(c, a, base, n, gtid);
    else if (c.world <= 4)
      reducePeers<T, 2, 4>(c, a, base, n, gtid);
    else
      reducePeers<T, 1, kMaxRanks>(c, a, base, n, gtid);
  }
}

template <typename T, bool NVLS>
__device__ __forceinline__ void reduceRole(const PipeChannelDev& c, const PipeArgs& a, const Geo& g,
                                           Ctl* ctl, uint32_t g0, int group, int gtid) {
  const int bar_id = 1 + group;
  uint32_t* my_pad = c.flags[c.rank];
  // This group's first chunk, then every kNR-th one.
  int k = (int)((uint32_t)(group + kNR) - g0 % kNR) % kNR;
  int slot = (int)((g0 + (uint32_t)k) % (uint32_t)g.slots);
  for (; k < g.nchunks; k += kNR, slot = (slot + kNR) % g.slots) {
    const uint32_t gg = g0 + (uint32_t)k;
    bool bad = false;
    // 1. This block's copy-in of the chunk: wait for the copy warp's word, make
    //    the chunk visible to the other GPUs, raise the counter everywhere.
    if (gtid == 0) {
      uint64_t t0 = 0;
      for (uint64_t n = 1;; ++n) {
        if ((int32_t)(ctl->cin_done - (gg + 1u)) >= 0) break;
        if ((n & 255) == 0) {
          if (ctl->failed) {
            bad = true;
            break;
          }
          const uint64_t now = globalTimerNs();
          if (t0 == 0) t0 = now;
          if (now - t0 > 2 * c.timeout_ns || n > (1ull << 34)) {
            recordFailure(c, ctl, kStatusTimeout, kWaitCopyInLocal, (uint32_t)c.rank, gg);
            bad = true;
            break;
          }
        }
      }
      if (!bad) {
        // One system-scope fence, then a relaxed store per rank by the same
        // thread: an SM works its system-scope membars off one after the other.
        __threadfence_system();
        for (int q = 0; q < g.W; ++q) stRelaxedSys(counterAt(c.flags[q], group, c.rank, g.b), gg + 1u);
      }
    }
    // 2. Every rank's copy-in of the chunk.
    if (gtid < 32) {
      bad = __shfl_sync(0xffffffffu, (int)bad, 0) != 0;
      if (!bad && gtid < g.W)
        bad = !waitCounter(c, ctl, counterAt(my_pad, group, gtid, g.b), gg + 1u, kWaitCopyIn,
                           (uint32_t)gtid);
    }
    if (namedBarrierOr(bar_id, kRedThreads, bad || ctl->failed != 0)) break;
    const int64_t c_lo = (int64_t)k * g.cv;
    const Piece p = pieceAt(g, c_lo, c.rank, g.b);  // whole vectors, the padded tail vector included
    if (p.hi > p.lo)
      reducePiece<T, NVLS>(c, a, slotOffset(c, slot), p.lo - c_lo, p.hi - p.lo, gtid);
    if (namedBarrierOr(bar_id, kRedThreads, ctl->failed != 0)) break;
    if (gtid == 0) {
      __threadfence_system();
      for (int q = 0; q < g.W; ++q)
        stRelaxedSys(counterAt(c.flags[q], kNR + group, c.rank, g.b), gg + 1u);
    }
  }
}

template <typename T, bool NVLS>
__global__ void __launch_bounds__(kPipeThreads, 1)
pipe_allreduce(const PipeChannelDev* __restrict__ chs, const __grid_constant__ PipeArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  const PipeChannelDev& c = chs[blockIdx.y];
  Ctl* ctl = reinterpret_cast<Ctl*>(smem);
  unsigned char* stages = smem + 256;  // Ctl fits in 256 bytes
  static_assert(sizeof(Ctl) <= 256, "control block");

  Geo g;
  g.nvec = ceilDiv(a.nbytes, kVecBytes);
  g.tail = (int32_t)(a.nbytes % kVecBytes);
  g.cv = a.chunk_bytes / kVecBytes;
  g.nchunks = (int32_t)ceilDiv(g.nvec, g.cv);
  g.W = c.world;
  g.G = gridDim.x;
  g.b = blockIdx.x;
  g.slots = c.slots;
  g.sv = ceilDiv(g.cv, g.W);
  g.pv = ceilDiv(g.sv, g.G);
  const uint32_t g0 = c.seq[g.b];

  if (threadIdx.x == 0) {
    for (int r = 0; r < 2; ++r)
      for (int s = 0; s < a.stages; ++s) mbarInit(&ctl->full[r][s], 1);
    ctl->cout_done = g0;
    ctl->cin_done = g0;
    ctl->failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  const int warp = threadIdx.x >> 5;
  if (warp == 0) {
    copyRole<true>(c, a, g, ctl, stages, g0, static_cast<const char*>(a.in[blockIdx.y]), nullptr);
  } else if (warp == 1) {
    copyRole<false>(c, a, g, ctl, stages + (size_t)a.stages * a.stage_bytes, g0, nullptr,
                    static_cast<char*>(a.out[blockIdx.y]));
  } else {
    const int group = (warp - kFirstRedWarp) / kRedWarps;
    const int gtid = (int)threadIdx.x - (kFirstRedWarp + group * kRedWarps) * 32;
    reduceRole<T, NVLS>(c, a, g, ctl, g0, group, gtid);
  }
  __syncthreads();
  if (threadIdx.x == 0 && ctl->failed == 0) c.seq[g.b] = g0 + (uint32_t)g.nchunks;
}

using PipeFn = void (*)(const PipeChannelDev*, const PipeArgs);

template <bool NVLS>
PipeFn pick(DType t) {
  switch (t) {
    case DType::F32: return pipe_allreduce<float, NVLS>;
    case DType::BF16: return pipe_allreduce<__nv_bfloat16, NVLS>;
    case DType::F16: return pipe_allreduce<__half, NVLS>;
    default: break;
  }
  if constexpr (!NVLS) {
    switch (t) {
      case DType::U8: return pipe_allreduce<uint8_t, false>;
      case DType::I8: return pipe_allreduce<int8_t, false>;
      case DType::I32: return pipe_allreduce<int32_t, false>;
      case DType::I64: return pipe_allreduce<int64_t, false>;
      case DType::F64: return pipe_allreduce<double, false>;
      default: break;
    }
  }
  return nullptr;
}

}  // namespace pipe

size_t pipeSharedBytes(int stage_bytes, int stages) {
  return 256 + 2 * (size_t)stage_bytes * (size_t)stages;
}

namespace {
cudaError_t launchPipe(const PipeChannelDev* chs, const PipeArgs& a, int world_y, int blocks,
                       bool cooperative, cudaStream_t stream) {
  if (blocks < 1 || blocks > kMaxBlocks) return cudaErrorInvalidValue;
  if (a.stages < 2 || a.stages > pipe::kMaxStages || a.stage_bytes < kVecBytes ||
      a.stage_bytes % kVecBytes != 0)
    return cudaErrorInvalidValue;
  if (a.nbytes <= 0 || a.chunk_bytes < kVecBytes || a.chunk_bytes % kVecBytes != 0)
    return cudaErrorInvalidValue;
  if (a.nvls && !nvlsSupported((DType)a.dtype, (RedOp)a.op)) return cudaErrorInvalidValue;
  pipe::PipeFn fn = a.nvls ? pipe::pick<true>((DType)a.dtype) : pipe::pick<false>((DType)a.dtype);
  if (fn == nullptr) return cudaErrorInvalidDeviceFunction;
  const size_t smem = pipeSharedBytes(a.stage_bytes, a.stages);
  cudaError_t e = cudaFuncSetAttribute((const void*)fn, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)smem);
  if (e != cudaSuccess) return e;
  if (cooperative) {
    void* params[] = {(void*)&chs, (void*)&a};
    e = cudaLaunchCooperativeKernel((const void*)fn, dim3(blocks, world_y), dim3(kPipeThreads),
                                    params, smem, stream);
  } else {
    fn<<<dim3(blocks, world_y), dim3(kPipeThreads), smem, stream>>>(chs, a);
    e = cudaGetLastError();
  }
  if (e == cudaSuccess) countLaunch();
  return e;
}
}  // namespace

cudaError_t launchPipeAllreduce(const PipeChannelDev* ch_dev, const PipeArgs& args, int blocks,
                                cudaStream_t stream) {
  return launchPipe(ch_dev, args, 1, blocks, false, stream);
}

cudaError_t launchPipeEmulated(const PipeChannelDev* chs_dev, const PipeArgs& args, int world,
                               int blocks, cudaStream_t stream) {
  if (world < 1 || world > kMaxRanks || args.nvls) return cudaErrorInvalidValue;
  return launchPipe(chs_dev, args, world, blocks, true, stream);
}

}  // namespace fairring
