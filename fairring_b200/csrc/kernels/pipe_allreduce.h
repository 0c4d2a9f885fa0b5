// Host interface of the pipelined all-reduce for ordinary (not peer-mapped)
// tensors.
//
// The message is cut into chunks.  Three roles inside every thread block work
// on different chunks at the same time:
//
//   copy-in   one warp; bulk-copies (cp.async.bulk through shared memory, one
//             elected thread) this block's pieces of chunk k from the user's
//             tensor into this GPU's slot of a ring of symmetric staging memory
//   reduce    fourteen warps in seven groups that take chunks in turn.  The
//             group of chunk g first publishes this block's copy-in of g (it
//             waits for copy-in's word in shared memory, fences, raises the
//             counter on every rank), then waits for every rank's counter and
//             reduces.  A system-scope fence on an SM that is streaming bulk
//             stores takes some ten microseconds: it must stall neither the
//             copy warps nor the other chunks, so every chunk's fences belong
//             to its own group and seven chunks are in flight.  Rank r reduces
//             sub-chunk r of the chunk over all GPUs and writes the result back
//             into every GPU's ring slot (multimem.ld_reduce + multimem.st
//             through the NVSwitch, or peer loads + peer stores)
//   copy-out  one warp; bulk-copies the reduced chunk from this GPU's ring slot
//             into the user's tensor
//
// Block b of every rank owns the same byte ranges of every chunk, so the roles
// of block b only ever wait for block b of the peers: per-(rank, block)
// counters in symmetric memory, written with release stores after the data,
// say "rank q, block b has copied in chunk g" and "... has reduced chunk g".
// Each group has its own pair of counters (chunks of different groups may
// finish out of order; a counter only ever grows).
// Chunks are numbered across launches, a ring slot is reused every `slots`
// chunks, and copy-in of chunk g waits for this block's copy-out of chunk
// g - slots, which in turn has waited for every peer's reduce of that chunk:
// no barrier is needed between consecutive all-reduces of a channel.
//
// This one launch does what the reference does per slice with five library
// calls on five streams (fairring/device.cc:444-634), with the stages of
// consecutive chunks overlapping inside the kernel.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

#include "../layout.h"

namespace fairring {

constexpr int kPipeRedGroups = 7;                  // reduce groups (2 warps each) taking chunks in turn
constexpr int kPipeLanes = 2 * kPipeRedGroups;     // counters per (rank, block): copied-in and reduced, per group
constexpr size_t kPipeFlagBytes = (size_t)kPipeLanes * kMaxRanks * kMaxBlocks * sizeof(uint32_t);
constexpr int kPipeThreads = 512;                  // copy-in warp, copy-out warp, 7 x 2 reduce warps

// One channel as seen by one rank; lives in device memory.
struct PipeChannelDev {
  char* ring[kMaxRanks];      // rank p's ring as mapped here: [slots][slot_bytes]
  char* ring_mc;              // multicast alias of the ring, or null
  uint32_t* flags[kMaxRanks]; // rank p's counters: [kPipeLanes][source rank][block]
  uint32_t* seq;              // local, [kMaxBlocks]: chunks this block has completed so far
  uint32_t* status;           // host-mapped, kStatusWords words, 0 == healthy
  const uint32_t* abort_flag; // host-mapped; non-zero makes every wait give up
  uint64_t slot_bytes;        // bytes of one ring slot (multiple of 16)
  uint64_t timeout_ns;        // limit of one wait
  int32_t slots;              // ring length
  int32_t world;
  int32_t rank;
  int32_t pad_;
};

struct PipeArgs {
  // Entry 0 in a real job; one entry per rank when all ranks are emulated on one GPU.
  const void* in[kMaxRanks];
  void* out[kMaxRanks];
  int64_t nbytes;       // message bytes; in/out are 16-byte aligned
  int64_t chunk_bytes;  // multiple of 16, at most slot_bytes
  float scale;          // applied to the reduced value (floating types)
  int32_t op;           // RedOp
  int32_t dtype;        // DType of the tensor (and of the wire)
  int32_t nvls;         // 1: reduce through the multicast address
  int32_t stage_bytes;  // bytes of one shared-memory stage (multiple of 16)
  int32_t stages;       // stages per copy role
};

// Shared memory the kernel needs for (stage_bytes, stages).
size_t pipeSharedBytes(int stage_bytes, int stages);

// One rank per process.  `ch_dev` points to the channel in device memory.
cudaError_t launchPipeAllreduce(const PipeChannelDev* ch_dev, const PipeArgs& args, int blocks,
                                cudaStream_t stream);
// All ranks in one cooperative launch on one GPU (grid.y = rank); peer-load
// flavour only.
cudaError_t launchPipeEmulated(const PipeChannelDev* chs_dev, const PipeArgs& args, int world,
                               int blocks, cudaStream_t stream);

}  // namespace fairring
