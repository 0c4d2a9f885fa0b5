// Host-visible interface of the sm_100a collective kernels.  Nothing here
// depends on torch; the engine fills these PODs and calls launch*().
//
// The kernels replace the library calls the reference strings together per
// slice (fairring/device.cc:444-634: ncclReduceScatter, ncclSend/ncclRecv,
// at::sum_out, ncclSend/ncclRecv, ncclAllGather) with loads and stores on peer
// GPUs' staging memory issued from inside the kernel.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

#include "../layout.h"

namespace fairring {

// Everything one channel's kernels need to reach their peers.  Built once,
// kept in device memory and passed by pointer.  A channel owns one staging
// slot (two halves used alternately by consecutive collectives), one flag pad
// and one stream.
struct ChannelDev {
  char* staging[kMaxRanks];     // rank p's slot as mapped in this process
  uint32_t* flags[kMaxRanks];   // rank p's flag pad: [source rank][block]
  char* mc_staging;             // NVLS multicast alias of the slot, or null
  char* ll[kMaxRanks];          // rank p's flag-in-data area (two halves), or null
  uint64_t ll_half_bytes;       // bytes of one half of that area
  uint32_t* seq;                // local, [kMaxBlocks]: collectives done by block b
  uint32_t* status;             // host-mapped, kStatusWords words, 0 == healthy
  const uint32_t* abort_flag;   // host-mapped; non-zero makes every wait give up
  uint64_t half_bytes;
  uint64_t timeout_ns;          // limit of one wait on a peer
  Topo topo;
};

constexpr int kStatusWords = 4;  // code, barrier index, peer, sequence number
enum StatusCode : uint32_t { kStatusOk = 0, kStatusTimeout = 1, kStatusAborted = 2 };

enum OpFlags : uint32_t {
  kToUser = 1u << 0,      // reduced data goes to `out`, not to staging (reduce_scatter)
  kAdvanceSeq = 1u << 1,  // last kernel of the collective: bump the sequence number
};

struct OpArgs {
  // Slice base in the user's input / output (may alias).  Entry 0 in a real
  // job; one entry per rank when all ranks are emulated on one GPU.
  const void* in[kMaxRanks];
  void* out[kMaxRanks];
  // Direct (zero-copy) kernels only: the tensor lives in symmetric memory, so
  // every rank's copy of it is addressable.  peer[p] is rank p's copy of the
  // slice as mapped here, mc its multicast alias (or null).
  void* peer[kMaxRanks];
  void* mc;
  Seg seg;
  float scale;      // multiplied in while the data is first read (floating types)
  int32_t op;       // RedOp
  int32_t io_dtype;    // DType of in/out
  int32_t wire_dtype;  // DType held in staging and sent over NVLink
  uint32_t flags;      // OpFlags
  int32_t unroll;      // in-place NVLS kernel: 16-byte accesses in flight per thread (4, 8, 16)
  int32_t full_blocks;  // blocks of the channel's widest launch; a narrower launch advances the
                        // collective counts of the blocks that it does not run (0: none to advance)
};

enum class KernelId : int32_t {
  ONESHOT = 0,          // push everything to everyone, one barrier, local reduce
  TWOSHOT,              // rs_intragroup + ag_intragroup in one launch (M == 1)
  RS_INTRAGROUP,        // push to group peers, reduce own rail chunks into the self slot
  SHARD_SERVER_REDUCE,  // pull own shard from rail peers, reduce, push it back to them
  AG_INTRAGROUP,        // pull reduced rail chunks from group peers into the user tensor
  DIFFUSE,              // all_gather stage 1: own chunk -> self slot of every rail peer
  NVLS_TWOSHOT,         // multimem.ld_reduce own chunk, multimem.st it to all
  NVLS_ONESHOT,         // multimem.ld_reduce the whole message
  P2P_DIRECT,           // in place on symmetric memory: pull + reduce own chunk, push it to all
  NVLS_DIRECT,          // in place on symmetric memory: multimem.ld_reduce + multimem.st
  LL_ONESHOT,           // small messages: every 16-byte store carries 8 bytes of data and two
                        // copies of the collective's number; receivers spin on the data itself
  LL_TWOSHOT,           // the same words, reduce-scattered and all-gathered (mid-size messages)
  PIPE,                 // ordinary tensors: copy-in / reduce / copy-out pipelined over chunks
                        // (pipe_allreduce.h; counted here, launched through launchPipeAllreduce)
  kCount
};

const char* kernelName(KernelId id);

// Which (io, wire) pairs have kernels: io == wire for all eight dtypes, plus
// fp32 tensors carried as bf16 or fp16 on the wire.
bool comboSupported(DType io, DType wire);
// multimem.ld_reduce exists only for some (dtype, op) pairs.
bool nvlsSupported(DType wire, RedOp op);

constexpr int kThreads = 512;

// One rank per process: the usual launch.  `ch_dev` points to the channel's
// description in device memory; args.in[0] / args.out[0] are used.
cudaError_t launchCollective(KernelId id, const ChannelDev* ch_dev, const OpArgs& args,
                             int blocks, cudaStream_t stream);

// All `world` ranks inside one cooperative launch on one GPU (grid.y = rank):
// how the multi-rank logic is exercised when fewer GPUs than ranks are at hand.
// `chs_dev` is a device array of `world` channel descriptions; args.in[r] /
// args.out[r] are rank r's tensors.
cudaError_t launchEmulated(KernelId id, const ChannelDev* chs_dev, const OpArgs& args,
                           int world, int blocks, cudaStream_t stream);

// Number of kernels this library has launched in this process.
uint64_t launchCount();
// Adds one to that number (for kernels launched outside launchCollective).
void countLaunch();

}  // namespace fairring
