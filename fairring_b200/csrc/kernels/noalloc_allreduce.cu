// See noalloc_allreduce.h: the one-shot all-reduce with all of its scratch in
// a static device array, for callers that cannot allocate.
#include "noalloc_allreduce.h"

#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <mutex>

#include "kernels.h"

namespace {

using namespace fairring;

constexpr int kNaMaxRanks = 8;
constexpr long long kNaMaxElems = 4096;
constexpr size_t kNaHalfBytes = 160 * 1024;  // one-shot staging of 4096 floats from 8 ranks, with margin
constexpr size_t kNaFlagBytes = (size_t)kMaxRanks * kMaxBlocks * sizeof(uint32_t);
constexpr size_t kNaSeqBytes = (size_t)kMaxBlocks * sizeof(uint32_t);
constexpr int kNaMaxDevices = 64;

// Layout of the static array (offsets are multiples of 256 bytes).
// One channel table per world size 2..8, all written by the first call on a
// device, so that later calls only clear the flags and launch.
constexpr size_t kOffChannels = 0;                                              // [7 tables][ChannelDev[8]]
constexpr int kNaTables = kNaMaxRanks - 1;
constexpr size_t kNaTableBytes = 2560;
constexpr size_t kOffFlags = 20480;                                             // [8][kNaFlagBytes]
constexpr size_t kOffSeq = kOffFlags + kNaMaxRanks * kNaFlagBytes;              // [8][kNaSeqBytes]
constexpr size_t kOffStatus = kOffSeq + kNaMaxRanks * kNaSeqBytes;              // [8][4] words + abort word
constexpr size_t kOffStaging = kOffStatus + 256;                                // [8][kNaHalfBytes]
constexpr size_t kNaTotal = kOffStaging + kNaMaxRanks * kNaHalfBytes;
static_assert(sizeof(ChannelDev) * kNaMaxRanks <= kNaTableBytes, "a channel table must fit its slot");
static_assert(kNaTables * kNaTableBytes <= kOffFlags, "the tables must fit before the flags");
static_assert(kOffStaging % 256 == 0, "staging must stay 256-byte aligned");

// The scratch itself.  In host code this name is only a handle for
// cudaGetSymbolAddress; it is not a device address.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNaTotal];

struct PerDevice {
  unsigned char* base = nullptr;  // device address of g_noalloc_scratch on that device
  bool laid_out = false;          // the channel tables have been written there
};
PerDevice g_dev[kNaMaxDevices];
std::mutex g_mu;

int fail(int code, char* err, unsigned long err_len, const char* msg) {
  if (err != nullptr && err_len > 0) std::snprintf(err, err_len, "%s", msg);
  return code;
}

}  // namespace

extern "C" int fairring_allreduce_f32_noalloc(float* const* bufs, int world, long long numel,
                                              void* stream_v, int check, char* err,
                                              unsigned long err_len) {
  if (bufs == nullptr) return fail(1, err, err_len, "bufs is null");
  if (world < 2 || world > kNaMaxRanks)
    return fail(1, err, err_len, "world must be between 2 and 8 buffers");
  if (numel < 1 || numel > kNaMaxElems)
    return fail(1, err, err_len,
                "numel must be between 1 and 4096 elements: the static scratch array holds no more");
  for (int r = 0; r < world; ++r)
    if (bufs[r] == nullptr) return fail(1, err, err_len, "a buffer pointer is null");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(2, err, err_len, cudaGetErrorString(e));
  if (dev < 0 || dev >= kNaMaxDevices) return fail(1, err, err_len, "device index out of range");

  for (int r = 0; r < world; ++r) {
    cudaPointerAttributes attr;
    e = cudaPointerGetAttributes(&attr, bufs[r]);
    if (e != cudaSuccess) return fail(2, err, err_len, cudaGetErrorString(e));
    if (attr.type != cudaMemoryTypeDevice && attr.type != cudaMemoryTypeManaged)
      return fail(1, err, err_len, "a buffer is not device memory");
    if (attr.type == cudaMemoryTypeDevice && attr.device != dev)
      return fail(1, err, err_len, "a buffer lives on another device than the current one");
  }

  std::lock_guard<std::mutex> lk(g_mu);
  PerDevice& pd = g_dev[dev];
  if (pd.base == nullptr) {
    // First call on this device: find where the static array lives there.
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) return fail(2, err, err_len, cudaGetErrorString(e));
    pd.base = static_cast<unsigned char*>(p);
    pd.laid_out = false;
  }
  unsigned char* base = pd.base;

  if (!pd.laid_out) {
    // Still the first call: write, for every world size, the table that tells
    // each emulated rank where its peers' staging and flags are.  Pageable-host
    // to device copies: staged by the driver, nothing is allocated.  The stream
    // is synchronised because the tables are built on this stack frame.
    for (int w = 2; w <= kNaMaxRanks; ++w) {
      ChannelDev chs[kNaMaxRanks];
      std::memset(chs, 0, sizeof(chs));
      for (int r = 0; r < w; ++r) {
        ChannelDev& c = chs[r];
        for (int p = 0; p < w; ++p) {
          c.staging[p] = reinterpret_cast<char*>(base + kOffStaging + (size_t)p * kNaHalfBytes);
          c.flags[p] = reinterpret_cast<uint32_t*>(base + kOffFlags + (size_t)p * kNaFlagBytes);
        }
        c.mc_staging = nullptr;
        c.seq = reinterpret_cast<uint32_t*>(base + kOffSeq + (size_t)r * kNaSeqBytes);
        c.status = reinterpret_cast<uint32_t*>(base + kOffStatus) + (size_t)r * kStatusWords;
        c.abort_flag = reinterpret_cast<uint32_t*>(base + kOffStatus) + kNaMaxRanks * kStatusWords;
        c.half_bytes = kNaHalfBytes;
        c.timeout_ns = 2ull * 1000 * 1000 * 1000;
        c.topo = makeTopo(w, w, false, r);
      }
      e = cudaMemcpyAsync(base + kOffChannels + (size_t)(w - 2) * kNaTableBytes, chs,
                          sizeof(ChannelDev) * w, cudaMemcpyHostToDevice, stream);
      if (e != cudaSuccess) return fail(2, err, err_len, cudaGetErrorString(e));
      e = cudaStreamSynchronize(stream);
      if (e != cudaSuccess) return fail(2, err, err_len, cudaGetErrorString(e));
    }
    pd.laid_out = true;
  }

  // The array keeps whatever the previous call left: flags, sequence counters
  // and status must start from zero (the staging need not: it is overwritten
  // before it is read).
  e = cudaMemsetAsync(base + kOffFlags, 0, kOffStaging - kOffFlags, stream);
  if (e != cudaSuccess) return fail(2, err, err_len, cudaGetErrorString(e));

  OpArgs a;
  std::memset(&a, 0, sizeof(a));
  for (int r = 0; r < world; ++r) {
    a.in[r] = bufs[r];
    a.out[r] = bufs[r];
  }
  a.seg = allreduceSeg(numel, (int)sizeof(float), world);
  a.scale = 1.0f;
  a.op = (int32_t)RedOp::SUM;
  a.io_dtype = a.wire_dtype = (int32_t)DType::F32;
  a.flags = kAdvanceSeq;
  if ((size_t)world * world * a.seg.qv * kVecBytes > kNaHalfBytes)
    return fail(1, err, err_len, "message does not fit the static staging area");
  e = launchEmulated(KernelId::ONESHOT,
                     reinterpret_cast<const ChannelDev*>(base + kOffChannels +
                                                         (size_t)(world - 2) * kNaTableBytes),
                     a, world, /*blocks=*/2, stream);
  if (e != cudaSuccess) return fail(2, err, err_len, cudaGetErrorString(e));

  if (check) {
    uint32_t status[kNaMaxRanks * kStatusWords];
    e = cudaMemcpyAsync(status, base + kOffStatus, sizeof(status), cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return fail(2, err, err_len, cudaGetErrorString(e));
    for (int r = 0; r < world; ++r)
      if (status[r * kStatusWords] != kStatusOk)
        return fail(3, err, err_len, "a wait inside the kernel ran into its time limit");
  }
  return 0;
}
