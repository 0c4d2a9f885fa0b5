// Host side of the collective kernels: picks the instantiation for a (tensor
// dtype, wire dtype) pair and launches it.  The device code is in
// collectives_impl.cuh, instantiated once per pair in collectives_<pair>.cu.
#include <cuda_runtime.h>

#include <atomic>

#include "kernels.h"

namespace fairring {

using KernelFn = void (*)(const ChannelDev*, const OpArgs);
KernelFn lookupKernel_u8(KernelId id);
KernelFn lookupKernel_i8(KernelId id);
KernelFn lookupKernel_i32(KernelId id);
KernelFn lookupKernel_i64(KernelId id);
KernelFn lookupKernel_f16(KernelId id);
KernelFn lookupKernel_bf16(KernelId id);
KernelFn lookupKernel_f32(KernelId id);
KernelFn lookupKernel_f64(KernelId id);
KernelFn lookupKernel_f32_bf16(KernelId id);
KernelFn lookupKernel_f32_f16(KernelId id);

namespace {

KernelFn lookup(DType io, DType wire, KernelId id) {
  if (io == DType::U8 && wire == DType::U8) return lookupKernel_u8(id);
  if (io == DType::I8 && wire == DType::I8) return lookupKernel_i8(id);
  if (io == DType::I32 && wire == DType::I32) return lookupKernel_i32(id);
  if (io == DType::I64 && wire == DType::I64) return lookupKernel_i64(id);
  if (io == DType::F16 && wire == DType::F16) return lookupKernel_f16(id);
  if (io == DType::BF16 && wire == DType::BF16) return lookupKernel_bf16(id);
  if (io == DType::F32 && wire == DType::F32) return lookupKernel_f32(id);
  if (io == DType::F64 && wire == DType::F64) return lookupKernel_f64(id);
  if (io == DType::F32 && wire == DType::BF16) return lookupKernel_f32_bf16(id);
  if (io == DType::F32 && wire == DType::F16) return lookupKernel_f32_f16(id);
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
    case KernelId::P2P_DIRECT: return "direct_allreduce";
    case KernelId::NVLS_DIRECT: return "nvls_direct_allreduce";
    case KernelId::LL_ONESHOT: return "ll_allreduce";
    case KernelId::LL_TWOSHOT: return "ll2_allreduce";
    case KernelId::PIPE: return "pipe_allreduce";
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

namespace {
cudaError_t launchImpl(KernelId id, const ChannelDev* chs, const OpArgs& args, int world_y,
                       int blocks, bool cooperative, cudaStream_t stream) {
  if (blocks < 1 || blocks > kMaxBlocks) return cudaErrorInvalidValue;
  KernelFn fn = lookup((DType)args.io_dtype, (DType)args.wire_dtype, id);
  if (fn == nullptr) return cudaErrorInvalidDeviceFunction;
  if ((id == KernelId::NVLS_TWOSHOT || id == KernelId::NVLS_ONESHOT ||
       id == KernelId::NVLS_DIRECT) &&
      !nvlsSupported((DType)args.wire_dtype, (RedOp)args.op))
    return cudaErrorInvalidValue;
  if (id == KernelId::NVLS_DIRECT && args.mc == nullptr) return cudaErrorInvalidValue;
  if (id == KernelId::PIPE) return cudaErrorInvalidValue;  // launched through launchPipeAllreduce
  cudaError_t e;
  if (cooperative) {
    // All blocks of all emulated ranks wait on one another: they must be
    // resident together, which only a cooperative launch guarantees.
    void* params[] = {(void*)&chs, (void*)&args};
    e = cudaLaunchCooperativeKernel((const void*)fn, dim3(blocks, world_y), dim3(kThreads), params,
                                    0, stream);
  } else {
    fn<<<dim3(blocks, world_y), dim3(kThreads), 0, stream>>>(chs, args);
    e = cudaGetLastError();
  }
  if (e == cudaSuccess) g_launches.fetch_add(1, std::memory_order_relaxed);
  return e;
}
}  // namespace

cudaError_t launchCollective(KernelId id, const ChannelDev* ch_dev, const OpArgs& args, int blocks,
                             cudaStream_t stream) {
  return launchImpl(id, ch_dev, args, 1, blocks, false, stream);
}

cudaError_t launchEmulated(KernelId id, const ChannelDev* chs_dev, const OpArgs& args, int world,
                           int blocks, cudaStream_t stream) {
  if (world < 1 || world > kMaxRanks) return cudaErrorInvalidValue;
  if (id == KernelId::NVLS_TWOSHOT || id == KernelId::NVLS_ONESHOT || id == KernelId::NVLS_DIRECT)
    return cudaErrorInvalidValue;  // multicast needs one GPU per rank
  return launchImpl(id, chs_dev, args, world, blocks, true, stream);
}

uint64_t launchCount() { return g_launches.load(std::memory_order_relaxed); }
void countLaunch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

}  // namespace fairring
