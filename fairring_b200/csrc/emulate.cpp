// Runs a whole multi-rank collective on ONE GPU: every rank's staging, flags
// and tensors live on the same device and one cooperative launch carries the
// blocks of all ranks (grid.y = rank).  The kernels' code is the same as in a
// real job; only the peer pointers happen to be local.  This is how the
// kernels are tested where fewer GPUs than ranks are available, and how a
// timed-out wait is demonstrated without a second process: a "silent" rank's
// signals are redirected into a scratch pad that nobody reads.
#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include <cstdlib>
#include <tuple>
#include <vector>

#include "check.h"
#include "engine.h"
#include "kernels/kernels.h"
#include "kernels/pipe_allreduce.h"

namespace fairring {

namespace {
bool toDTypeEmu(at::ScalarType st, DType* out) {
  switch (st) {
    case at::kByte: *out = DType::U8; return true;
    case at::kChar: *out = DType::I8; return true;
    case at::kInt: *out = DType::I32; return true;
    case at::kLong: *out = DType::I64; return true;
    case at::kHalf: *out = DType::F16; return true;
    case at::kBFloat16: *out = DType::BF16; return true;
    case at::kFloat: *out = DType::F32; return true;
    case at::kDouble: *out = DType::F64; return true;
    default: return false;
  }
}
}  // namespace

// kind: "allreduce" | "reduce_scatter" | "allgather"
// algo: "oneshot" | "twoshot" | "hier" (hier = the three-kernel pipeline; valid for M == 1 too)
// Returns (outputs, status words [world][kStatusWords]).
std::tuple<std::vector<at::Tensor>, at::Tensor> emulatedCollective(
    const std::string& kind, std::vector<at::Tensor> inputs, int64_t gpus_per_machine,
    bool favorable, const std::string& op, double scale, c10::optional<at::ScalarType> wire_dtype,
    const std::string& algo, int64_t blocks, int64_t half_bytes, int64_t timeout_ms,
    int64_t silent_rank, int64_t repeats) {
  const int W = (int)inputs.size();
  TORCH_CHECK(W >= 1 && W <= kMaxRanks, "1..", kMaxRanks, " emulated ranks");
  TORCH_CHECK(gpus_per_machine >= 1 && W % gpus_per_machine == 0, "grouping must divide the world");
  TORCH_CHECK(blocks >= 1 && blocks <= kMaxBlocks, "blocks out of range");
  for (auto& t : inputs)
    TORCH_CHECK(t.is_cuda() && t.device() == inputs[0].device() && t.is_contiguous() &&
                    t.scalar_type() == inputs[0].scalar_type() && t.numel() == inputs[0].numel(),
                "emulated ranks need same-shaped contiguous tensors on one GPU");
  c10::cuda::CUDAGuard guard(inputs[0].device());
  auto stream = c10::cuda::getCurrentCUDAStream();

  DType io, wire;
  TORCH_CHECK(toDTypeEmu(inputs[0].scalar_type(), &io), "unsupported dtype");
  wire = io;
  if (wire_dtype.has_value()) TORCH_CHECK(toDTypeEmu(*wire_dtype, &wire), "unsupported wire dtype");
  TORCH_CHECK(comboSupported(io, wire), "unsupported (dtype, wire dtype) pair");
  RedOp rop = op == "max" ? RedOp::MAX : (op == "min" ? RedOp::MIN : RedOp::SUM);
  const int wes = dtypeSize(wire);
  const int64_t V = kVecBytes / wes;

  const bool is_ar = kind == "allreduce", is_rs = kind == "reduce_scatter", is_ag = kind == "allgather";
  TORCH_CHECK(is_ar || is_rs || is_ag, "unknown collective ", kind);
  const int64_t n_in = inputs[0].numel();
  TORCH_CHECK(!is_rs || n_in % W == 0, "reduce_scatter input must be world * n");
  const int64_t per_rank = is_rs ? n_in / W : n_in;

  auto bopt = inputs[0].options();
  auto u8 = bopt.dtype(at::kByte);
  auto i32 = bopt.dtype(at::kInt);
  std::vector<at::Tensor> staging, flags, seqs, outs, lls;
  // flag-in-data areas: two halves of [rank][unit] 16-byte words
  const int64_t ll_msg = (algo == "ll" || algo == "ll2") ? n_in * dtypeSize(io) : 8;
  const int64_t ll_half = std::max<int64_t>((int64_t)kMaxRanks * roundUp(ceilDiv(ll_msg, 8), 64) * 16,
                                            4 * ll_msg + 32 * kMaxRanks * 64);
  for (int r = 0; r < W; ++r) {
    lls.push_back(at::zeros({2 * ll_half}, u8));
    staging.push_back(at::zeros({2 * half_bytes}, u8));
    flags.push_back(at::zeros({kMaxRanks * kMaxBlocks}, i32));
    seqs.push_back(at::zeros({kMaxBlocks}, i32));
    if (is_ar) outs.push_back(inputs[r]);  // in place, like the real thing
    else if (is_rs) outs.push_back(at::zeros({per_rank}, bopt));
    else outs.push_back(at::zeros({per_rank * W}, bopt));
  }
  at::Tensor scratch = at::zeros({kMaxRanks * kMaxBlocks}, i32);
  at::Tensor ll_scratch = at::zeros({2 * ll_half}, u8);
  uint32_t* status_host = nullptr;
  FR_CUDA(cudaHostAlloc((void**)&status_host, sizeof(uint32_t) * (W * kStatusWords + 1),
                        cudaHostAllocMapped));
  std::memset(status_host, 0, sizeof(uint32_t) * (W * kStatusWords + 1));
  uint32_t* status_dev = nullptr;
  FR_CUDA(cudaHostGetDevicePointer((void**)&status_dev, status_host, 0));

  std::vector<ChannelDev> chs(W);
  for (int r = 0; r < W; ++r) {
    ChannelDev& c = chs[r];
    std::memset(&c, 0, sizeof(c));
    for (int p = 0; p < W; ++p) {
      c.staging[p] = static_cast<char*>(staging[p].data_ptr());
      c.flags[p] = static_cast<uint32_t*>(flags[p].data_ptr());
      c.ll[p] = static_cast<char*>(lls[p].data_ptr());
      if (r == silent_rank && p != r) {
        c.flags[p] = static_cast<uint32_t*>(scratch.data_ptr());
        c.ll[p] = static_cast<char*>(ll_scratch.data_ptr());
      }
    }
    c.ll_half_bytes = (uint64_t)ll_half;
    c.mc_staging = nullptr;
    c.seq = static_cast<uint32_t*>(seqs[r].data_ptr());
    c.status = status_dev + r * kStatusWords;
    c.abort_flag = status_dev + W * kStatusWords;
    c.half_bytes = (uint64_t)half_bytes;
    c.timeout_ns = (uint64_t)timeout_ms * 1000000ull;
    c.topo = makeTopo(W, (int)gpus_per_machine, favorable, r);
  }
  const Topo t0 = chs[0].topo;
  at::Tensor chs_dev = at::empty({(int64_t)(sizeof(ChannelDev) * W)}, u8);
  FR_CUDA(cudaMemcpyAsync(chs_dev.data_ptr(), chs.data(), sizeof(ChannelDev) * W,
                          cudaMemcpyHostToDevice, stream));

  auto launchAll = [&](KernelId id, const Seg& seg, int64_t in_off, int64_t out_off, uint32_t fl) {
    const int ies = dtypeSize(io);
    OpArgs a;
    std::memset(&a, 0, sizeof(a));
    for (int r = 0; r < W; ++r) {
      a.in[r] = static_cast<const char*>(inputs[r].data_ptr()) + in_off * ies;
      a.out[r] = static_cast<char*>(outs[r].data_ptr()) + out_off * ies;
    }
    a.seg = seg;
    a.scale = (float)scale;
    a.op = (int32_t)rop;
    a.io_dtype = (int32_t)io;
    a.wire_dtype = (int32_t)wire;
    a.flags = fl;
    cudaError_t e = launchEmulated(id, static_cast<const ChannelDev*>(chs_dev.data_ptr()), a, W,
                                   (int)blocks, stream);
    TORCH_CHECK(e == cudaSuccess, "emulated launch of ", kernelName(id), " failed: ",
                cudaGetErrorString(e));
  };

  for (int64_t rep = 0; rep < repeats; ++rep) {
    if (is_ar) {
      if (algo == "direct") {
        // In place on the ranks' own tensors: what the engine does for tensors
        // in symmetric memory.
        TORCH_CHECK(io == wire && (n_in * wes) % kVecBytes == 0, "direct needs whole vectors");
        OpArgs a;
        std::memset(&a, 0, sizeof(a));
        for (int r = 0; r < W; ++r) {
          TORCH_CHECK((reinterpret_cast<uintptr_t>(inputs[r].data_ptr()) & 15u) == 0, "misaligned");
          a.peer[r] = inputs[r].data_ptr();
          a.in[r] = a.out[r] = inputs[r].data_ptr();
        }
        a.seg = allreduceSeg(n_in, wes, W);
        a.scale = (float)scale;
        a.op = (int32_t)rop;
        a.io_dtype = a.wire_dtype = (int32_t)io;
        a.flags = kAdvanceSeq;
        cudaError_t e = launchEmulated(KernelId::P2P_DIRECT,
                                       static_cast<const ChannelDev*>(chs_dev.data_ptr()), a, W,
                                       (int)blocks, stream);
        TORCH_CHECK(e == cudaSuccess, "emulated direct launch failed: ", cudaGetErrorString(e));
      } else if (algo == "ll" || algo == "ll2") {
        TORCH_CHECK(io == wire, "the flag-in-data kernels carry the tensor's own dtype");
        launchAll(algo == "ll" ? KernelId::LL_ONESHOT : KernelId::LL_TWOSHOT,
                  allreduceSeg(n_in, wes, W), 0, 0, kAdvanceSeq);
      } else if (algo == "oneshot") {
        const Seg s = allreduceSeg(n_in, wes, W);
        TORCH_CHECK((int64_t)W * W * s.qv * kVecBytes <= half_bytes, "message too large for one-shot");
        launchAll(KernelId::ONESHOT, s, 0, 0, kAdvanceSeq);
      } else {
        const SlicePlan sp = planSlices(n_in, wes, W, roundDown(half_bytes, (int64_t)kVecBytes * W));
        for (int64_t k = 0; k < sp.num_slices; ++k) {
          const int64_t off = k * sp.slice_elems;
          const int64_t n = std::min(sp.slice_elems, n_in - off);
          const Seg s = allreduceSeg(n, wes, W);
          if (algo == "twoshot") {
            TORCH_CHECK(t0.M == 1, "twoshot is the flat (one machine) kernel");
            launchAll(KernelId::TWOSHOT, s, off, off, kAdvanceSeq);
          } else {
            launchAll(KernelId::RS_INTRAGROUP, s, off, off, 0);
            if (t0.M > 1) launchAll(KernelId::SHARD_SERVER_REDUCE, s, off, off, 0);
            launchAll(KernelId::AG_INTRAGROUP, s, off, off, kAdvanceSeq);
          }
        }
      }
    } else {
      int64_t max_len = roundDown(roundDown(half_bytes, (int64_t)kVecBytes * W) / wes / W, V);
      if (max_len < V) max_len = V;
      for (int64_t off = 0; off < per_rank; off += max_len) {
        const int64_t len = std::min(max_len, per_rank - off);
        const Seg s = scatterSeg(len, per_rank, wes);
        if (is_rs) {
          if (t0.M == 1) {
            launchAll(KernelId::RS_INTRAGROUP, s, off, off, kToUser | kAdvanceSeq);
          } else {
            launchAll(KernelId::RS_INTRAGROUP, s, off, off, 0);
            launchAll(KernelId::SHARD_SERVER_REDUCE, s, off, off, kToUser | kAdvanceSeq);
          }
        } else {
          launchAll(KernelId::DIFFUSE, s, off, off, 0);
          launchAll(KernelId::AG_INTRAGROUP, s, off, off, kAdvanceSeq);
        }
      }
    }
  }
  FR_CUDA(cudaStreamSynchronize(stream));
  at::Tensor status = at::zeros({W, kStatusWords}, at::kInt);
  std::memcpy(status.data_ptr(), status_host, sizeof(uint32_t) * W * kStatusWords);
  cudaFreeHost(status_host);
  return std::make_tuple(outs, status);
}

// Device time per launch of the last emulatedPipeAllreduce call (CUDA events
// around the launches only), for kernel timing on one GPU.
static double g_last_emulated_us = 0;
double lastEmulatedUs() { return g_last_emulated_us; }

// The pipelined all-reduce (kernels/pipe_allreduce.h) with all ranks on one GPU,
// peer-load flavour.  Every launch all-reduces the inputs in place; `repeats`
// launches run back to back on one ring, so that chunk numbering and ring reuse
// carry over from one launch to the next as they do in a real job.
// Returns (inputs after the last launch, status words [world][kStatusWords]).
std::tuple<std::vector<at::Tensor>, at::Tensor> emulatedPipeAllreduce(
    std::vector<at::Tensor> inputs, const std::string& op, double scale, int64_t blocks,
    int64_t chunk_bytes, int64_t slot_bytes, int64_t slots, int64_t stage_bytes, int64_t stages,
    int64_t timeout_ms, int64_t silent_rank, int64_t repeats) {
  const int W = (int)inputs.size();
  TORCH_CHECK(W >= 1 && W <= kMaxRanks, "1..", kMaxRanks, " emulated ranks");
  TORCH_CHECK(blocks >= 1 && blocks <= kMaxBlocks, "blocks out of range");
  TORCH_CHECK(chunk_bytes % kVecBytes == 0 && chunk_bytes > 0 && chunk_bytes <= slot_bytes,
              "chunk must be whole vectors and fit a ring slot");
  TORCH_CHECK(slots >= 2, "the ring needs at least two slots");
  for (auto& t : inputs)
    TORCH_CHECK(t.is_cuda() && t.device() == inputs[0].device() && t.is_contiguous() &&
                    t.scalar_type() == inputs[0].scalar_type() && t.numel() == inputs[0].numel() &&
                    (reinterpret_cast<uintptr_t>(t.data_ptr()) & 15u) == 0,
                "emulated ranks need same-shaped contiguous 16-byte aligned tensors on one GPU");
  c10::cuda::CUDAGuard guard(inputs[0].device());
  auto stream = c10::cuda::getCurrentCUDAStream();
  DType dt;
  TORCH_CHECK(toDTypeEmu(inputs[0].scalar_type(), &dt), "unsupported dtype");
  const RedOp rop = op == "max" ? RedOp::MAX : (op == "min" ? RedOp::MIN : RedOp::SUM);

  auto u8 = inputs[0].options().dtype(at::kByte);
  auto i32 = inputs[0].options().dtype(at::kInt);
  std::vector<at::Tensor> rings, flags, seqs;
  for (int r = 0; r < W; ++r) {
    rings.push_back(at::zeros({slots * slot_bytes}, u8));
    flags.push_back(at::zeros({(int64_t)(kPipeFlagBytes / sizeof(uint32_t))}, i32));
    seqs.push_back(at::zeros({kMaxBlocks}, i32));
  }
  at::Tensor scratch = at::zeros({(int64_t)(kPipeFlagBytes / sizeof(uint32_t))}, i32);
  uint32_t* status_host = nullptr;
  FR_CUDA(cudaHostAlloc((void**)&status_host, sizeof(uint32_t) * (W * kStatusWords + 1),
                        cudaHostAllocMapped));
  std::memset(status_host, 0, sizeof(uint32_t) * (W * kStatusWords + 1));
  uint32_t* status_dev = nullptr;
  FR_CUDA(cudaHostGetDevicePointer((void**)&status_dev, status_host, 0));

  std::vector<PipeChannelDev> chs(W);
  for (int r = 0; r < W; ++r) {
    PipeChannelDev& c = chs[r];
    std::memset(&c, 0, sizeof(c));
    for (int p = 0; p < W; ++p) {
      c.ring[p] = static_cast<char*>(rings[p].data_ptr());
      c.flags[p] = static_cast<uint32_t*>(flags[p].data_ptr());
      // A silent rank's counters land in a pad nobody reads.
      if (r == silent_rank && p != r) c.flags[p] = static_cast<uint32_t*>(scratch.data_ptr());
    }
    c.ring_mc = nullptr;
    c.seq = static_cast<uint32_t*>(seqs[r].data_ptr());
    c.status = status_dev + r * kStatusWords;
    c.abort_flag = status_dev + W * kStatusWords;
    c.slot_bytes = (uint64_t)slot_bytes;
    c.timeout_ns = (uint64_t)timeout_ms * 1000000ull;
    c.slots = (int32_t)slots;
    c.world = W;
    c.rank = r;
  }
  at::Tensor chs_dev = at::empty({(int64_t)(sizeof(PipeChannelDev) * W)}, u8);
  FR_CUDA(cudaMemcpyAsync(chs_dev.data_ptr(), chs.data(), sizeof(PipeChannelDev) * W,
                          cudaMemcpyHostToDevice, stream));
  PipeArgs a;
  std::memset(&a, 0, sizeof(a));
  for (int r = 0; r < W; ++r) {
    a.in[r] = inputs[r].data_ptr();
    a.out[r] = inputs[r].data_ptr();
  }
  a.nbytes = inputs[0].numel() * inputs[0].element_size();
  a.chunk_bytes = chunk_bytes;
  a.scale = (float)scale;
  a.op = (int32_t)rop;
  a.dtype = (int32_t)dt;
  a.nvls = 0;
  a.stage_bytes = (int32_t)stage_bytes;
  a.stages = (int32_t)stages;
  cudaEvent_t t0, t1;
  FR_CUDA(cudaEventCreate(&t0));
  FR_CUDA(cudaEventCreate(&t1));
  FR_CUDA(cudaEventRecord(t0, stream));
  for (int64_t rep = 0; rep < repeats; ++rep) {
    cudaError_t e = launchPipeEmulated(static_cast<const PipeChannelDev*>(chs_dev.data_ptr()), a, W,
                                       (int)blocks, stream);
    TORCH_CHECK(e == cudaSuccess, "emulated launch of pipe_allreduce failed: ",
                cudaGetErrorString(e));
  }
  FR_CUDA(cudaEventRecord(t1, stream));
  FR_CUDA(cudaStreamSynchronize(stream));
  float ms = 0;
  cudaEventElapsedTime(&ms, t0, t1);
  g_last_emulated_us = (double)ms * 1e3 / (double)std::max<int64_t>(1, repeats);
  cudaEventDestroy(t0);
  cudaEventDestroy(t1);
  at::Tensor status = at::zeros({W, kStatusWords}, at::kInt);
  std::memcpy(status.data_ptr(), status_host, sizeof(uint32_t) * W * kStatusWords);
  cudaFreeHost(status_host);
  return std::make_tuple(inputs, status);
}

}  // namespace fairring
