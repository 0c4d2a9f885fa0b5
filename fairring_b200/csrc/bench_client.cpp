// Native micro-benchmark client: N buckets of a given size are all-reduced per
// epoch through any c10d backend (this library or NCCL), with the buckets in
// flight together.  Counterpart of benchmark/benchmark.cc in the reference,
// with three differences: the epoch is timed on the device with CUDA events
// (the reference uses the host's steady_clock around enqueue + wait), inputs
// can be N(0,1) per rank instead of all-ones, and the check recomputes the
// exact expected sum from the per-rank seeds instead of comparing with W.
#include "bench_client.h"

#include <ATen/ATen.h>
#include <ATen/cuda/CUDAGeneratorImpl.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

namespace fairring {

BenchClient::BenchClient(c10::intrusive_ptr<c10d::Backend> backend, int64_t num_buckets,
                         int64_t bucket_elems, at::ScalarType dtype, int64_t num_epochs,
                         int64_t warmup_epochs, bool gaussian, bool check, int64_t device)
    : backend_(std::move(backend)), num_buckets_(num_buckets), bucket_elems_(bucket_elems),
      dtype_(dtype), num_epochs_(num_epochs), warmup_epochs_(warmup_epochs), gaussian_(gaussian),
      check_(check), device_(device) {
  TORCH_CHECK(num_buckets_ >= 1 && bucket_elems_ >= 1 && num_epochs_ >= 1, "bad benchmark shape");
}

at::Tensor BenchClient::fill(int64_t epoch, int rank_as) const {
  // What rank `rank_as` puts into its buckets in this epoch.
  auto opts = at::TensorOptions().device(at::kCUDA, (c10::DeviceIndex)device_).dtype(at::kFloat);
  if (!gaussian_) return at::ones({num_buckets_, bucket_elems_}, opts).to(dtype_);
  auto gen = at::cuda::detail::createCUDAGenerator((c10::DeviceIndex)device_);
  gen.set_current_seed((uint64_t)(1000003 * (epoch + 1) + rank_as));
  return at::randn({num_buckets_, bucket_elems_}, gen, opts).to(dtype_);
}

std::vector<double> BenchClient::run() {
  c10::cuda::CUDAGuard guard((c10::DeviceIndex)device_);
  const int W = backend_->getSize(), me = backend_->getRank();
  auto stream = c10::cuda::getCurrentCUDAStream();
  cudaEvent_t e0, e1;
  C10_CUDA_CHECK(cudaEventCreate(&e0));
  C10_CUDA_CHECK(cudaEventCreate(&e1));
  // Something larger than L2 to write between epochs, so that no epoch starts
  // with its buckets cached.
  at::Tensor flush = at::empty({256ll << 20}, at::TensorOptions().device(at::kCUDA, (c10::DeviceIndex)device_).dtype(at::kByte));
  std::vector<double> us;
  for (int64_t epoch = 0; epoch < warmup_epochs_ + num_epochs_; ++epoch) {
    at::Tensor buckets = fill(epoch, me);
    flush.fill_(1);
    std::vector<c10::intrusive_ptr<c10d::Work>> works;
    works.reserve(num_buckets_);
    C10_CUDA_CHECK(cudaStreamSynchronize(stream));
    C10_CUDA_CHECK(cudaEventRecord(e0, stream));
    for (int64_t b = 0; b < num_buckets_; ++b) {
      std::vector<at::Tensor> v{buckets[b]};
      works.push_back(backend_->allreduce(v, c10d::AllreduceOptions()));
    }
    for (auto& w : works) w->wait();
    C10_CUDA_CHECK(cudaEventRecord(e1, stream));
    C10_CUDA_CHECK(cudaEventSynchronize(e1));
    float ms = 0;
    C10_CUDA_CHECK(cudaEventElapsedTime(&ms, e0, e1));
    if (epoch >= warmup_epochs_) us.push_back((double)ms * 1000.0);
    if (check_) {
      at::Tensor expect;
      if (!gaussian_) {
        expect = at::full({num_buckets_, bucket_elems_}, (double)W, buckets.options().dtype(at::kFloat));
      } else {
        expect = at::zeros({num_buckets_, bucket_elems_}, buckets.options().dtype(at::kFloat));
        for (int r = 0; r < W; ++r) expect.add_(fill(epoch, r).to(at::kFloat));
      }
      const double rtol = dtype_ == at::kFloat ? 1e-5 : 2e-2;
      const double atol = dtype_ == at::kFloat ? 1e-5 : 2e-2 * std::sqrt((double)W);
      TORCH_CHECK(at::allclose(buckets.to(at::kFloat), expect, rtol, atol),
                  "fairring benchmark: bad all_reduce result in epoch ", epoch);
    }
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  return us;
}

}  // namespace fairring
