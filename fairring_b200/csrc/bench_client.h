#pragma once

#include <ATen/ATen.h>
#include <torch/csrc/distributed/c10d/Backend.hpp>

#include <vector>

namespace fairring {

class BenchClient {
 public:
  BenchClient(c10::intrusive_ptr<c10d::Backend> backend, int64_t num_buckets, int64_t bucket_elems,
              at::ScalarType dtype, int64_t num_epochs, int64_t warmup_epochs, bool gaussian,
              bool check, int64_t device);
  // Microseconds per timed epoch, measured on the device.
  std::vector<double> run();

 private:
  at::Tensor fill(int64_t epoch, int rank_as) const;
  c10::intrusive_ptr<c10d::Backend> backend_;
  int64_t num_buckets_, bucket_elems_;
  at::ScalarType dtype_;
  int64_t num_epochs_, warmup_epochs_;
  bool gaussian_, check_;
  int64_t device_;
};

}  // namespace fairring
