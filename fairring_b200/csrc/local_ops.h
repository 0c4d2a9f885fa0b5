// torch-facing wrappers of the single-GPU fused kernels.
#pragma once

#include <pybind11/pybind11.h>

#include <cstdint>

namespace fairring {
void bindLocalOps(pybind11::module_& m);
uint64_t localLaunchCount();
}  // namespace fairring
