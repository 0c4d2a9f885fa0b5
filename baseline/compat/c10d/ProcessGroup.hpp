// Forwarding header for sources written against PyTorch 1.11's c10d layout.
//
// Those sources include <c10d/ProcessGroup.hpp> and friends and derive their
// process group from c10d::ProcessGroup with a nested Work class.  In current
// PyTorch the headers live under torch/csrc/distributed/c10d/, a custom
// backend derives from c10d::Backend, and Work is a top-level class.  This
// header maps the old spelling onto the new classes without touching the
// sources that include it: everything PyTorch-side is included first, then the
// token `ProcessGroup` is redirected to a thin subclass of c10d::Backend that
// carries the old nested names.
#pragma once

#include <torch/torch.h>
#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/NCCLUtils.hpp>
#include <torch/csrc/distributed/c10d/PrefixStore.hpp>
#include <torch/csrc/distributed/c10d/ProcessGroup.hpp>
#include <torch/csrc/distributed/c10d/ProcessGroupNCCL.hpp>
#include <torch/csrc/distributed/c10d/Store.hpp>
#include <torch/csrc/distributed/c10d/Types.hpp>
#include <torch/csrc/distributed/c10d/Work.hpp>
#include <pybind11/chrono.h>
#include <pybind11/pybind11.h>
#include <torch/csrc/utils/pybind.h>

namespace c10d {

// What the old c10d::ProcessGroup was to a backend author: the base class of
// the backend, with Work and Options nested inside it.
class LegacyProcessGroupBase : public Backend {
 public:
  using Work = ::c10d::Work;
  using Options = ::c10d::Backend::Options;
  LegacyProcessGroupBase(int rank, int size) : Backend(rank, size) {}
};

}  // namespace c10d

// The module initialiser of such a source names the old base class in its
// pybind11 class declaration.  pybind11 must know that base, so it is
// registered (as a subclass of torch's own Backend binding) right before the
// module body runs.
#undef PYBIND11_MODULE
#define PYBIND11_MODULE(name, variable, ...)                                             \
  static void legacy_compat_module_body_##name(::pybind11::module_&);                   \
  PYBIND11_MODULE_PYINIT(name, (pybind11::detail::get_num_interpreters_seen() += 1),    \
                         ##__VA_ARGS__)                                                  \
  PYBIND11_MODULE_EXEC(name, legacy_compat_m) {                                          \
    ::pybind11::module_::import("torch.distributed");                                    \
    ::pybind11::class_<::c10d::LegacyProcessGroupBase,                                   \
                       c10::intrusive_ptr<::c10d::LegacyProcessGroupBase>,               \
                       ::c10d::Backend>(legacy_compat_m, "_LegacyProcessGroupBase");     \
    legacy_compat_module_body_##name(legacy_compat_m);                                   \
  }                                                                                      \
  void legacy_compat_module_body_##name(::pybind11::module_& variable)

#define ProcessGroup LegacyProcessGroupBase
