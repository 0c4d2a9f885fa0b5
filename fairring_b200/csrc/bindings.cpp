// Python module `fairring_b200._C`.  Counterpart of fairring/bindings.cc in the
// reference (ProcessGroup + Options with intrusive_ptr holders, constructor
// with the GIL released), plus what the tests and tools need: the planner and
// index math, topology detection, the one-GPU multi-rank emulator, the native
// benchmark client and the fused local ops.
#include <pybind11/chrono.h>
#include <pybind11/functional.h>
#include <pybind11/stl.h>
#include <torch/csrc/distributed/c10d/Store.hpp>
#include <torch/csrc/utils/pybind.h>
#include <torch/extension.h>

#include "backend.h"
#include "bench_client.h"
#include "local_ops.h"
#include "store_adapter.h"

#include <execinfo.h>
#include <signal.h>
#include <unistd.h>

namespace py = pybind11;
using namespace fairring;

namespace {
// FAIRRING_DEBUG_SEGV=1: print the native stack on SIGSEGV before dying.
void segvHandler(int sig) {
  void* frames[64];
  int n = backtrace(frames, 64);
  backtrace_symbols_fd(frames, n, STDERR_FILENO);
  signal(sig, SIG_DFL);
  raise(sig);
}
}  // namespace

namespace fairring {
void bindSelfTest(pybind11::module_& m);
std::tuple<std::vector<at::Tensor>, at::Tensor> emulatedCollective(
    const std::string& kind, std::vector<at::Tensor> inputs, int64_t gpus_per_machine,
    bool favorable, const std::string& op, double scale, c10::optional<at::ScalarType> wire_dtype,
    const std::string& algo, int64_t blocks, int64_t half_bytes, int64_t timeout_ms,
    int64_t silent_rank, int64_t repeats);
std::tuple<std::vector<at::Tensor>, at::Tensor> emulatedPipeAllreduce(
    std::vector<at::Tensor> inputs, const std::string& op, double scale, int64_t blocks,
    int64_t chunk_bytes, int64_t slot_bytes, int64_t slots, int64_t stage_bytes, int64_t stages,
    int64_t timeout_ms, int64_t silent_rank, int64_t repeats);
double lastEmulatedUs();
}

template <typename T>
using intrusive_class = py::class_<T, c10::intrusive_ptr<T>>;

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "fairring_b200 native module (sm_100a kernels, engine, c10d backend)";
  if (const char* dbg = std::getenv("FAIRRING_DEBUG_SEGV"))
    if (dbg[0] == '1') signal(SIGSEGV, segvHandler);

  intrusive_class<OptionsFairring>(m, "Options")
      .def(py::init([](std::chrono::milliseconds timeout) {
             return c10::make_intrusive<OptionsFairring>(timeout);
           }),
           py::arg("timeout") = kBackendDefaultTimeout)
      .def_readwrite("max_memory_allocated_in_bytes", &OptionsFairring::max_memory_allocated_in_bytes)
      .def_readwrite("max_padding_allocated_in_bytes", &OptionsFairring::max_padding_allocated_in_bytes)
      .def_readwrite("min_parallelism", &OptionsFairring::min_parallelism)
      .def_readwrite("is_high_priority_stream", &OptionsFairring::is_high_priority_stream)
      .def_readwrite("slice_size_in_bytes", &OptionsFairring::slice_size_in_bytes)
      .def_readwrite("gpus_per_machine", &OptionsFairring::gpus_per_machine)
      .def_readwrite("favorable_layout", &OptionsFairring::favorable_layout)
      .def_readwrite("algo", &OptionsFairring::algo)
      .def_readwrite("blocks", &OptionsFairring::blocks)
      .def_readwrite("sm_budget", &OptionsFairring::sm_budget)
      .def_readwrite("oneshot_max_bytes", &OptionsFairring::oneshot_max_bytes)
      .def_readwrite("ll_max_bytes", &OptionsFairring::ll_max_bytes)
      .def_readwrite("ll2_max_bytes", &OptionsFairring::ll2_max_bytes)
      .def_readwrite("ll_channels", &OptionsFairring::ll_channels)
      .def_readwrite("inline_small", &OptionsFairring::inline_small)
      .def_readwrite("direct_blocks", &OptionsFairring::direct_blocks)
      .def_readwrite("direct_unroll", &OptionsFairring::direct_unroll)
      .def_readwrite("nvls_min_bytes", &OptionsFairring::nvls_min_bytes)
      .def_readwrite("nvls_oneshot_max_bytes", &OptionsFairring::nvls_oneshot_max_bytes)
      .def_readwrite("device_timeout_ms", &OptionsFairring::device_timeout_ms)
      .def_readwrite("nvls", &OptionsFairring::nvls)
      .def_readwrite("transport", &OptionsFairring::transport)
      .def_readwrite("direct", &OptionsFairring::direct)
      .def_readwrite("pipe", &OptionsFairring::pipe)
      .def_readwrite("pipe_min_bytes", &OptionsFairring::pipe_min_bytes)
      .def_readwrite("pipe_blocks", &OptionsFairring::pipe_blocks)
      .def_readwrite("pipe_channels", &OptionsFairring::pipe_channels)
      .def_readwrite("pipe_slots", &OptionsFairring::pipe_slots)
      .def_readwrite("pipe_chunk_bytes", &OptionsFairring::pipe_chunk_bytes)
      .def_readwrite("pipe_stage_bytes", &OptionsFairring::pipe_stage_bytes)
      .def_readwrite("pipe_stages", &OptionsFairring::pipe_stages)
      .def_readwrite("direct_max_slices", &OptionsFairring::direct_max_slices)
      .def_readwrite("direct_min_slice_bytes", &OptionsFairring::direct_min_slice_bytes)
      .def_readwrite("command_thread", &OptionsFairring::command_thread)
      .def_readwrite("blocking_wait", &OptionsFairring::blocking_wait)
      .def_readwrite("boot_id_override", &OptionsFairring::boot_id_override)
      .def_readwrite("timeout", &OptionsFairring::timeout);

  py::class_<BackendFairring, c10d::Backend, c10::intrusive_ptr<BackendFairring>>(m, "Backend")
      .def(py::init([](const c10::intrusive_ptr<c10d::Store>& store, int rank, int size,
                       c10::intrusive_ptr<OptionsFairring> options) {
             return c10::make_intrusive<BackendFairring>(store, rank, size, std::move(options));
           }),
           py::arg("store"), py::arg("rank"), py::arg("size"), py::arg("options"),
           py::call_guard<py::gil_scoped_release>())
      .def(
          "set_delegate_factory",
          [](BackendFairring& self, py::function fn) {
            // The callable is invoked from C++ threads that do not hold the GIL
            // and must be released under it.
            auto holder = std::shared_ptr<py::function>(new py::function(std::move(fn)),
                                                        [](py::function* f) {
                                                          py::gil_scoped_acquire g;
                                                          delete f;
                                                        });
            self.setDelegateFactory([holder](const std::string& kind) {
              py::gil_scoped_acquire g;
              py::object o = (*holder)(kind);
              return o.cast<c10::intrusive_ptr<c10d::Backend>>();
            });
          })
      .def(
          "allreduce_fused",
          [](BackendFairring& self, at::Tensor t, double scale,
             c10::optional<at::ScalarType> wire_dtype, const std::string& op) {
            return self.allreduceFused(std::move(t), scale, wire_dtype, op);
          },
          py::arg("tensor"), py::arg("scale") = 1.0, py::arg("wire_dtype") = py::none(),
          py::arg("op") = "sum", py::call_guard<py::gil_scoped_release>())
      .def("describe", &BackendFairring::describe, py::call_guard<py::gil_scoped_release>())
      .def("stats", &BackendFairring::stats, py::call_guard<py::gil_scoped_release>())
      .def("deployment", &BackendFairring::deployment, py::call_guard<py::gil_scoped_release>())
      .def("trace", &BackendFairring::trace, py::call_guard<py::gil_scoped_release>())
      .def("check_health", &BackendFairring::checkHealth, py::call_guard<py::gil_scoped_release>())
      .def("health", &BackendFairring::health, py::call_guard<py::gil_scoped_release>())
      .def("set_option", &BackendFairring::setOption, py::arg("name"), py::arg("value"),
           py::call_guard<py::gil_scoped_release>())
      .def("release_symmetric", &BackendFairring::releaseSymmetric,
           py::call_guard<py::gil_scoped_release>())
      .def("reset", &BackendFairring::reset, py::call_guard<py::gil_scoped_release>())
      .def("abort", &BackendFairring::abort, py::call_guard<py::gil_scoped_release>())
      .def("shutdown", &BackendFairring::shutdown, py::call_guard<py::gil_scoped_release>())
      .def("symmetric_empty", &BackendFairring::symmetricEmpty, py::arg("numel"), py::arg("dtype"),
           py::call_guard<py::gil_scoped_release>())
      .def("skip_cpu_signals", &BackendFairring::skipCpuSignals,
           py::call_guard<py::gil_scoped_release>());

  py::class_<BenchClient>(m, "BenchClient")
      .def(py::init<c10::intrusive_ptr<c10d::Backend>, int64_t, int64_t, at::ScalarType, int64_t,
                    int64_t, bool, bool, int64_t>(),
           py::arg("backend"), py::arg("num_buckets"), py::arg("bucket_elems"), py::arg("dtype"),
           py::arg("num_epochs"), py::arg("warmup_epochs") = 1, py::arg("gaussian") = false,
           py::arg("check") = true, py::arg("device") = 0)
      .def("run", &BenchClient::run, py::call_guard<py::gil_scoped_release>());

  // ---- planner / index math, for oracle tests --------------------------------
  m.def("plan_memory", [](int64_t total, int64_t slice, int64_t par, int64_t world,
                          int64_t min_half) {
    MemoryPlan p = planMemory(total, slice, (int32_t)par, (int)world, min_half);
    return py::dict(py::arg("total_bytes") = p.total_bytes, py::arg("channels") = p.channels,
                    py::arg("slot_bytes") = p.slot_bytes, py::arg("half_bytes") = p.half_bytes,
                    py::arg("max_slice_bytes") = p.max_slice_bytes);
  }, py::arg("total_bytes"), py::arg("slice_bytes"), py::arg("parallelism"), py::arg("world"),
     py::arg("min_half_bytes") = 1 << 20);
  m.def("plan_slices", [](int64_t numel, int64_t esize, int64_t world, int64_t max_slice_bytes) {
    SlicePlan s = planSlices(numel, (int)esize, (int)world, max_slice_bytes);
    return std::make_pair(s.num_slices, s.slice_elems);
  });
  auto segDict = [](const Seg& s) {
    return py::dict(py::arg("chunk_len") = s.chunk_len, py::arg("chunk_stride") = s.chunk_stride,
                    py::arg("limit") = s.limit, py::arg("qv") = s.qv);
  };
  m.def("allreduce_seg", [segDict](int64_t n, int64_t esize, int64_t world) {
    return segDict(allreduceSeg(n, (int)esize, (int)world));
  });
  m.def("scatter_seg", [segDict](int64_t len, int64_t per_rank, int64_t esize) {
    return segDict(scatterSeg(len, per_rank, (int)esize));
  });
  m.def("rank_of", [](int64_t world, int64_t D, bool fav, int64_t mm, int64_t dd) {
    return rankOf(makeTopo((int)world, (int)D, fav, 0), (int)mm, (int)dd);
  });
  m.def("machine_device_of", [](int64_t world, int64_t D, bool fav, int64_t rank) {
    Topo t = makeTopo((int)world, (int)D, fav, (int)rank);
    return std::make_pair(t.m, t.d);
  });
  m.def("valid_in_vector", [](int64_t chunk_len, int64_t chunk_stride, int64_t limit, int64_t qv,
                              int64_t c, int64_t v, int64_t V) {
    Seg s{chunk_len, chunk_stride, limit, qv};
    return validInVector(s, (int)c, v, (int)V);
  });
  m.def("staging_vec", [](int64_t world, int64_t D, int64_t qv, int64_t slot, int64_t j) {
    Seg s{0, 0, 0, qv};
    return stagingVec(makeTopo((int)world, (int)D, false, 0), s, (int)slot, (int)j);
  });
  m.def(
      "detect_deployment",
      [](const c10::intrusive_ptr<c10d::Store>& store, int rank, int world, int gpus_per_machine,
         bool favorable, const std::string& boot_id) {
        Deployment d;
        {
          py::gil_scoped_release nogil;  // blocks on the store until all ranks have published
          StoreAdapter s(store, "fairring/");
          d = detectDeployment(s, rank, world, gpus_per_machine, favorable, boot_id);
        }
        return py::dict(py::arg("D") = d.topo.D, py::arg("M") = d.topo.M,
                        py::arg("favorable") = d.topo.favorable, py::arg("m") = d.topo.m,
                        py::arg("d") = d.topo.d, py::arg("num_hosts") = d.num_hosts,
                        py::arg("ranks_per_host") = d.ranks_per_host,
                        py::arg("single_host") = d.single_host);
      },
      py::arg("store"), py::arg("rank"), py::arg("world"), py::arg("gpus_per_machine") = 0,
      py::arg("favorable") = false, py::arg("boot_id") = "");

  m.def("emulated_collective", &emulatedCollective, py::arg("kind"), py::arg("inputs"),
        py::arg("gpus_per_machine"), py::arg("favorable") = false, py::arg("op") = "sum",
        py::arg("scale") = 1.0, py::arg("wire_dtype") = py::none(), py::arg("algo") = "twoshot",
        py::arg("blocks") = 4, py::arg("half_bytes") = 1 << 20, py::arg("timeout_ms") = 2000,
        py::arg("silent_rank") = -1, py::arg("repeats") = 1);

  m.def("emulated_pipe_allreduce", &emulatedPipeAllreduce, py::arg("inputs"), py::arg("op") = "sum",
        py::arg("scale") = 1.0, py::arg("blocks") = 4, py::arg("chunk_bytes") = 64 << 10,
        py::arg("slot_bytes") = 64 << 10, py::arg("slots") = 4, py::arg("stage_bytes") = 4096,
        py::arg("stages") = 4, py::arg("timeout_ms") = 2000, py::arg("silent_rank") = -1,
        py::arg("repeats") = 1);

  m.def("last_emulated_us", &lastEmulatedUs);
  m.def("launch_count", []() { return (int64_t)(launchCount() + localLaunchCount()); });
  m.def("collective_launch_count", []() { return (int64_t)launchCount(); });
  m.attr("MAX_RANKS") = kMaxRanks;
  m.attr("MAX_BLOCKS") = kMaxBlocks;
  m.attr("VEC_BYTES") = kVecBytes;

  bindLocalOps(m);
  bindSelfTest(m);
}
