// In-process self-test of the host path: `world` threads play the ranks, an
// in-memory key/value store stands in for the c10d store, and every thread
// runs the same collectives through its own CpuEngine on POSIX shared memory.
// Gives fast, exhaustive coverage of groupings, rank numberings, slicing and
// the double-buffered staging without spawning processes.
//
// Built twice: into the Python module (bindSelfTest), and, with
// -DFR_SELFTEST_STANDALONE, as a plain program that runs the same bodies under
// a thread sanitizer (tests/test_sanitizer.py): the command queue and the
// shared-memory signalling are the host code whose races a test on results
// alone would not see.
#ifndef FR_SELFTEST_STANDALONE
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#endif

#include <cmath>
#include <cstdio>
#include <condition_variable>
#include <map>
#include <mutex>
#include <thread>

#include "command_queue.h"
#include "cpu_path.h"
#include "kvstore.h"

namespace fairring {

namespace {

class MemoryStore : public KvStore {
 public:
  void set(const std::string& key, const std::vector<uint8_t>& value) override {
    {
      std::lock_guard<std::mutex> lk(mu_);
      data_[key] = value;
    }
    cv_.notify_all();
  }
  std::vector<uint8_t> get(const std::string& key) override {
    std::unique_lock<std::mutex> lk(mu_);
    const bool ok = cv_.wait_for(lk, std::chrono::seconds(30), [&] { return data_.count(key) > 0; });
    FR_CHECK(ok, "store key '", key, "' never appeared");
    return data_[key];
  }
  int64_t add(const std::string& key, int64_t delta) override {
    std::lock_guard<std::mutex> lk(mu_);
    return counters_[key] += delta;
  }

 private:
  std::mutex mu_;
  std::condition_variable cv_;
  std::map<std::string, std::vector<uint8_t>> data_;
  std::map<std::string, int64_t> counters_;
};

// Deterministic small integers (exactly representable in every dtype used).
inline double valueOf(int rank, int64_t i, int salt) {
  return (double)(((rank * 131 + i * 7 + salt * 13) % 17) - 8);
}

}  // namespace

// Returns the number of mismatching elements over all ranks and collectives
// (0 = pass).  `numels`: sizes to all-reduce in order; reduce_scatter and
// all_gather run once with per_rank = numels[0].
int64_t cpuSelfTest(int world, int gpus_per_machine, bool favorable, std::vector<int64_t> numels,
                    int64_t total_memory, int64_t slice_bytes, int64_t oneshot_max, bool use_max) {
  FR_CHECK(world >= 1 && world <= kMaxRanks && gpus_per_machine >= 1 && world % gpus_per_machine == 0,
           "bad self-test shape");
  auto store = std::make_shared<MemoryStore>();
  std::vector<int64_t> bad(world, 0);
  std::vector<std::string> errors(world);
  std::vector<std::thread> threads;
  const RedOp op = use_max ? RedOp::MAX : RedOp::SUM;
  for (int r = 0; r < world; ++r) {
    threads.emplace_back([&, r] {
      try {
        const Topo topo = makeTopo(world, gpus_per_machine, favorable, r);
        const MemoryPlan plan = planMemory(total_memory, slice_bytes, 1, world, 256);
        CpuEngine eng(store, topo, plan, std::chrono::milliseconds(20000));
        eng.oneshotMaxBytes = oneshot_max;
        int salt = 0;
        for (int64_t n : numels) {
          ++salt;
          std::vector<float> x(n);
          for (int64_t i = 0; i < n; ++i) x[i] = (float)valueOf(r, i, salt);
          eng.allReduce(x.data(), x.data(), n, DType::F32, op, 1.0f);
          for (int64_t i = 0; i < n; ++i) {
            double e = use_max ? -1e30 : 0.0;
            for (int q = 0; q < world; ++q) {
              const double v = valueOf(q, i, salt);
              e = use_max ? std::max(e, v) : e + v;
            }
            if ((double)x[i] != e) ++bad[r];
          }
        }
        const int64_t per = numels.empty() ? 0 : numels[0];
        if (per > 0) {
          std::vector<int32_t> in((size_t)per * world), out(per);
          for (int64_t i = 0; i < per * world; ++i) in[i] = (int32_t)valueOf(r, i, 99);
          eng.reduceScatter(in.data(), out.data(), per, DType::I32, RedOp::SUM, 1.0f);
          for (int64_t i = 0; i < per; ++i) {
            int64_t e = 0;
            for (int q = 0; q < world; ++q) e += (int64_t)valueOf(q, (int64_t)r * per + i, 99);
            if (out[i] != (int32_t)e) ++bad[r];
          }
          std::vector<double> mine(per), all((size_t)per * world);
          for (int64_t i = 0; i < per; ++i) mine[i] = valueOf(r, i, 7);
          eng.allGather(mine.data(), all.data(), per, DType::F64);
          for (int q = 0; q < world; ++q)
            for (int64_t i = 0; i < per; ++i)
              if (all[(size_t)q * per + i] != valueOf(q, i, 7)) ++bad[r];
        }
      } catch (const std::exception& e) {
        errors[r] = e.what();
        bad[r] += 1000000;
      }
    });
  }
  for (auto& t : threads) t.join();
  int64_t total = 0;
  for (int r = 0; r < world; ++r) {
    FR_CHECK(errors[r].empty(), "rank ", r, ": ", errors[r]);
    total += bad[r];
  }
  return total;
}

// Several producer threads push numbered closures; one consumer drains the
// queue as the engine's command thread does.  Returns the number of violations
// of "every item runs exactly once, and items of one producer run in order".
int64_t commandQueueSelfTest(int producers, int items_per_producer) {
  CommandQueue q;
  std::vector<std::vector<int>> seen(producers);
  std::thread consumer([&] {
    for (;;) {
      auto fn = q.pop();
      if (!fn) break;
      fn();
    }
  });
  std::vector<std::thread> ps;
  for (int p = 0; p < producers; ++p)
    ps.emplace_back([&, p] {
      for (int i = 0; i < items_per_producer; ++i) q.push([&seen, p, i] { seen[p].push_back(i); });
    });
  for (auto& t : ps) t.join();
  q.push(std::function<void()>());
  consumer.join();
  int64_t bad = 0;
  for (int p = 0; p < producers; ++p) {
    if ((int)seen[p].size() != items_per_producer) ++bad;
    for (size_t i = 0; i < seen[p].size(); ++i)
      if (seen[p][i] != (int)i) ++bad;
  }
  return bad;
}

#ifndef FR_SELFTEST_STANDALONE
void bindSelfTest(pybind11::module_& m) {
  namespace py = pybind11;
  m.def("cpu_self_test", &cpuSelfTest, py::arg("world"), py::arg("gpus_per_machine"),
        py::arg("favorable"), py::arg("numels"), py::arg("total_memory") = 1 << 20,
        py::arg("slice_bytes") = 0, py::arg("oneshot_max") = 1024, py::arg("use_max") = false,
        py::call_guard<py::gil_scoped_release>());
  m.def("command_queue_self_test", &commandQueueSelfTest, py::arg("producers") = 4,
        py::arg("items_per_producer") = 10000, py::call_guard<py::gil_scoped_release>());
}

#endif

}  // namespace fairring

#ifdef FR_SELFTEST_STANDALONE
int main() {
  using namespace fairring;
  int64_t bad = commandQueueSelfTest(4, 20000);
  std::printf("command queue: %lld violations\n", (long long)bad);
  for (int gpm : {4, 2, 1}) {
    const int64_t b = cpuSelfTest(4, gpm, false, {1, 37, 1000, 70001}, 1 << 20, 64 << 10, 1024, false);
    std::printf("host all-reduce, 4 ranks in groups of %d: %lld mismatches\n", gpm, (long long)b);
    bad += b;
  }
  return bad == 0 ? 0 : 1;
}
#endif
