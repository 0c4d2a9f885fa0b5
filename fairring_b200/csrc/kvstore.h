// Minimal key/value rendezvous interface.  The backend adapts a c10d::Store to
// it; tests use an in-process implementation.  Counterpart of the Store byte
// helpers in the reference (fairring/utils.h:178-219).
#pragma once

#include <chrono>
#include <cstdint>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "check.h"

namespace fairring {

class KvStore {
 public:
  virtual ~KvStore() = default;
  virtual void set(const std::string& key, const std::vector<uint8_t>& value) = 0;
  // Blocks until the key exists or the store's own timeout expires (throws).
  virtual std::vector<uint8_t> get(const std::string& key) = 0;
  virtual int64_t add(const std::string& key, int64_t delta) = 0;

  void setString(const std::string& key, const std::string& v) {
    set(key, std::vector<uint8_t>(v.begin(), v.end()));
  }
  std::string getString(const std::string& key) {
    auto v = get(key);
    return std::string(v.begin(), v.end());
  }
  template <typename T>
  void setPod(const std::string& key, const T& v) {
    std::vector<uint8_t> b(sizeof(T));
    std::memcpy(b.data(), &v, sizeof(T));
    set(key, b);
  }
  template <typename T>
  T getPod(const std::string& key) {
    auto b = get(key);
    FR_CHECK(b.size() == sizeof(T), "store value for ", key, " has ", b.size(), " bytes, expected ",
             sizeof(T));
    T v;
    std::memcpy(&v, b.data(), sizeof(T));
    return v;
  }

  // All `world` ranks call this with the same name; returns when all have.
  void barrier(const std::string& name, int world, std::chrono::milliseconds timeout) {
    add(name, 1);
    auto t0 = std::chrono::steady_clock::now();
    while (add(name, 0) < world) {
      FR_CHECK(std::chrono::steady_clock::now() - t0 < timeout, "store barrier '", name,
               "' timed out: a rank never arrived");
      std::this_thread::sleep_for(std::chrono::microseconds(200));
    }
  }
};

}  // namespace fairring
