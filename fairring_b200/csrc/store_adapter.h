// c10d::Store seen through the torch-free KvStore interface, with a key prefix.
#pragma once

#include <torch/csrc/distributed/c10d/Store.hpp>

#include <chrono>
#include <string>
#include <thread>
#include <utility>
#include <vector>

#include "kvstore.h"

namespace fairring {

class StoreAdapter : public KvStore {
 public:
  StoreAdapter(c10::intrusive_ptr<c10d::Store> s, std::string prefix)
      : store_(std::move(s)), prefix_(std::move(prefix)) {}
  void set(const std::string& key, const std::vector<uint8_t>& value) override {
    store_->set(prefix_ + key, value);
  }
  // Polls until the key exists instead of blocking inside the store: a store
  // client serialises its operations, and with several GPUs per process two
  // ranks share one client -- a blocking get of rank A would lock out the very
  // set of rank B that it waits for.
  std::vector<uint8_t> get(const std::string& key) override {
    const std::string k = prefix_ + key;
    const auto limit = store_->getTimeout();
    const auto t0 = std::chrono::steady_clock::now();
    while (!store_->check({k})) {
      FR_CHECK(limit.count() <= 0 || std::chrono::steady_clock::now() - t0 < limit, "store key '", k,
               "' never appeared: a rank is missing");
      std::this_thread::sleep_for(std::chrono::microseconds(200));
    }
    return store_->get(k);
  }
  int64_t add(const std::string& key, int64_t delta) override {
    return store_->add(prefix_ + key, delta);
  }

 private:
  c10::intrusive_ptr<c10d::Store> store_;
  std::string prefix_;
};

}  // namespace fairring
