// c10d::Store seen through the torch-free KvStore interface, with a key prefix.
#pragma once

#include <torch/csrc/distributed/c10d/Store.hpp>

#include <string>
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
  std::vector<uint8_t> get(const std::string& key) override { return store_->get(prefix_ + key); }
  int64_t add(const std::string& key, int64_t delta) override {
    return store_->add(prefix_ + key, delta);
  }

 private:
  c10::intrusive_ptr<c10d::Store> store_;
  std::string prefix_;
};

}  // namespace fairring
