// FIFO of closures drained by one thread (fairring/utils.h:329-351 in the
// reference).  The engine uses it when FAIRRING_COMMAND_THREAD=1.  Header-only
// and free of CUDA so that it can be built under a thread sanitizer.
#pragma once

#include <condition_variable>
#include <deque>
#include <functional>
#include <mutex>

namespace fairring {

class CommandQueue {
 public:
  void push(std::function<void()> fn) {
    {
      std::lock_guard<std::mutex> lk(mu_);
      q_.push_back(std::move(fn));
    }
    cv_.notify_one();
  }
  // Blocks; an empty function means "stop".
  std::function<void()> pop() {
    std::unique_lock<std::mutex> lk(mu_);
    cv_.wait(lk, [&] { return !q_.empty(); });
    auto fn = std::move(q_.front());
    q_.pop_front();
    return fn;
  }

 private:
  std::mutex mu_;
  std::condition_variable cv_;
  std::deque<std::function<void()>> q_;
};

}  // namespace fairring
