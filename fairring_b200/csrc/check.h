// Error handling without torch: every failed check throws, nothing calls
// std::terminate (the reference's MY_CHECK does, fairring/utils.h:29-33, which
// takes the whole training job down for a bad argument).
#pragma once

#include <cuda_runtime.h>

#include <sstream>
#include <stdexcept>
#include <string>

namespace fairring {

class Error : public std::runtime_error {
 public:
  using std::runtime_error::runtime_error;
};

namespace detail {
inline void streamAll(std::ostringstream&) {}
template <typename T, typename... R>
void streamAll(std::ostringstream& os, const T& t, const R&... r) {
  os << t;
  streamAll(os, r...);
}
template <typename... A>
[[noreturn]] void fail(const char* file, int line, const char* what, const A&... a) {
  std::ostringstream os;
  os << "fairring: " << what << " at " << file << ":" << line;
  if (sizeof...(a) > 0) {
    os << ": ";
    streamAll(os, a...);
  }
  throw Error(os.str());
}
}  // namespace detail

#define FR_CHECK(cond, ...)                                                        \
  do {                                                                             \
    if (!(cond)) ::fairring::detail::fail(__FILE__, __LINE__, "check failed: " #cond, ##__VA_ARGS__); \
  } while (0)

#define FR_CUDA(expr)                                                              \
  do {                                                                             \
    cudaError_t fr_err_ = (expr);                                                  \
    if (fr_err_ != cudaSuccess)                                                    \
      ::fairring::detail::fail(__FILE__, __LINE__, "CUDA call failed: " #expr,     \
                               cudaGetErrorString(fr_err_));                       \
  } while (0)

}  // namespace fairring
