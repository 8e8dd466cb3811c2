// Error handling for the host side of the library.
//
// Three checked-call macros (CUDA runtime, CUDA driver, POSIX) that throw
// b200ipc::Error carrying file:line and the decoded error string, and a scope
// guard for releasing sockets, file descriptors, mappings and device memory on
// every exit path.
//
// Capability parity: the reference throws on every failing Level Zero call and
// every failing system call (ze_exception.hpp:9-51, ipc_exchange.cpp:35-40) and
// frees resources with a scope guard (utils.hpp:5-13).
#pragma once

#include <cerrno>
#include <cstring>
#include <sstream>
#include <stdexcept>
#include <string>
#include <utility>

#include <cuda.h>
#include <cuda_runtime_api.h>

namespace b200ipc {

class Error : public std::runtime_error {
 public:
  explicit Error(const std::string& what) : std::runtime_error(what) {}
};

inline std::string where(const char* file, int line) {
  std::ostringstream os;
  os << file << ":" << line;
  return os.str();
}

[[noreturn]] inline void fail(const std::string& kind, const std::string& expr,
                              const std::string& detail, const char* file, int line) {
  std::ostringstream os;
  os << "[b200ipc] " << kind << " failed at " << where(file, line) << ": " << expr << " -> " << detail;
  throw Error(os.str());
}

// Defined in cu_driver.cpp (resolves the driver lazily).
std::string cu_error_string(CUresult r);

template <typename F>
class ScopeGuard {
 public:
  explicit ScopeGuard(F f) : f_(std::move(f)) {}
  ScopeGuard(const ScopeGuard&) = delete;
  ScopeGuard& operator=(const ScopeGuard&) = delete;
  ScopeGuard(ScopeGuard&& o) noexcept : f_(std::move(o.f_)), armed_(o.armed_) { o.armed_ = false; }
  ~ScopeGuard() {
    if (armed_) {
      try { f_(); } catch (...) {}
    }
  }
  void dismiss() { armed_ = false; }
  void run_now() {
    if (armed_) { armed_ = false; f_(); }
  }

 private:
  F f_;
  bool armed_ = true;
};

template <typename F>
ScopeGuard<F> make_guard(F f) { return ScopeGuard<F>(std::move(f)); }

}  // namespace b200ipc

#define B200_CUDA_CHECK(expr)                                                              \
  do {                                                                                     \
    cudaError_t _e = (expr);                                                               \
    if (_e != cudaSuccess) {                                                               \
      ::b200ipc::fail("CUDA runtime call", #expr,                                          \
                      std::string(cudaGetErrorName(_e)) + ": " + cudaGetErrorString(_e),   \
                      __FILE__, __LINE__);                                                 \
    }                                                                                      \
  } while (0)

#define B200_CU_CHECK(expr)                                                                \
  do {                                                                                     \
    CUresult _r = (expr);                                                                  \
    if (_r != CUDA_SUCCESS) {                                                              \
      ::b200ipc::fail("CUDA driver call", #expr, ::b200ipc::cu_error_string(_r), __FILE__, \
                      __LINE__);                                                           \
    }                                                                                      \
  } while (0)

// For POSIX calls that return -1 and set errno.
#define B200_SYS_CHECK(expr)                                                               \
  do {                                                                                     \
    if ((expr) == -1) {                                                                    \
      ::b200ipc::fail("system call", #expr, std::strerror(errno), __FILE__, __LINE__);     \
    }                                                                                      \
  } while (0)

#define B200_REQUIRE(cond, msg)                                                            \
  do {                                                                                     \
    if (!(cond)) {                                                                         \
      std::ostringstream _os;                                                              \
      _os << msg;                                                                          \
      ::b200ipc::fail("requirement", #cond, _os.str(), __FILE__, __LINE__);                \
    }                                                                                      \
  } while (0)
