// Error type shared by every native component, plus CUDA runtime / driver checks.
// Plays the role of the reference's FabricLibError enum (fabric-lib/src/error.rs:10-77)
// and of cuda_check!/cuda_unwrap! (rust/cuda-lib/src/error.rs:22-44).
#pragma once

#include <cuda_runtime.h>

#include <cerrno>
#include <cstring>
#include <stdexcept>
#include <string>

namespace pplx {

enum class ErrorKind {
  kCustom,
  kCudaRuntime,
  kCudaDriver,
  kErrno,
  kCompletion,   // a transfer completed with an error
  kDomain,       // a transport provider refused an operation
  kWorkerDown,   // a worker thread is no longer running
  kTimeout,
  kInvalidArgument,
};

class Error : public std::runtime_error {
 public:
  Error(ErrorKind kind, const std::string& what) : std::runtime_error(what), kind_(kind) {}
  ErrorKind kind() const { return kind_; }

  static Error from_errno(const std::string& ctx, int err = errno) {
    return Error(ErrorKind::kErrno, ctx + ": " + std::strerror(err) + " (errno " +
                                        std::to_string(err) + ")");
  }

 private:
  ErrorKind kind_;
};

inline void cuda_check(cudaError_t e, const char* expr, const char* file, int line) {
  if (e != cudaSuccess) {
    throw Error(ErrorKind::kCudaRuntime, std::string("CUDA runtime error ") +
                                             cudaGetErrorName(e) + " (" + cudaGetErrorString(e) +
                                             ") in `" + expr + "` at " + file + ":" +
                                             std::to_string(line));
  }
}

#define PPLX_CUDA_CHECK(expr) ::pplx::cuda_check((expr), #expr, __FILE__, __LINE__)

#define PPLX_REQUIRE(cond, msg)                                                              \
  do {                                                                                       \
    if (!(cond)) {                                                                           \
      throw ::pplx::Error(::pplx::ErrorKind::kInvalidArgument,                               \
                          std::string(msg) + " [" #cond "]");                                \
    }                                                                                        \
  } while (0)

}  // namespace pplx
