// Shared helpers of the evo::cuda source-compatibility layer.
//
// The layer defines what upstream evo.cpp declares in include/evo/cuda/{runtime,ops,hyena,attention}.hpp
// (classes and operator functions, on this library's C operator entry points, include/evo_b200_ops.h) and
// in include/evo/cuda/model.hpp (the model classes, on the model-level C ABI, include/evo/evo.h and
// include/evo/evo_b200.h).  It is compiled against upstream's own headers, found through an include path
// given at build time, so that code written against `evo::cuda` (upstream's test programs
// tests/test_cuda_{ops,hyena,attention,model,pipeline}.cu among it) links against this build unchanged.
// Nothing here computes on the device: every kernel that runs belongs to libevo_b200_ops or libevo; the
// layer checks sizes, keeps host-side bookkeeping (cache lengths, plan counters, page tables), issues
// copies and writes dump files.
#pragma once

#include <cstddef>
#include <cstdint>
#include <limits>
#include <string>

#include <cuda_runtime_api.h>

#include "evo/cuda/runtime.hpp"
#include "evo/status.hpp"

#include "../../include/evo_b200_ops.h"

namespace evo_b200_compat {

constexpr std::size_t kBf16Bytes = 2;

inline evo::Status invalid(const char *what) { return {evo::ErrorCode::kInvalidArgument, what}; }

// Status of a C entry point (0 ok, otherwise upstream's numeric error codes) as an evo::Status.
inline evo::Status from_code(const int code, const char *operation) {
  if (code == 0) return evo::Status::Ok();
  const char *detail = evo_b200_last_error();
  std::string message = operation;
  if (detail != nullptr && detail[0] != '\0') {
    message += ": ";
    message += detail;
  }
  evo::ErrorCode mapped = evo::ErrorCode::kInternal;
  switch (code) {
    case 2: mapped = evo::ErrorCode::kInvalidArgument; break;
    case 5: mapped = evo::ErrorCode::kUnsupported; break;
    case 6: mapped = evo::ErrorCode::kCuda; break;
    default: break;
  }
  return {mapped, message};
}

// a * b * c in size_t, or false on overflow.
inline bool product(const std::size_t a, const std::size_t b, const std::size_t c, std::size_t *out) {
  constexpr std::size_t top = std::numeric_limits<std::size_t>::max();
  if (a != 0 && b > top / a) return false;
  const std::size_t ab = a * b;
  if (ab != 0 && c > top / ab) return false;
  *out = ab * c;
  return true;
}

// True when `buffer` is allocated and holds at least `bytes`.
inline bool holds(const evo::cuda::DeviceBuffer &buffer, const std::size_t bytes) {
  return buffer.valid() && buffer.bytes() >= bytes;
}
inline bool holds(const evo::cuda::DeviceBuffer *buffer, const std::size_t bytes) {
  return buffer != nullptr && holds(*buffer, bytes);
}

// Makes `device` current for the scope and restores the previous one.
class DeviceScope final {
 public:
  explicit DeviceScope(const int device) {
    if (cudaGetDevice(&previous_) != cudaSuccess) previous_ = -1;
    if (device >= 0 && device != previous_) {
      changed_ = cudaSetDevice(device) == cudaSuccess;
    }
  }
  ~DeviceScope() {
    if (changed_ && previous_ >= 0) (void)cudaSetDevice(previous_);
  }
  DeviceScope(const DeviceScope &) = delete;
  DeviceScope &operator=(const DeviceScope &) = delete;

 private:
  int previous_{-1};
  bool changed_{false};
};

// Scratch that lives until the work queued on `stream` so far has drained: allocated and freed in
// stream order, so no call of the layer synchronises the device for it.
class StreamScratch final {
 public:
  StreamScratch() = default;
  ~StreamScratch() { release(); }
  StreamScratch(const StreamScratch &) = delete;
  StreamScratch &operator=(const StreamScratch &) = delete;

  evo::Status allocate(const std::size_t bytes, cudaStream_t stream) {
    release();
    stream_ = stream;
    const cudaError_t error = cudaMallocAsync(&data_, bytes == 0 ? 1 : bytes, stream);
    if (error != cudaSuccess) {
      data_ = nullptr;
      return {evo::ErrorCode::kCuda, std::string("cudaMallocAsync: ") + cudaGetErrorString(error)};
    }
    return evo::Status::Ok();
  }
  void release() noexcept {
    if (data_ != nullptr) (void)cudaFreeAsync(data_, stream_);
    data_ = nullptr;
  }
  void *data() const noexcept { return data_; }

 private:
  void *data_{nullptr};
  cudaStream_t stream_{nullptr};
};

}  // namespace evo_b200_compat
