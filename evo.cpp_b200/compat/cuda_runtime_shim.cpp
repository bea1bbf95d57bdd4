// evo::cuda runtime objects (upstream include/evo/cuda/runtime.hpp:14-117: status helpers, Stream,
// DeviceBuffer, Blas, BlasLt) for code that is compiled against upstream's headers and linked against
// this library.  Blas and BlasLt carry no cuBLAS state here: the operators of this build run their own
// GEMM kernels, so `create()` only records the device and hands out a non-null token that keeps
// `valid()` and upstream's argument checks meaningful.
#include "compat_common.hpp"

#include <memory>
#include <utility>

namespace evo::cuda {

using evo_b200_compat::DeviceScope;

Status cuda_status(const cudaError_t error, const char *const operation) {
  if (error == cudaSuccess) return Status::Ok();
  std::string message = operation == nullptr ? "CUDA call" : operation;
  message += " failed: ";
  message += cudaGetErrorString(error);
  return {ErrorCode::kCuda, message};
}

Status cublas_status(const cublasStatus_t error, const char *const operation) {
  if (error == CUBLAS_STATUS_SUCCESS) return Status::Ok();
  std::string message = operation == nullptr ? "cuBLAS call" : operation;
  message += " failed with cuBLAS status ";
  message += std::to_string(static_cast<int>(error));
  return {ErrorCode::kCuda, message};
}

Status select_device(const int device) {
  int count = 0;
  auto status = cuda_status(cudaGetDeviceCount(&count), "cudaGetDeviceCount");
  if (!status.ok()) return status;
  if (device < 0 || device >= count)
    return {ErrorCode::kInvalidArgument, "CUDA device index " + std::to_string(device) + " is out of range"};
  return cuda_status(cudaSetDevice(device), "cudaSetDevice");
}

Status synchronize_device() { return cuda_status(cudaDeviceSynchronize(), "cudaDeviceSynchronize"); }

Status enable_peer_access(const int device, const int peer_device) {
  if (device == peer_device) return Status::Ok();
  int possible = 0;
  auto status = cuda_status(cudaDeviceCanAccessPeer(&possible, device, peer_device), "cudaDeviceCanAccessPeer");
  if (!status.ok()) return status;
  if (possible == 0) return {ErrorCode::kUnsupported, "the two CUDA devices cannot access each other's memory"};
  const DeviceScope scope(device);
  const cudaError_t error = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (error == cudaErrorPeerAccessAlreadyEnabled) {
    (void)cudaGetLastError();
    return Status::Ok();
  }
  return cuda_status(error, "cudaDeviceEnablePeerAccess");
}

// ---- Stream -------------------------------------------------------------------------------------

Stream::~Stream() { reset(); }

// Moves are swaps: every member has an "empty" default, so a moved-into object starts empty, trades
// places with its source, and whatever it held before leaves with the temporary.
Stream::Stream(Stream &&other) noexcept {
  std::swap(stream_, other.stream_);
  std::swap(device_, other.device_);
}

Stream &Stream::operator=(Stream &&other) noexcept {
  Stream incoming(std::move(other));
  std::swap(stream_, incoming.stream_);
  std::swap(device_, incoming.device_);
  return *this;  // `incoming` now owns the old stream and destroys it
}

Status Stream::create(const unsigned int flags) {
  reset();
  int device = -1;
  auto status = cuda_status(cudaGetDevice(&device), "cudaGetDevice");
  if (!status.ok()) return status;
  cudaStream_t made = nullptr;
  status = cuda_status(cudaStreamCreateWithFlags(&made, flags), "cudaStreamCreateWithFlags");
  if (!status.ok()) return status;
  stream_ = made;
  device_ = device;
  return Status::Ok();
}

void Stream::reset() noexcept {
  if (stream_ != nullptr) {
    const DeviceScope scope(device_);
    (void)cudaStreamDestroy(stream_);
  }
  stream_ = nullptr;
  device_ = -1;
}

Status Stream::synchronize() const {
  if (stream_ == nullptr) return {ErrorCode::kInvalidArgument, "the stream has not been created"};
  return cuda_status(cudaStreamSynchronize(stream_), "cudaStreamSynchronize");
}

// ---- DeviceBuffer -------------------------------------------------------------------------------

namespace {

// Frees on the device the block was allocated on, whichever device is current by then.
struct DeviceBlock final {
  void *pointer{nullptr};
  int device{-1};
  ~DeviceBlock() {
    if (pointer == nullptr) return;
    const DeviceScope scope(device);
    (void)cudaFree(pointer);
  }
};

Status check_transfer(const bool allocated, const void *host, const std::size_t wanted, const std::size_t capacity,
                      const Stream &stream, const int device, const char *what) {
  if (!allocated) return {ErrorCode::kInvalidArgument, std::string(what) + ": the device buffer is not allocated"};
  if (wanted > capacity) return {ErrorCode::kInvalidArgument, std::string(what) + ": more bytes than the buffer holds"};
  if (wanted != 0 && host == nullptr) return {ErrorCode::kInvalidArgument, std::string(what) + ": null host pointer"};
  if (!stream.valid() || stream.device() != device)
    return {ErrorCode::kInvalidArgument, std::string(what) + ": the stream does not belong to the buffer's device"};
  return Status::Ok();
}

}  // namespace

DeviceBuffer::~DeviceBuffer() { reset(); }

DeviceBuffer::DeviceBuffer(DeviceBuffer &&other) noexcept {
  allocation_.swap(other.allocation_);
  std::swap(data_, other.data_);
  std::swap(bytes_, other.bytes_);
  std::swap(device_, other.device_);
}

DeviceBuffer &DeviceBuffer::operator=(DeviceBuffer &&other) noexcept {
  DeviceBuffer incoming(std::move(other));
  allocation_.swap(incoming.allocation_);
  std::swap(data_, incoming.data_);
  std::swap(bytes_, incoming.bytes_);
  std::swap(device_, incoming.device_);
  return *this;
}

Status DeviceBuffer::allocate(const int device, const std::size_t bytes) {
  if (bytes == 0) return {ErrorCode::kInvalidArgument, "a device buffer of zero bytes was requested"};
  int count = 0;
  auto status = cuda_status(cudaGetDeviceCount(&count), "cudaGetDeviceCount");
  if (!status.ok()) return status;
  if (device < 0 || device >= count) return {ErrorCode::kInvalidArgument, "device buffer: no such CUDA device"};
  reset();
  const DeviceScope scope(device);
  auto block = std::make_shared<DeviceBlock>();
  status = cuda_status(cudaMalloc(&block->pointer, bytes), "cudaMalloc");
  if (!status.ok()) {
    block->pointer = nullptr;
    return status;
  }
  block->device = device;
  data_ = block->pointer;
  bytes_ = bytes;
  device_ = device;
  allocation_ = std::shared_ptr<void>(block, block->pointer);
  return Status::Ok();
}

Status DeviceBuffer::share_from(const DeviceBuffer &source) {
  if (!source.valid()) return {ErrorCode::kInvalidArgument, "cannot share an unallocated device buffer"};
  if (this == &source) return Status::Ok();
  reset();
  allocation_ = source.allocation_;
  data_ = source.data_;
  bytes_ = source.bytes_;
  device_ = source.device_;
  return Status::Ok();
}

void DeviceBuffer::reset() noexcept {
  allocation_.reset();
  data_ = nullptr;
  bytes_ = 0;
  device_ = -1;
}

Status DeviceBuffer::copy_from_host(const void *const source, const std::size_t bytes, const Stream &stream) {
  auto status = check_transfer(valid(), source, bytes, bytes_, stream, device_, "copy_from_host");
  if (!status.ok() || bytes == 0) return status;
  return cuda_status(cudaMemcpyAsync(data_, source, bytes, cudaMemcpyHostToDevice, stream.get()),
                     "cudaMemcpyAsync (host to device)");
}

Status DeviceBuffer::copy_to_host(void *const destination, const std::size_t bytes, const Stream &stream) const {
  auto status = check_transfer(valid(), destination, bytes, bytes_, stream, device_, "copy_to_host");
  if (!status.ok() || bytes == 0) return status;
  return cuda_status(cudaMemcpyAsync(destination, data_, bytes, cudaMemcpyDeviceToHost, stream.get()),
                     "cudaMemcpyAsync (device to host)");
}

Status DeviceBuffer::copy_from_peer(const DeviceBuffer &source, const std::size_t bytes, const Stream &stream) {
  if (!valid() || !source.valid() || source.device_ == device_)
    return {ErrorCode::kInvalidArgument, "copy_from_peer needs two allocated buffers on different devices"};
  if (bytes > bytes_ || bytes > source.bytes_)
    return {ErrorCode::kInvalidArgument, "copy_from_peer: more bytes than one of the buffers holds"};
  if (!stream.valid()) return {ErrorCode::kInvalidArgument, "copy_from_peer: the stream has not been created"};
  if (bytes == 0) return Status::Ok();
  return cuda_status(cudaMemcpyPeerAsync(data_, device_, source.data_, source.device_, bytes, stream.get()),
                     "cudaMemcpyPeerAsync");
}

Status DeviceBuffer::zero(const Stream &stream) {
  if (!valid()) return {ErrorCode::kInvalidArgument, "zero: the device buffer is not allocated"};
  if (!stream.valid() || stream.device() != device_)
    return {ErrorCode::kInvalidArgument, "zero: the stream does not belong to the buffer's device"};
  return cuda_status(cudaMemsetAsync(data_, 0, bytes_, stream.get()), "cudaMemsetAsync");
}

// ---- Blas / BlasLt ------------------------------------------------------------------------------
// Tokens only (see the file comment).  The token is the object's own address at creation, never
// dereferenced, and nothing is destroyed on reset.

Blas::~Blas() { reset(); }

Blas::Blas(Blas &&other) noexcept {
  std::swap(handle_, other.handle_);
  std::swap(device_, other.device_);
}

Blas &Blas::operator=(Blas &&other) noexcept {
  Blas incoming(std::move(other));
  std::swap(handle_, incoming.handle_);
  std::swap(device_, incoming.device_);
  return *this;
}

Status Blas::create() {
  int device = -1;
  auto status = cuda_status(cudaGetDevice(&device), "cudaGetDevice");
  if (!status.ok()) return status;
  handle_ = reinterpret_cast<cublasHandle_t>(this);
  device_ = device;
  return Status::Ok();
}

void Blas::reset() noexcept {
  handle_ = nullptr;
  device_ = -1;
}

BlasLt::~BlasLt() { reset(); }

BlasLt::BlasLt(BlasLt &&other) noexcept { std::swap(handle_, other.handle_); }

BlasLt &BlasLt::operator=(BlasLt &&other) noexcept {
  BlasLt incoming(std::move(other));
  std::swap(handle_, incoming.handle_);
  return *this;
}

Status BlasLt::create() {
  int device = -1;
  auto status = cuda_status(cudaGetDevice(&device), "cudaGetDevice");
  if (!status.ok()) return status;
  handle_ = reinterpret_cast<cublasLtHandle_t>(this);
  return Status::Ok();
}

void BlasLt::reset() noexcept { handle_ = nullptr; }

}  // namespace evo::cuda
