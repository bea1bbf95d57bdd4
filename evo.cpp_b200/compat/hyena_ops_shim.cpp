// evo::cuda Hyena operators (upstream include/evo/cuda/hyena.hpp:13-270) on this library's C entry
// points; see compat_common.hpp for what the layer is.
//
// Differences a caller can observe:
//  * There is no cuFFT path.  The medium and long convolutions of this build are direct (a Toeplitz
//    product on the tensor cores, a chunked modal scan), so bf16_fir_prefill_fft, bf16_hcm_prefill and
//    the FFT modes of bf16_hcl_prefill run the same kernels as their direct / recurrent forms and agree
//    with them bit for bit.  FftWorkspace keeps upstream's bookkeeping (dimensions, generation counter,
//    exact-match requirement) and owns no plans or device memory.
//  * Prefill runs as one fused pass (inner gate, filter, direct term, outer gate); the `scratch`
//    buffer still receives the BF16 inner gate x1 * v as upstream leaves it there.
//  * bf16_hcl_prefill keeps its per-segment states in a fixed 16 MiB array inside the library
//    (evo_b200_bf16_hcl_prefill_noalloc), so two HCL prefills must not overlap on one GPU.
#include "compat_common.hpp"

#include <algorithm>
#include <utility>

#include "evo/cuda/hyena.hpp"

namespace evo::cuda {

using evo_b200_compat::from_code;
using evo_b200_compat::holds;
using evo_b200_compat::invalid;
using evo_b200_compat::kBf16Bytes;
using evo_b200_compat::product;
using evo_b200_compat::StreamScratch;

namespace {

void *raw(const Stream &stream) { return static_cast<void *>(stream.get()); }

bool on_device(const Stream &stream, const DeviceBuffer &buffer) {
  return stream.valid() && buffer.valid() && buffer.device() == stream.device();
}

int orientation_code(const FirOrientation orientation) {
  return orientation == FirOrientation::kCrossCorrelation ? 0 : 1;
}
int bias_code(const FirBiasMode mode) { return mode == FirBiasMode::kAdd ? 0 : 1; }
int weight_code(const FirWeightType type) { return type == FirWeightType::kF32 ? 1 : 0; }
std::size_t weight_element_bytes(const FirWeightType type) {
  return type == FirWeightType::kF32 ? sizeof(float) : kBf16Bytes;
}

// Sizes every FIR-shaped call shares; `sequence_bytes` is one BF16 [length, channels] tensor.
struct FirShape final {
  std::size_t sequence_bytes{0};
  std::size_t weight_bytes{0};
};

Status fir_shape(const std::size_t length, const std::size_t channels, const std::size_t groups,
                 const std::size_t kernel_size, const FirWeightType type, FirShape *shape) {
  if (length == 0 || channels == 0 || groups == 0 || kernel_size == 0 || channels % groups != 0)
    return invalid("FIR: length, channels, groups and kernel size must be positive and groups must divide channels");
  if (!product(length, channels, kBf16Bytes, &shape->sequence_bytes) ||
      !product(groups, kernel_size, weight_element_bytes(type), &shape->weight_bytes))
    return invalid("FIR: dimensions are not representable");
  return Status::Ok();
}

Status check_fir_cache(const FirCache *cache, const std::size_t channels, const std::size_t kernel_size,
                       const Stream &stream) {
  if (cache == nullptr) return Status::Ok();
  std::size_t bytes = 0;
  if (cache->channels != channels || cache->kernel_size != kernel_size || cache->length + 1 > kernel_size ||
      !product(channels, kernel_size - 1, sizeof(float), &bytes) ||
      (bytes != 0 && (!holds(cache->state, bytes) || !on_device(stream, cache->state))))
    return invalid("FIR cache does not match the operator's channels and kernel size");
  return Status::Ok();
}

float *cache_pointer(FirCache *cache) {
  return cache == nullptr || !cache->state.valid() ? nullptr : static_cast<float *>(cache->state.data());
}

// History rows after `added` more inputs.
std::size_t grown(const std::size_t have, const std::size_t added, const std::size_t kernel_size) {
  const std::size_t capacity = kernel_size - 1;
  return added >= capacity - std::min(have, capacity) ? capacity : have + added;
}

}  // namespace

// ---- caches and the FFT workspace ---------------------------------------------------------------

Status FirCache::allocate(const int device, const std::size_t channel_count, const std::size_t filter_length,
                          const Stream &stream) {
  std::size_t bytes = 0;
  if (channel_count == 0 || filter_length == 0 || !product(channel_count, filter_length - 1, sizeof(float), &bytes))
    return invalid("FIR cache: channels and kernel size must be positive and representable");
  if (!stream.valid() || stream.device() != device) return invalid("FIR cache: the stream belongs to another device");
  state.reset();
  if (bytes != 0) {
    auto status = state.allocate(device, bytes);
    if (!status.ok()) return status;
    status = state.zero(stream);
    if (!status.ok()) return status;
  }
  channels = channel_count;
  kernel_size = filter_length;
  length = 0;
  return Status::Ok();
}

Status IirCache::allocate(const int device, const std::size_t channel_count, const std::size_t mode_count,
                          const Stream &stream) {
  std::size_t bytes = 0;
  if (channel_count == 0 || mode_count == 0 || !product(channel_count, mode_count, sizeof(float), &bytes))
    return invalid("modal cache: channels and modes must be positive and representable");
  if (!stream.valid() || stream.device() != device) return invalid("modal cache: the stream belongs to another device");
  auto status = state.allocate(device, bytes);
  if (!status.ok()) return status;
  status = state.zero(stream);
  if (!status.ok()) return status;
  channels = channel_count;
  state_size = mode_count;
  return Status::Ok();
}

FftWorkspace::~FftWorkspace() { reset(); }

FftWorkspace::FftWorkspace(FftWorkspace &&other) noexcept
    : device_(std::exchange(other.device_, -1)),
      channels_(std::exchange(other.channels_, 0)),
      filter_groups_(std::exchange(other.filter_groups_, 0)),
      fft_size_(std::exchange(other.fft_size_, 0)),
      state_size_(std::exchange(other.state_size_, 0)),
      input_mode_(std::exchange(other.input_mode_, FftInputMode::kRealCompact)),
      generation_(std::exchange(other.generation_, 0)) {}

FftWorkspace &FftWorkspace::operator=(FftWorkspace &&other) noexcept {
  if (this != &other) {
    reset();
    device_ = std::exchange(other.device_, -1);
    channels_ = std::exchange(other.channels_, 0);
    filter_groups_ = std::exchange(other.filter_groups_, 0);
    fft_size_ = std::exchange(other.fft_size_, 0);
    state_size_ = std::exchange(other.state_size_, 0);
    input_mode_ = std::exchange(other.input_mode_, FftInputMode::kRealCompact);
    generation_ = std::exchange(other.generation_, 0);
  }
  return *this;
}

Status FftWorkspace::allocate(const int device, const std::size_t channels, const std::size_t filter_groups,
                              const std::size_t fft_size, const FftInputMode input_mode) {
  if (device_ >= 0) return invalid("FFT workspace: reset it before giving it other dimensions");
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count)
    return invalid("FFT workspace: no such CUDA device");
  std::size_t ignored = 0;
  if (channels == 0 || filter_groups == 0 || fft_size < 2 || channels % filter_groups != 0 ||
      !product(channels, fft_size, 2 * sizeof(float), &ignored))
    return invalid("FFT workspace: channels, groups and transform size do not form a valid problem");
  device_ = device;
  channels_ = channels;
  filter_groups_ = filter_groups;
  fft_size_ = fft_size;
  input_mode_ = input_mode;
  state_size_ = 0;
  ++generation_;
  return Status::Ok();
}

void FftWorkspace::reset() noexcept {
  device_ = -1;
  channels_ = 0;
  filter_groups_ = 0;
  fft_size_ = 0;
  state_size_ = 0;
  input_mode_ = FftInputMode::kRealCompact;
}

bool FftWorkspace::matches(const int device, const std::size_t channels, const std::size_t filter_groups,
                           const std::size_t fft_size, const FftInputMode input_mode) const noexcept {
  return device_ >= 0 && device_ == device && channels_ == channels && filter_groups_ == filter_groups &&
         fft_size_ == fft_size && input_mode_ == input_mode;
}

std::size_t fir_fft_size(const std::size_t length, const std::size_t kernel_size) noexcept {
  constexpr std::size_t top = std::numeric_limits<std::size_t>::max();
  if (length == 0 || kernel_size == 0 || kernel_size - 1 > top - length) return 0;
  const std::size_t needed = length + (kernel_size - 1);
  std::size_t size = 1;
  while (size < needed) {
    if (size > top / 2) return 0;
    size <<= 1;
  }
  return size;
}

// ---- projection split and plain FIR -------------------------------------------------------------

Status bf16_split_hyena_projection(const DeviceBuffer &projection, const std::size_t length, const std::size_t width,
                                   DeviceBuffer *const x2, DeviceBuffer *const x1, DeviceBuffer *const value,
                                   const Stream &stream) {
  std::size_t bytes = 0;
  if (length == 0 || width == 0 || !product(length, width, kBf16Bytes, &bytes) ||
      bytes > std::numeric_limits<std::size_t>::max() / 3)
    return invalid("Hyena projection split: dimensions must be positive and representable");
  if (!holds(projection, 3 * bytes) || !holds(x2, bytes) || !holds(x1, bytes) || !holds(value, bytes) ||
      !on_device(stream, projection))
    return invalid("Hyena projection split: buffers are missing, too small or on another device");
  return from_code(evo_b200_bf16_split_hyena_projection(projection.data(), length, width, x2->data(), x1->data(),
                                                        value->data(), raw(stream)),
                   "Hyena projection split");
}

namespace {

Status check_fir_buffers(const DeviceBuffer &input, const DeviceBuffer &weight, const DeviceBuffer *bias,
                         const std::size_t channels, const DeviceBuffer *output, const FirShape &shape,
                         const Stream &stream) {
  if (!holds(input, shape.sequence_bytes) || !holds(weight, shape.weight_bytes) || !holds(output, shape.sequence_bytes) ||
      (bias != nullptr && !holds(*bias, channels * kBf16Bytes)) || !on_device(stream, input) ||
      !on_device(stream, weight) || !on_device(stream, *output))
    return invalid("FIR: buffers are missing, too small or on another device");
  return Status::Ok();
}

}  // namespace

Status bf16_fir_prefill_direct(const DeviceBuffer &input, const DeviceBuffer &weight, const DeviceBuffer *const bias,
                               const std::size_t length, const std::size_t channels, const std::size_t filter_groups,
                               const std::size_t kernel_size, const FirOrientation orientation,
                               const FirBiasMode bias_mode, DeviceBuffer *const output, FirCache *const cache,
                               const Stream &stream, const FirWeightType weight_type) {
  FirShape shape;
  auto status = fir_shape(length, channels, filter_groups, kernel_size, weight_type, &shape);
  if (!status.ok()) return status;
  status = check_fir_buffers(input, weight, bias, channels, output, shape, stream);
  if (!status.ok()) return status;
  status = check_fir_cache(cache, channels, kernel_size, stream);
  if (!status.ok()) return status;
  status = from_code(evo_b200_bf16_fir_prefill_direct(input.data(), weight.data(), weight_code(weight_type),
                                                      bias == nullptr ? nullptr : bias->data(), length, channels,
                                                      filter_groups, kernel_size, orientation_code(orientation),
                                                      bias_code(bias_mode), output->data(), cache_pointer(cache),
                                                      raw(stream)),
                     "FIR prefill");
  if (status.ok() && cache != nullptr) cache->length = std::min(length, kernel_size - 1);
  return status;
}

Status bf16_fir_continue_direct(const DeviceBuffer &input, const DeviceBuffer &weight, const DeviceBuffer *const bias,
                                const std::size_t length, const std::size_t channels, const std::size_t filter_groups,
                                const std::size_t kernel_size, const FirOrientation orientation,
                                const FirBiasMode bias_mode, DeviceBuffer *const output, FirCache *const cache,
                                const Stream &stream, const FirWeightType weight_type) {
  if (cache == nullptr) return invalid("FIR continuation needs a cache");
  FirShape shape;
  auto status = fir_shape(length, channels, filter_groups, kernel_size, weight_type, &shape);
  if (!status.ok()) return status;
  status = check_fir_buffers(input, weight, bias, channels, output, shape, stream);
  if (!status.ok()) return status;
  status = check_fir_cache(cache, channels, kernel_size, stream);
  if (!status.ok()) return status;
  if (kernel_size == 1) {
    // no history at all: the continuation is the prefill
    return from_code(evo_b200_bf16_fir_prefill_direct(input.data(), weight.data(), weight_code(weight_type),
                                                      bias == nullptr ? nullptr : bias->data(), length, channels,
                                                      filter_groups, kernel_size, orientation_code(orientation),
                                                      bias_code(bias_mode), output->data(), nullptr, raw(stream)),
                     "FIR continuation");
  }
  status = from_code(evo_b200_bf16_fir_continue_direct(input.data(), weight.data(), weight_code(weight_type),
                                                       bias == nullptr ? nullptr : bias->data(), length, channels,
                                                       filter_groups, kernel_size, orientation_code(orientation),
                                                       bias_code(bias_mode), cache_pointer(cache), cache->length,
                                                       output->data(), raw(stream)),
                     "FIR continuation");
  if (status.ok()) cache->length = grown(cache->length, length, kernel_size);
  return status;
}

Status bf16_fir_prefill_fft(const DeviceBuffer &input, const DeviceBuffer &weight, const DeviceBuffer *const bias,
                            const std::size_t length, const std::size_t channels, const std::size_t filter_groups,
                            const std::size_t kernel_size, const FirOrientation orientation, const FirBiasMode bias_mode,
                            DeviceBuffer *const output, FirCache *const cache, FftWorkspace *const workspace,
                            const Stream &stream, const FirWeightType weight_type) {
  if (workspace == nullptr || !stream.valid() ||
      !workspace->matches(stream.device(), channels, filter_groups, workspace->fft_size()) ||
      workspace->fft_size() < length)
    return invalid("FFT FIR prefill needs a workspace allocated for these channels, groups and length");
  return bf16_fir_prefill_direct(input, weight, bias, length, channels, filter_groups, kernel_size, orientation,
                                 bias_mode, output, cache, stream, weight_type);
}

Status bf16_fir_decode(const DeviceBuffer &input, const DeviceBuffer &weight, const DeviceBuffer *const bias,
                       const std::size_t channels, const std::size_t filter_groups, const std::size_t kernel_size,
                       const FirOrientation orientation, const FirBiasMode bias_mode, FirCache *const cache,
                       DeviceBuffer *const output, const Stream &stream, const FirWeightType weight_type) {
  return bf16_fir_continue_direct(input, weight, bias, 1, channels, filter_groups, kernel_size, orientation, bias_mode,
                                  output, cache, stream, weight_type);
}

// ---- gated short / medium convolutions ----------------------------------------------------------

namespace {

struct GatedCall final {
  const DeviceBuffer *x2;
  const DeviceBuffer *x1;
  const DeviceBuffer *value;
  const DeviceBuffer *weight;
  const DeviceBuffer *direct;  // null for HCS
  std::size_t length;
  std::size_t width;
  std::size_t groups;
  std::size_t kernel_size;
  FirOrientation orientation;
  FirWeightType weight_type;
  FirCache *cache;
  DeviceBuffer *scratch;
  DeviceBuffer *output;
};

Status check_gated(const GatedCall &call, const Stream &stream, FirShape *shape) {
  if (call.scratch == nullptr || call.output == nullptr) return invalid("gated FIR: scratch and output are required");
  auto status = fir_shape(call.length, call.width, call.groups, call.kernel_size, call.weight_type, shape);
  if (!status.ok()) return status;
  for (const DeviceBuffer *const buffer : {call.x2, call.x1, call.value,
                                           static_cast<const DeviceBuffer *>(call.scratch),
                                           static_cast<const DeviceBuffer *>(call.output)}) {
    if (!holds(*buffer, shape->sequence_bytes) || !on_device(stream, *buffer))
      return invalid("gated FIR: a sequence buffer is missing, too small or on another device");
  }
  if (!holds(*call.weight, shape->weight_bytes) || !on_device(stream, *call.weight) ||
      (call.direct != nullptr && (!holds(*call.direct, call.width * kBf16Bytes) || !on_device(stream, *call.direct))))
    return invalid("gated FIR: the filter or the direct term is missing, too small or on another device");
  return check_fir_cache(call.cache, call.width, call.kernel_size, stream);
}

// Whole-sequence form: one fused pass.
Status gated_prefill(const GatedCall &call, const Stream &stream, const char *what) {
  FirShape shape;
  auto status = check_gated(call, stream, &shape);
  if (!status.ok()) return status;
  status = from_code(
      evo_b200_bf16_gated_fir_prefill(call.x2->data(), call.x1->data(), call.value->data(), call.weight->data(),
                                      weight_code(call.weight_type), call.direct == nullptr ? nullptr : call.direct->data(),
                                      call.length, call.width, call.groups, call.kernel_size,
                                      orientation_code(call.orientation), call.scratch->data(), cache_pointer(call.cache),
                                      call.output->data(), raw(stream)),
      what);
  if (status.ok() && call.cache != nullptr) call.cache->length = std::min(call.length, call.kernel_size - 1);
  return status;
}

// Continuation from an F32 cache (decode is the one-row case): inner gate into the scratch buffer,
// the cached FIR on it, the outer gate in place.
Status gated_continue(const GatedCall &call, const Stream &stream, const char *what) {
  if (call.cache == nullptr) return invalid("gated FIR continuation needs a cache");
  FirShape shape;
  auto status = check_gated(call, stream, &shape);
  if (!status.ok()) return status;
  const std::size_t elements = call.length * call.width;
  status = from_code(evo_b200_bf16_gated_elementwise(call.x1->data(), call.value->data(), elements, 0,
                                                     call.scratch->data(), raw(stream)),
                     what);
  if (!status.ok()) return status;
  const void *const direct = call.direct == nullptr ? nullptr : call.direct->data();
  if (call.kernel_size == 1) {
    status = from_code(evo_b200_bf16_fir_prefill_direct(call.scratch->data(), call.weight->data(),
                                                        weight_code(call.weight_type), direct, call.length, call.width,
                                                        call.groups, 1, orientation_code(call.orientation), 1,
                                                        call.output->data(), nullptr, raw(stream)),
                       what);
  } else {
    status = from_code(evo_b200_bf16_fir_continue_direct(
                           call.scratch->data(), call.weight->data(), weight_code(call.weight_type), direct, call.length,
                           call.width, call.groups, call.kernel_size, orientation_code(call.orientation), 1,
                           cache_pointer(call.cache), call.cache->length, call.output->data(), raw(stream)),
                       what);
  }
  if (!status.ok()) return status;
  call.cache->length = grown(call.cache->length, call.length, call.kernel_size);
  return from_code(evo_b200_bf16_gated_elementwise(call.output->data(), call.x2->data(), elements, 0,
                                                   call.output->data(), raw(stream)),
                   what);
}

}  // namespace

Status bf16_hcs_prefill(const DeviceBuffer &x2, const DeviceBuffer &x1, const DeviceBuffer &value,
                        const DeviceBuffer &weight, const std::size_t length, const std::size_t width,
                        const std::size_t filter_groups, const std::size_t kernel_size, FirCache *const cache,
                        DeviceBuffer *const scratch, DeviceBuffer *const output, const Stream &stream) {
  return gated_prefill({&x2, &x1, &value, &weight, nullptr, length, width, filter_groups, kernel_size,
                        FirOrientation::kCrossCorrelation, FirWeightType::kBF16, cache, scratch, output},
                       stream, "HCS prefill");
}

Status bf16_hcs_decode(const DeviceBuffer &x2, const DeviceBuffer &x1, const DeviceBuffer &value,
                       const DeviceBuffer &weight, const std::size_t width, const std::size_t filter_groups,
                       const std::size_t kernel_size, FirCache *const cache, DeviceBuffer *const scratch,
                       DeviceBuffer *const output, const Stream &stream) {
  return gated_continue({&x2, &x1, &value, &weight, nullptr, 1, width, filter_groups, kernel_size,
                         FirOrientation::kCrossCorrelation, FirWeightType::kBF16, cache, scratch, output},
                        stream, "HCS decode");
}

Status bf16_hcs_continue(const DeviceBuffer &x2, const DeviceBuffer &x1, const DeviceBuffer &value,
                         const DeviceBuffer &weight, const std::size_t length, const std::size_t width,
                         const std::size_t filter_groups, const std::size_t kernel_size, FirCache *const cache,
                         DeviceBuffer *const scratch, DeviceBuffer *const output, const Stream &stream) {
  return gated_continue({&x2, &x1, &value, &weight, nullptr, length, width, filter_groups, kernel_size,
                         FirOrientation::kCrossCorrelation, FirWeightType::kBF16, cache, scratch, output},
                        stream, "HCS continuation");
}

Status bf16_hcm_prefill_direct(const DeviceBuffer &x2, const DeviceBuffer &x1, const DeviceBuffer &value,
                               const DeviceBuffer &weight, const DeviceBuffer &direct, const std::size_t length,
                               const std::size_t width, const std::size_t filter_groups, const std::size_t kernel_size,
                               FirCache *const cache, DeviceBuffer *const scratch, DeviceBuffer *const output,
                               const Stream &stream, const FirWeightType weight_type) {
  return gated_prefill({&x2, &x1, &value, &weight, &direct, length, width, filter_groups, kernel_size,
                        FirOrientation::kCausalConvolution, weight_type, cache, scratch, output},
                       stream, "HCM prefill");
}

Status bf16_hcm_prefill(const DeviceBuffer &x2, const DeviceBuffer &x1, const DeviceBuffer &value,
                        const DeviceBuffer &weight, const DeviceBuffer &direct, const std::size_t length,
                        const std::size_t width, const std::size_t filter_groups, const std::size_t kernel_size,
                        FirCache *const cache, DeviceBuffer *const scratch, DeviceBuffer *const output,
                        FftWorkspace *const workspace, const Stream &stream, const FirWeightType weight_type) {
  if (workspace == nullptr || !stream.valid() ||
      !workspace->matches(stream.device(), width, filter_groups, hcm_fft_size(length)))
    return invalid("HCM prefill needs an FFT workspace allocated for exactly this width, groups and 2 x length");
  return bf16_hcm_prefill_direct(x2, x1, value, weight, direct, length, width, filter_groups, kernel_size, cache,
                                 scratch, output, stream, weight_type);
}

Status bf16_hcm_decode(const DeviceBuffer &x2, const DeviceBuffer &x1, const DeviceBuffer &value,
                       const DeviceBuffer &weight, const DeviceBuffer &direct, const std::size_t width,
                       const std::size_t filter_groups, const std::size_t kernel_size, FirCache *const cache,
                       DeviceBuffer *const scratch, DeviceBuffer *const output, const Stream &stream,
                       const FirWeightType weight_type) {
  return gated_continue({&x2, &x1, &value, &weight, &direct, 1, width, filter_groups, kernel_size,
                         FirOrientation::kCausalConvolution, weight_type, cache, scratch, output},
                        stream, "HCM decode");
}

Status bf16_hcm_continue(const DeviceBuffer &x2, const DeviceBuffer &x1, const DeviceBuffer &value,
                         const DeviceBuffer &weight, const DeviceBuffer &direct, const std::size_t length,
                         const std::size_t width, const std::size_t filter_groups, const std::size_t kernel_size,
                         FirCache *const cache, DeviceBuffer *const scratch, DeviceBuffer *const output,
                         const Stream &stream, const FirWeightType weight_type) {
  return gated_continue({&x2, &x1, &value, &weight, &direct, length, width, filter_groups, kernel_size,
                         FirOrientation::kCausalConvolution, weight_type, cache, scratch, output},
                        stream, "HCM continuation");
}

// ---- long (modal) convolution -------------------------------------------------------------------

namespace {

Status check_modal(const DeviceBuffer &x2, const DeviceBuffer &x1, const DeviceBuffer &value, const DeviceBuffer &direct,
                   const DeviceBuffer &log_poles, const DeviceBuffer &residues, const std::size_t length,
                   const std::size_t width, const std::size_t state_size, const IirCache *cache,
                   const DeviceBuffer *scratch, const DeviceBuffer *output, const Stream &stream) {
  std::size_t sequence_bytes = 0, modal_bytes = 0;
  if (length == 0 || width == 0 || state_size == 0 || !product(length, width, kBf16Bytes, &sequence_bytes) ||
      !product(width, state_size, sizeof(float), &modal_bytes))
    return invalid("HCL: length, width and state size must be positive and representable");
  for (const DeviceBuffer *const buffer : {&x2, &x1, &value, scratch, output}) {
    if (buffer == nullptr || !holds(*buffer, sequence_bytes) || !on_device(stream, *buffer))
      return invalid("HCL: a sequence buffer is missing, too small or on another device");
  }
  if (!holds(direct, width * kBf16Bytes) || !holds(log_poles, modal_bytes) || !holds(residues, modal_bytes) ||
      !on_device(stream, direct) || !on_device(stream, log_poles) || !on_device(stream, residues))
    return invalid("HCL: the direct term, poles or residues are missing, too small or on another device");
  if (cache != nullptr && (cache->channels != width || cache->state_size != state_size ||
                           !holds(cache->state, modal_bytes) || !on_device(stream, cache->state)))
    return invalid("HCL: the modal cache does not match width and state size");
  return Status::Ok();
}

}  // namespace

Status bf16_hcl_prefill(const DeviceBuffer &x2, const DeviceBuffer &x1, const DeviceBuffer &value,
                        const DeviceBuffer &direct, const DeviceBuffer &log_poles, const DeviceBuffer &residues,
                        const std::size_t length, const std::size_t width, const std::size_t state_size,
                        const HclPrefillMode mode, IirCache *const cache, DeviceBuffer *const scratch,
                        DeviceBuffer *const output, FftWorkspace *const workspace, const Stream &stream) {
  auto status =
      check_modal(x2, x1, value, direct, log_poles, residues, length, width, state_size, cache, scratch, output, stream);
  if (!status.ok()) return status;
  const bool fft_mode = mode == HclPrefillMode::kFft || mode == HclPrefillMode::kFftStateless;
  if (fft_mode && (workspace == nullptr || !workspace->matches(stream.device(), width, width, hcl_fft_size(length),
                                                               FftInputMode::kRealFullSpectrum)))
    return invalid("HCL FFT prefill needs a full-spectrum workspace allocated for exactly this width and 2 x length");
  if (mode != HclPrefillMode::kFftStateless && cache == nullptr)
    return invalid("HCL prefill needs a modal cache unless it is stateless");
  float *const state =
      mode == HclPrefillMode::kFftStateless ? nullptr : static_cast<float *>(cache->state.data());
  const int continue_from_state = mode == HclPrefillMode::kRecurrenceContinue ? 1 : 0;
  return from_code(evo_b200_bf16_hcl_prefill_noalloc(
                       x2.data(), x1.data(), value.data(), direct.data(), static_cast<const float *>(log_poles.data()),
                       static_cast<const float *>(residues.data()), length, width, state_size, continue_from_state, state,
                       scratch->data(), output->data(), raw(stream)),
                   "HCL prefill");
}

Status bf16_hcl_decode(const DeviceBuffer &x2, const DeviceBuffer &x1, const DeviceBuffer &value,
                       const DeviceBuffer &direct, const DeviceBuffer &log_poles, const DeviceBuffer &residues,
                       const std::size_t width, const std::size_t state_size, IirCache *const cache,
                       DeviceBuffer *const gated, DeviceBuffer *const output, const Stream &stream) {
  if (cache == nullptr) return invalid("HCL decode needs a modal cache");
  auto status = check_modal(x2, x1, value, direct, log_poles, residues, 1, width, state_size, cache, gated, output, stream);
  if (!status.ok()) return status;
  return from_code(evo_b200_bf16_hcl_decode(x2.data(), x1.data(), value.data(), direct.data(),
                                            static_cast<const float *>(log_poles.data()),
                                            static_cast<const float *>(residues.data()), width, state_size,
                                            static_cast<float *>(cache->state.data()), gated->data(), output->data(),
                                            raw(stream)),
                   "HCL decode");
}

}  // namespace evo::cuda
