// Dense-linear offload with upstream's LinearExecutor contract
// (src/linear_executor.hpp:13-28): F32 host activations [rows, in], a host
// weight view [out, in] row-major (F32, BF16 or raw E4M3 codes), optional bias,
// F32 host output; the executor may keep device copies of weights keyed by their host
// address (upstream's Metal executor does, src/mps/model.mm:218-238), and
// serialises calls internally.
//
// The contract is F32 arithmetic, the fast units are BF16 tensor cores, so
// operands are split into BF16 planes: x = x0 + x1 + x2 with x0 = bf16(x),
// x1 = bf16(x - x0), x2 = bf16(x - x0 - x1) represents an F32 value to ~2^-24,
// every BF16 x BF16 product is exact in the F32 accumulator, and
//   y = [x0 | x1 | x2] . W^T                      (BF16 weights: one launch)
//   y = x012 . W0^T + x01 . W1^T + x0 . W2^T      (F32 weights: three launches)
// runs on the tcgen05 projection kernel in its F32-result mode, the weight's K
// coordinate wrapping so the planes of x meet the same weight columns.  What is
// left of the error is the tensor-core accumulator's truncation when it aligns
// partial sums: a few 1e-6 of sum(|x||w|) at K = 4096.
#include <cuda_runtime.h>

#include <map>
#include <mutex>
#include <new>
#include <string>
#include <tuple>

#include "common.cuh"
#include "ops_internal.hpp"

namespace evob {
namespace {

constexpr std::size_t kBlock = 64;  // K is padded to whole tensor-core K blocks

std::size_t padded(const std::size_t k) { return (k + kBlock - 1) / kBlock * kBlock; }

// planes of BF16 residuals of an F32 matrix, each [rows, pitch] with zero padding;
// destination layout [rows, planes * pitch] (planes side by side) when interleaved,
// else planes stacked as separate [rows, pitch] matrices.
__global__ void split_planes_kernel(const float *__restrict__ source, bf16 *__restrict__ planes,
                                    const std::size_t rows, const std::size_t width,
                                    const std::size_t pitch, const int count, const bool side_by_side) {
  const std::size_t total = rows * pitch;
  const std::size_t stride = static_cast<std::size_t>(blockDim.x) * gridDim.x;
  for (std::size_t i = static_cast<std::size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const std::size_t row = i / pitch, column = i % pitch;
    float remainder = column < width ? source[row * width + column] : 0.0F;
    for (int plane = 0; plane < count; ++plane) {
      const bf16 part = f2bf(remainder);
      remainder -= bf2f(part);
      const std::size_t at = side_by_side ? (row * count + plane) * pitch + column
                                          : (static_cast<std::size_t>(plane) * rows + row) * pitch + column;
      planes[at] = part;
    }
  }
}

__global__ void widen_bf16_kernel(const bf16 *__restrict__ source, float *__restrict__ target, const std::size_t count) {
  const std::size_t stride = static_cast<std::size_t>(blockDim.x) * gridDim.x;
  for (std::size_t i = static_cast<std::size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride)
    target[i] = bf2f(source[i]);
}

// BF16 host weight -> padded device copy [rows, pitch]
__global__ void pad_bf16_kernel(const bf16 *__restrict__ source, bf16 *__restrict__ target, const std::size_t rows,
                                const std::size_t width, const std::size_t pitch) {
  const std::size_t total = rows * pitch;
  const std::size_t stride = static_cast<std::size_t>(blockDim.x) * gridDim.x;
  for (std::size_t i = static_cast<std::size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const std::size_t row = i / pitch, column = i % pitch;
    target[i] = column < width ? source[row * width + column] : f2bf(0.0F);
  }
}

// E4M3 codes -> padded BF16 [rows, pitch].  Every finite E4M3 value is a BF16
// value, so one plane holds the weight exactly (upstream's Metal executor
// decodes the codes the same way, without a scale: src/mps/model.mm:42-58).
__global__ void decode_e4m3_kernel(const std::uint8_t *__restrict__ source, bf16 *__restrict__ target,
                                   const std::size_t rows, const std::size_t width, const std::size_t pitch) {
  const std::size_t total = rows * pitch;
  const std::size_t stride = static_cast<std::size_t>(blockDim.x) * gridDim.x;
  for (std::size_t i = static_cast<std::size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const std::size_t row = i / pitch, column = i % pitch;
    float value = 0.0F;
    if (column < width) {
      const unsigned int code = source[row * width + column];
      const unsigned int magnitude = code & 0x7fU, exponent = magnitude >> 3U, fraction = magnitude & 7U;
      value = magnitude == 0x7fU ? __int_as_float(0x7fc00000)
              : exponent == 0    ? static_cast<float>(fraction) * 0.001953125F
                                 : ldexpf(static_cast<float>(8U + fraction), static_cast<int>(exponent) - 10);
      if ((code & 0x80U) != 0) value = -value;
    }
    target[i] = f2bf(value);
  }
}

unsigned int grid_for(const std::size_t items) {
  const std::size_t blocks = (items + 255) / 256;
  return static_cast<unsigned int>(blocks < 1 ? 1 : (blocks > 148 * 32 ? 148 * 32 : blocks));
}

struct DeviceBuffer {
  void *data = nullptr;
  std::size_t bytes = 0;
  int reserve(const std::size_t wanted) {
    if (wanted <= bytes) return kOk;
    if (data != nullptr) cudaFree(data);
    data = nullptr;
    bytes = 0;
    if (cudaMalloc(&data, wanted) != cudaSuccess)
      return fail(kCuda, "linear executor: cannot allocate " + std::to_string(wanted >> 20) + " MiB");
    bytes = wanted;
    return kOk;
  }
  ~DeviceBuffer() {
    if (data != nullptr) cudaFree(data);
  }
};

struct CachedWeight {
  bf16 *planes = nullptr;  // [plane_count][out, pitch]
  int plane_count = 0;
  std::size_t out = 0, pitch = 0;
};

}  // namespace

struct LinearExecutorState {
  int device = 0;
  cudaStream_t stream = nullptr;
  std::mutex mutex;
  std::map<std::tuple<const void *, std::size_t, int>, CachedWeight> weights;
  DeviceBuffer staging, input_planes, output, bias;
  std::size_t cached_bytes = 0;

  ~LinearExecutorState() {
    cudaSetDevice(device);
    if (stream != nullptr) cudaStreamSynchronize(stream);
    for (auto &entry : weights) cudaFree(entry.second.planes);
    if (stream != nullptr) cudaStreamDestroy(stream);
  }
};

int linear_executor_create(const int device, LinearExecutorState **out) {
  if (out == nullptr) return fail(kInvalidArgument, "linear executor output is null");
  *out = nullptr;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count)
    return fail(kInvalidArgument, "linear executor: CUDA device index is out of range");
  auto *state = new (std::nothrow) LinearExecutorState();
  if (state == nullptr) return fail(kInternal, "out of host memory");
  state->device = device;
  if (cudaSetDevice(device) != cudaSuccess ||
      cudaStreamCreateWithFlags(&state->stream, cudaStreamNonBlocking) != cudaSuccess) {
    delete state;
    return fail(kCuda, "linear executor: cannot create a stream");
  }
  *out = state;
  return kOk;
}

void linear_executor_free(LinearExecutorState *state) { delete state; }

std::size_t linear_executor_cached_bytes(LinearExecutorState *state) {
  if (state == nullptr) return 0;
  std::lock_guard<std::mutex> lock(state->mutex);
  return state->cached_bytes;
}

// dtype: 0 = F32, 1 = BF16, 2 = E4M3 codes (upstream TensorDType kF32 / kBF16 /
// kE4M3Software); biases are F32 or BF16
int linear_executor_linear(LinearExecutorState *state, const float *input, const std::size_t rows,
                           const std::size_t input_width, const void *weight, const int weight_dtype,
                           const std::size_t weight_elements, const std::size_t output_width,
                           const void *bias, const int bias_dtype, const std::size_t bias_elements,
                           float *output) {
  if (state == nullptr || input == nullptr || weight == nullptr || output == nullptr || input_width == 0 ||
      output_width == 0)
    return fail(kInvalidArgument, "linear executor arguments are invalid");
  if (weight_elements != output_width * input_width)
    return fail(kInternal, "host linear dimensions are inconsistent");
  if (weight_dtype < 0 || weight_dtype > 2 || (bias != nullptr && bias_dtype != 0 && bias_dtype != 1))
    return fail(kUnsupported, "linear executor takes F32, BF16 or E4M3 weights and F32 or BF16 biases");
  if (bias != nullptr && bias_elements != output_width)
    return fail(kInternal, "host linear bias width is inconsistent");
  if (rows == 0) return kOk;
  if (output_width < 64)
    return fail(kUnsupported, "linear executor: outputs narrower than 64 stay on the host");
  std::lock_guard<std::mutex> lock(state->mutex);
  int previous = 0;
  cudaGetDevice(&previous);
  if (cudaSetDevice(state->device) != cudaSuccess) return fail(kCuda, "linear executor: cannot select its device");
  struct Restore {
    int device;
    ~Restore() { cudaSetDevice(device); }
  } restore{previous};
  cudaStream_t stream = state->stream;
  const std::size_t pitch = padded(input_width);

  // ---- weight planes, cached by host address
  const auto key = std::make_tuple(weight, weight_elements, weight_dtype);
  auto found = state->weights.find(key);
  if (found == state->weights.end()) {
    CachedWeight entry;
    entry.plane_count = weight_dtype == 0 ? 3 : 1;
    entry.out = output_width;
    entry.pitch = pitch;
    const std::size_t element = weight_dtype == 0 ? 4 : weight_dtype == 1 ? 2 : 1;
    const std::size_t plane_bytes = output_width * pitch * 2;
    int status = state->staging.reserve(weight_elements * element);
    if (status != kOk) return status;
    void *planes = nullptr;
    if (cudaMalloc(&planes, plane_bytes * entry.plane_count) != cudaSuccess)
      return fail(kCuda, "linear executor: cannot allocate a device copy of the weight");
    entry.planes = static_cast<bf16 *>(planes);
    if (cudaMemcpyAsync(state->staging.data, weight, weight_elements * element, cudaMemcpyHostToDevice, stream) !=
        cudaSuccess) {
      cudaFree(planes);
      return fail(kCuda, "linear executor: weight upload failed");
    }
    if (weight_dtype == 0)
      split_planes_kernel<<<grid_for(output_width * pitch), 256, 0, stream>>>(
          static_cast<const float *>(state->staging.data), entry.planes, output_width, input_width, pitch, 3, false);
    else if (weight_dtype == 1)
      pad_bf16_kernel<<<grid_for(output_width * pitch), 256, 0, stream>>>(
          static_cast<const bf16 *>(state->staging.data), entry.planes, output_width, input_width, pitch);
    else
      decode_e4m3_kernel<<<grid_for(output_width * pitch), 256, 0, stream>>>(
          static_cast<const std::uint8_t *>(state->staging.data), entry.planes, output_width, input_width, pitch);
    status = check_launch("linear executor weight conversion");
    if (status != kOk || cudaStreamSynchronize(stream) != cudaSuccess) {
      cudaFree(planes);
      return status != kOk ? status : fail(kCuda, "linear executor: weight conversion failed");
    }
    state->cached_bytes += plane_bytes * entry.plane_count;
    found = state->weights.emplace(key, entry).first;
  }
  const CachedWeight &cached = found->second;

  // ---- activations: upload, split into three planes side by side
  int status = state->staging.reserve(rows * input_width * 4);
  if (status == kOk) status = state->input_planes.reserve(rows * 3 * pitch * 2 * 2);  // 3-plane and narrower forms
  if (status == kOk) status = state->output.reserve(rows * output_width * 4);
  if (status != kOk) return status;
  if (cudaMemcpyAsync(state->staging.data, input, rows * input_width * 4, cudaMemcpyHostToDevice, stream) !=
      cudaSuccess)
    return fail(kCuda, "linear executor: activation upload failed");
  const float *bias_device = nullptr;
  if (bias != nullptr) {
    status = state->bias.reserve(output_width * 4 + output_width * 2);
    if (status != kOk) return status;
    float *const target = static_cast<float *>(state->bias.data);
    if (bias_dtype == 0) {
      if (cudaMemcpyAsync(target, bias, output_width * 4, cudaMemcpyHostToDevice, stream) != cudaSuccess)
        return fail(kCuda, "linear executor: bias upload failed");
    } else {
      bf16 *const raw = reinterpret_cast<bf16 *>(target + output_width);
      if (cudaMemcpyAsync(raw, bias, output_width * 2, cudaMemcpyHostToDevice, stream) != cudaSuccess)
        return fail(kCuda, "linear executor: bias upload failed");
      widen_bf16_kernel<<<grid_for(output_width), 256, 0, stream>>>(raw, target, output_width);
    }
    bias_device = target;
  }
  bf16 *const planes3 = static_cast<bf16 *>(state->input_planes.data);
  bf16 *const narrower = planes3 + rows * 3 * pitch;
  for (int term = 0; term < cached.plane_count && status == kOk; ++term) {
    // weight plane `term` meets the 3 - term most significant activation planes
    const int count = 3 - term;
    bf16 *const a = term == 0 ? planes3 : narrower;
    split_planes_kernel<<<grid_for(rows * pitch), 256, 0, stream>>>(static_cast<const float *>(state->staging.data), a,
                                                                    rows, input_width, pitch, count, true);
    status = check_launch("linear executor activation split");
    if (status != kOk) break;
    LinearArgs args;
    args.input = a;
    args.weight = cached.planes + static_cast<std::size_t>(term) * cached.out * cached.pitch;
    args.rows = rows;
    args.in_features = static_cast<std::size_t>(count) * pitch;
    args.out_features = output_width;
    args.output_f32 = static_cast<float *>(state->output.data);
    args.bias_f32 = term == 0 ? bias_device : nullptr;
    args.accumulate_f32 = term != 0;
    args.weight_wrap_features = pitch;
    status = linear(args, stream);
  }
  if (status != kOk) return status;
  if (cudaMemcpyAsync(output, state->output.data, rows * output_width * 4, cudaMemcpyDeviceToHost, stream) !=
          cudaSuccess ||
      cudaStreamSynchronize(stream) != cudaSuccess)
    return fail(kCuda, std::string("linear executor: result read-back failed: ") +
                           cudaGetErrorString(cudaGetLastError()));
  return gemm_error_state(stream);
}

}  // namespace evob
