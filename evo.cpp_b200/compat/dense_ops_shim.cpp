// evo::cuda dense operators (upstream include/evo/cuda/ops.hpp:13-141) on this library's C entry
// points.  Each function checks the buffers against the sizes its arguments imply, then makes one or
// a few evo_b200_* calls on the caller's stream; see compat_common.hpp for what the layer is.
//
// Differences a caller can observe:
//  * Bf16LinearPlan holds no cuBLASLt objects.  It remembers the problem (sizes, layouts, whether a
//    bias is fused) it was last used for, and build_count() counts how often that changed, which is
//    when upstream would have rebuilt its plan.
//  * The `workspace` of bf16_linear and the `blas` buffer of MlpWorkspace are accepted and unused
//    unless a projection of 9..128 rows can use them for split-K partial sums.
#include "compat_common.hpp"

#include <memory>
#include <utility>

#include "evo/cuda/ops.hpp"

namespace evo::cuda {

using evo_b200_compat::from_code;
using evo_b200_compat::holds;
using evo_b200_compat::invalid;
using evo_b200_compat::kBf16Bytes;
using evo_b200_compat::product;
using evo_b200_compat::StreamScratch;

namespace {

void *raw(const Stream &stream) { return static_cast<void *>(stream.get()); }

bool usable(const Stream &stream, const DeviceBuffer &any) {
  return stream.valid() && any.valid() && stream.device() == any.device();
}

}  // namespace

// ---- Bf16LinearPlan -----------------------------------------------------------------------------

struct Bf16LinearPlan::Impl final {
  std::size_t rows{0};
  std::size_t in_features{0};
  std::size_t out_features{0};
  bool fused_bias{false};
  LinearWeightLayout weight_layout{LinearWeightLayout::kOutputMajor};
  LinearInputLayout input_layout{LinearInputLayout::kRowMajor};
  bool used{false};

  bool same(const Impl &other) const noexcept {
    return used && other.used && rows == other.rows && in_features == other.in_features &&
           out_features == other.out_features && fused_bias == other.fused_bias &&
           weight_layout == other.weight_layout && input_layout == other.input_layout;
  }
};

Bf16LinearPlan::Bf16LinearPlan() = default;
Bf16LinearPlan::~Bf16LinearPlan() = default;

Bf16LinearPlan::Bf16LinearPlan(Bf16LinearPlan &&other) noexcept
    : impl_(std::move(other.impl_)), build_count_(std::exchange(other.build_count_, 0)) {}

Bf16LinearPlan &Bf16LinearPlan::operator=(Bf16LinearPlan &&other) noexcept {
  if (this != &other) {
    impl_ = std::move(other.impl_);
    build_count_ = std::exchange(other.build_count_, 0);
  }
  return *this;
}

// ---- MlpWorkspace -------------------------------------------------------------------------------

Status MlpWorkspace::allocate(const int device, const std::size_t rows, const std::size_t inner_width,
                              const std::size_t blas_bytes) {
  std::size_t bytes = 0;
  if (rows == 0 || inner_width == 0 || !product(rows, inner_width, kBf16Bytes, &bytes))
    return invalid("MLP workspace: rows and inner width must be positive and their product representable");
  for (DeviceBuffer *const buffer : {&first, &second, &activated, &gated}) {
    auto status = buffer->allocate(device, bytes);
    if (!status.ok()) return status;
  }
  if (blas_bytes != 0) return blas.allocate(device, blas_bytes);
  blas.reset();
  return Status::Ok();
}

// ---- projections --------------------------------------------------------------------------------

Status bf16_linear(const BlasLt &handle, const DeviceBuffer &input, const DeviceBuffer &weight,
                   const DeviceBuffer *const bias, const std::size_t rows, const std::size_t in_features,
                   const std::size_t out_features, DeviceBuffer *const output, DeviceBuffer *const workspace,
                   const Stream &stream, Bf16LinearPlan *const plan, const LinearWeightLayout weight_layout,
                   const LinearInputLayout input_layout) {
  std::size_t input_bytes = 0, weight_bytes = 0, output_bytes = 0;
  if (!handle.valid()) return invalid("BF16 linear: the BLAS handle has not been created");
  if (rows == 0 || in_features == 0 || out_features == 0 || !product(rows, in_features, kBf16Bytes, &input_bytes) ||
      !product(out_features, in_features, kBf16Bytes, &weight_bytes) ||
      !product(rows, out_features, kBf16Bytes, &output_bytes))
    return invalid("BF16 linear: dimensions must be positive and representable");
  if (!holds(input, input_bytes) || !holds(weight, weight_bytes) || !holds(output, output_bytes) ||
      (bias != nullptr && !holds(*bias, out_features * kBf16Bytes)))
    return invalid("BF16 linear: a buffer is missing or smaller than the dimensions require");
  if (!usable(stream, input) || weight.device() != input.device() || output->device() != input.device() ||
      (bias != nullptr && bias->device() != input.device()))
    return invalid("BF16 linear: buffers and stream must live on one device");

  if (plan != nullptr) {
    Bf16LinearPlan::Impl wanted;
    wanted.rows = rows;
    wanted.in_features = in_features;
    wanted.out_features = out_features;
    wanted.fused_bias = bias != nullptr;
    wanted.weight_layout = weight_layout;
    wanted.input_layout = input_layout;
    wanted.used = true;
    if (plan->impl_ == nullptr || !plan->impl_->same(wanted)) {
      plan->impl_ = std::make_unique<Bf16LinearPlan::Impl>(wanted);
      ++plan->build_count_;
    }
  }

  // The kernels take row-major activations and an output-major weight; the other two layouts are
  // brought into that form by the bit-exact transpose operator first.
  StreamScratch input_rows, weight_rows;
  const void *input_pointer = input.data();
  const void *weight_pointer = weight.data();
  if (input_layout == LinearInputLayout::kColumnMajor) {
    auto status = input_rows.allocate(input_bytes, stream.get());
    if (!status.ok()) return status;
    status = from_code(evo_b200_bf16_row_to_column_major(input.data(), in_features, rows, input_rows.data(), raw(stream)),
                       "BF16 linear: column-major input");
    if (!status.ok()) return status;
    input_pointer = input_rows.data();
  }
  if (weight_layout == LinearWeightLayout::kInputMajor) {
    auto status = weight_rows.allocate(weight_bytes, stream.get());
    if (!status.ok()) return status;
    status = from_code(
        evo_b200_bf16_row_to_column_major(weight.data(), in_features, out_features, weight_rows.data(), raw(stream)),
        "BF16 linear: input-major weight");
    if (!status.ok()) return status;
    weight_pointer = weight_rows.data();
  }
  const void *const bias_pointer = bias == nullptr ? nullptr : bias->data();
  const int bias_mode = bias == nullptr ? 0 : 1;  // upstream fuses the bias into the F32 sum
  if (workspace != nullptr && workspace->valid() && workspace->device() == input.device() && rows >= 9 && rows <= 128) {
    return from_code(evo_b200_bf16_linear_split_k(input_pointer, weight_pointer, bias_pointer, nullptr, rows, in_features,
                                                  out_features, bias_mode, 0, workspace->data(), workspace->bytes(),
                                                  output->data(), raw(stream)),
                     "BF16 linear");
  }
  return from_code(evo_b200_bf16_linear(input_pointer, weight_pointer, bias_pointer, nullptr, rows, in_features,
                                        out_features, bias_mode, 0, output->data(), raw(stream)),
                   "BF16 linear");
}

Status bf16_row_to_column_major(const DeviceBuffer &input, const std::size_t rows, const std::size_t columns,
                                DeviceBuffer *const output, const Stream &stream) {
  std::size_t bytes = 0;
  if (rows == 0 || columns == 0 || !product(rows, columns, kBf16Bytes, &bytes))
    return invalid("BF16 transpose: dimensions must be positive and representable");
  if (!holds(input, bytes) || !holds(output, bytes) || !usable(stream, input) || output->device() != input.device())
    return invalid("BF16 transpose: buffers are missing, too small or on another device");
  if (output->data() == input.data()) return invalid("BF16 transpose cannot run in place");
  return from_code(evo_b200_bf16_row_to_column_major(input.data(), rows, columns, output->data(), raw(stream)),
                   "BF16 transpose");
}

// ---- E4M3 ---------------------------------------------------------------------------------------

namespace {

Status check_scale(const float scale) {
  if (!(scale > 0.0F) || scale > std::numeric_limits<float>::max())
    return invalid("E4M3 quantisation needs a positive finite scale");
  return Status::Ok();
}

}  // namespace

Status software_e4m3_quantize_bf16(const DeviceBuffer &input, const std::size_t elements, const float scale,
                                   DeviceBuffer *const codes, DeviceBuffer *const dequantized_f32, const Stream &stream) {
  auto status = check_scale(scale);
  if (!status.ok()) return status;
  std::size_t value_bytes = 0;
  if (elements == 0 || !product(elements, sizeof(float), 1, &value_bytes))
    return invalid("E4M3 quantisation: the element count must be positive and representable");
  if (!holds(input, elements * kBf16Bytes) || !holds(dequantized_f32, value_bytes) ||
      (codes != nullptr && !holds(*codes, elements)) || !usable(stream, input))
    return invalid("E4M3 quantisation: buffers are missing, too small or on another device");
  return from_code(evo_b200_software_e4m3_quantize_bf16(input.data(), elements, scale,
                                                        codes == nullptr ? nullptr : codes->data(),
                                                        static_cast<float *>(dequantized_f32->data()), raw(stream)),
                   "E4M3 quantisation");
}

Status software_e4m3_quantize_bf16_codes(const DeviceBuffer &input, const std::size_t elements, const float scale,
                                         DeviceBuffer *const codes, const Stream &stream) {
  auto status = check_scale(scale);
  if (!status.ok()) return status;
  if (elements == 0 || elements > std::numeric_limits<std::size_t>::max() / kBf16Bytes)
    return invalid("E4M3 code quantisation: the element count must be positive and representable");
  if (!holds(input, elements * kBf16Bytes) || !holds(codes, elements) || !usable(stream, input))
    return invalid("E4M3 code quantisation: buffers are missing, too small or on another device");
  return from_code(
      evo_b200_software_e4m3_quantize_bf16(input.data(), elements, scale, codes->data(), nullptr, raw(stream)),
      "E4M3 code quantisation");
}

Status software_e4m3_quantize_f32_codes(const DeviceBuffer &input, const std::size_t elements, const float scale,
                                        DeviceBuffer *const codes, const Stream &stream) {
  auto status = check_scale(scale);
  if (!status.ok()) return status;
  std::size_t input_bytes = 0;
  if (elements == 0 || !product(elements, sizeof(float), 1, &input_bytes))
    return invalid("F32 to E4M3: the element count must be positive and representable");
  if (!holds(input, input_bytes) || !holds(codes, elements) || !usable(stream, input))
    return invalid("F32 to E4M3: buffers are missing, too small or on another device");
  return from_code(evo_b200_software_e4m3_quantize_f32_codes(static_cast<const float *>(input.data()), elements, scale,
                                                             codes->data(), raw(stream)),
                   "F32 to E4M3");
}

Status software_e4m3_h100_linear(const DeviceBuffer &input, const DeviceBuffer &weight_codes, const std::size_t rows,
                                 const std::size_t in_features, const std::size_t out_features, const float input_scale,
                                 const float output_scale, DeviceBuffer *const input_codes_workspace,
                                 DeviceBuffer *const output, const Stream &stream) {
  std::size_t code_bytes = 0, weight_bytes = 0, output_bytes = 0;
  if (rows == 0 || in_features == 0 || out_features == 0 || !product(rows, in_features, kBf16Bytes, &code_bytes) ||
      !product(out_features, in_features, 1, &weight_bytes) || !product(rows, out_features, kBf16Bytes, &output_bytes))
    return invalid("software QGMMA: dimensions must be positive and representable");
  code_bytes /= kBf16Bytes;
  if (in_features % 32 != 0) return invalid("software QGMMA: the inner dimension must be a multiple of 32");
  auto status = check_scale(input_scale);
  if (!status.ok()) return status;
  if (!(output_scale == output_scale) || output_scale > std::numeric_limits<float>::max() ||
      output_scale < -std::numeric_limits<float>::max())
    return invalid("software QGMMA: the output scale must be finite");
  if (!holds(input, code_bytes * kBf16Bytes) || !holds(weight_codes, weight_bytes) ||
      !holds(input_codes_workspace, code_bytes) || !holds(output, output_bytes) || !usable(stream, input))
    return invalid("software QGMMA: buffers are missing, too small or on another device");
  return from_code(evo_b200_software_e4m3_h100_linear(input.data(), weight_codes.data(), rows, in_features, out_features,
                                                      input_scale, output_scale, input_codes_workspace->data(),
                                                      output->data(), raw(stream)),
                   "software QGMMA");
}

// ---- normalisation and element-wise -------------------------------------------------------------

Status bf16_rms_norm(const DeviceBuffer &input, const DeviceBuffer &scale, const std::size_t rows, const std::size_t width,
                     const float epsilon, DeviceBuffer *const output, const Stream &stream) {
  std::size_t bytes = 0;
  if (rows == 0 || width == 0 || !product(rows, width, kBf16Bytes, &bytes))
    return invalid("RMSNorm: dimensions must be positive and representable");
  if (!(epsilon >= 0.0F) || epsilon > std::numeric_limits<float>::max())
    return invalid("RMSNorm: epsilon must be finite and not negative");
  if (!holds(input, bytes) || !holds(scale, width * sizeof(float)) || !holds(output, bytes) || !usable(stream, input))
    return invalid("RMSNorm: buffers are missing, too small or on another device");
  return from_code(evo_b200_bf16_rms_norm(input.data(), static_cast<const float *>(scale.data()), rows, width, epsilon,
                                          output->data(), nullptr, 1.0F, raw(stream)),
                   "RMSNorm");
}

namespace {

Status check_elementwise(const DeviceBuffer &first, const DeviceBuffer *second, const std::size_t elements,
                         const DeviceBuffer *output, const Stream &stream, const char *what) {
  if (elements == 0 || elements > std::numeric_limits<std::size_t>::max() / kBf16Bytes) return invalid(what);
  const std::size_t bytes = elements * kBf16Bytes;
  if (!holds(first, bytes) || (second != nullptr && !holds(*second, bytes)) || !holds(output, bytes) ||
      !usable(stream, first))
    return invalid(what);
  return Status::Ok();
}

}  // namespace

Status bf16_gated_elementwise(const DeviceBuffer &first, const DeviceBuffer &second, const std::size_t elements,
                              const GatedActivation activation, DeviceBuffer *const output, const Stream &stream) {
  auto status = check_elementwise(first, &second, elements, output, stream,
                                  "gated product: element count or buffers do not fit");
  if (!status.ok()) return status;
  return from_code(evo_b200_bf16_gated_elementwise(first.data(), second.data(), elements,
                                                   activation == GatedActivation::kGelu ? 1 : 0, output->data(),
                                                   raw(stream)),
                   "gated product");
}

Status bf16_gelu(const DeviceBuffer &input, const std::size_t elements, DeviceBuffer *const output, const Stream &stream) {
  auto status = check_elementwise(input, nullptr, elements, output, stream, "GELU: element count or buffers do not fit");
  if (!status.ok()) return status;
  return from_code(evo_b200_bf16_gelu(input.data(), elements, output->data(), raw(stream)), "GELU");
}

Status bf16_add_inplace(DeviceBuffer *const output, const DeviceBuffer &residual, const std::size_t elements,
                        const Stream &stream) {
  if (output == nullptr) return invalid("residual add: no output buffer");
  auto status = check_elementwise(residual, output, elements, output, stream,
                                  "residual add: element count or buffers do not fit");
  if (!status.ok()) return status;
  return from_code(evo_b200_bf16_add(output->data(), residual.data(), elements, output->data(), raw(stream)),
                   "residual add");
}

Status bf16_add_bias_inplace(DeviceBuffer *const output, const DeviceBuffer &bias, const std::size_t rows,
                             const std::size_t width, const Stream &stream) {
  std::size_t bytes = 0;
  if (rows == 0 || width == 0 || !product(rows, width, kBf16Bytes, &bytes))
    return invalid("bias add: dimensions must be positive and representable");
  if (!holds(output, bytes) || !holds(bias, width * kBf16Bytes) || !usable(stream, bias) ||
      output->device() != bias.device())
    return invalid("bias add: buffers are missing, too small or on another device");
  return from_code(evo_b200_bf16_add_bias_inplace(output->data(), bias.data(), rows, width, raw(stream)), "bias add");
}

// ---- gated MLP ----------------------------------------------------------------------------------
// Upstream runs l1 and l2 as two projections, the gate as its own pass and l3 last (src/cuda/ops.cu
// bf16_mlp); the model runtime of this build fuses the first three into one GEMM over an interleaved
// weight prepared at load time.  This entry has no load time, so it keeps upstream's sequence and
// leaves the intermediate results in the workspace buffers where upstream leaves them.
Status bf16_mlp(const BlasLt &handle, const DeviceBuffer &input, const DeviceBuffer &l1_weight,
                const DeviceBuffer &l2_weight, const DeviceBuffer &l3_weight, const std::size_t rows,
                const std::size_t width, const std::size_t inner_width, const GatedActivation activation,
                MlpWorkspace *const workspace, DeviceBuffer *const output, const Stream &stream) {
  if (workspace == nullptr || output == nullptr) return invalid("MLP: workspace and output are required");
  DeviceBuffer *const split_k = workspace->blas.valid() ? &workspace->blas : nullptr;
  auto status = bf16_linear(handle, input, l1_weight, nullptr, rows, width, inner_width, &workspace->first, split_k,
                            stream, &workspace->up_plan);
  if (!status.ok()) return status;
  status = bf16_linear(handle, input, l2_weight, nullptr, rows, width, inner_width, &workspace->second, split_k, stream,
                       &workspace->up_plan);
  if (!status.ok()) return status;
  std::size_t elements = 0;
  if (!product(rows, inner_width, 1, &elements)) return invalid("MLP: dimensions are not representable");
  status = bf16_gated_elementwise(workspace->first, workspace->second, elements, activation, &workspace->gated, stream);
  if (!status.ok()) return status;
  return bf16_linear(handle, workspace->gated, l3_weight, nullptr, rows, inner_width, width, output, split_k, stream,
                     &workspace->down_plan);
}

}  // namespace evo::cuda
