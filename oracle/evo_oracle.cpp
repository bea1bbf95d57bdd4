// TEST INFRASTRUCTURE ONLY - CPU restatement of the numerics of the
// StripedHyena2 prefill / cached-decode hot path, used by tests/, by
// __graft_entry__.smoke() and by bench.py's CPU-baseline legs as the checker.
// The product libraries never link, load or call anything in this file.
//
// Each function restates, in plain scalar C++, what the upstream CUDA operator
// computes, one rounding at a time; citations are path:line in the upstream
// project (tcztzy/evo.cpp).  Built with -ffp-contract=off: every fused
// multiply-add below is an explicit fmaf, matching nvcc's default contraction
// of `a += b * c` in the upstream kernels.
//
// Pinning: orc_e4m3_encode is checked against the 29 known-answer pairs of
// tests/test_fp8.cpp:21-63 and against upstream's own encoder compiled from
// src/fp8.cpp; orc_qgmma_* against upstream's pure-Python statement
// (tests/test_triton_fp8.py:51-115) through committed golden vectors and
// against the test configuration of tests/test_cuda_ops.cu:433-503; the F32
// operator math against upstream's src/cpu_reference.cpp and
// tests/vectors/cpu_ops.json; GELU against the seven pinned bit patterns
// (src/cuda/ops.cu:125-139); the decode reduction tree against the known
// answer of tests/test_cuda_hyena.cu:775-826.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>

#define ORC_API extern "C" __attribute__((visibility("default")))

namespace {

using u16 = std::uint16_t;
using u8 = std::uint8_t;

inline std::uint32_t f2u(const float f) {
  std::uint32_t u;
  std::memcpy(&u, &f, 4);
  return u;
}
inline float u2f(const std::uint32_t u) {
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
inline float bf(const u16 bits) { return u2f(static_cast<std::uint32_t>(bits) << 16); }
// float -> bf16, round to nearest even (NaN kept quiet).
inline u16 to_bf16(const float value) {
  std::uint32_t bits = f2u(value);
  if ((bits & 0x7fffffffU) > 0x7f800000U) return static_cast<u16>((bits >> 16) | 0x40U);
  bits += 0x7fffU + ((bits >> 16) & 1U);
  return static_cast<u16>(bits >> 16);
}
inline float rbf(const float value) { return bf(to_bf16(value)); }

// ---- E4M3FN (src/fp8.cpp:10-65; device conversion src/cuda/ops.cu:258-260)
inline float e4m3_positive(const unsigned magnitude) {
  const unsigned e = (magnitude >> 3) & 0xfU, m = magnitude & 7U;
  return e == 0 ? std::ldexp(static_cast<float>(m), -9)
                : std::ldexp(1.0F + static_cast<float>(m) / 8.0F, static_cast<int>(e) - 7);
}
inline u8 e4m3_encode(const float value) {
  const u8 sign = std::signbit(value) ? 0x80U : 0U;
  if (std::isnan(value)) return sign | 0x7fU;
  const float magnitude = std::fabs(value);
  if (!std::isfinite(magnitude) || magnitude >= 448.0F) return sign | 0x7eU;
  // Largest code not above the magnitude, then round half to even.
  unsigned lower = 0, upper = 0x7e;
  while (upper - lower > 1) {
    const unsigned mid = (lower + upper) / 2;
    if (e4m3_positive(mid) <= magnitude) lower = mid; else upper = mid;
  }
  const float below = magnitude - e4m3_positive(lower);
  const float above = e4m3_positive(upper) - magnitude;
  unsigned rounded = lower;
  if (above < below || (above == below && (upper & 1U) == 0U)) rounded = upper;
  return static_cast<u8>(sign | rounded);
}
inline float e4m3_decode(const u8 code) {
  const unsigned magnitude = code & 0x7fU;
  if (magnitude == 0x7fU) return std::numeric_limits<float>::quiet_NaN();
  const float value = e4m3_positive(magnitude);
  return (code & 0x80U) ? -value : value;
}

// ---- QGMMA emulation (src/cuda/ops.cu:277-441; tests/test_cuda_ops.cu:119-187)
inline int exponent_of(const float value) {
  return static_cast<int>((f2u(std::fabs(value)) >> 23) & 0xffU) - 127;
}
inline std::int32_t align(const float value, const int operand_exponent,
                          const int maximum_exponent, const bool denormalized_product) {
  if (value == 0.0F) return 0;
  const std::uint32_t bits = f2u(value);
  const std::uint32_t magnitude = bits & 0x7fffffffU;
  std::uint32_t significand = (magnitude & 0x7fffffU) | 0x800000U;
  if (denormalized_product) {
    const int normalized = static_cast<int>((magnitude >> 23) & 0xffU) - 127;
    significand <<= static_cast<unsigned>(normalized - operand_exponent);
  }
  significand >>= 10;
  const int shift = maximum_exponent - operand_exponent;
  if (shift > 31) significand = 0;
  else if (shift > 0) significand >>= static_cast<unsigned>(shift);
  const auto aligned = static_cast<std::int32_t>(significand);
  return (bits & 0x80000000U) ? -aligned : aligned;
}
float qgmma_dot(const float *left, const float *right, const std::size_t inner) {
  float accumulator = 0.0F;
  for (std::size_t start = 0; start < inner; start += 32) {
    int maximum = accumulator == 0.0F ? -1024 : exponent_of(accumulator);
    for (std::size_t i = 0; i < 32; ++i) {
      const float a = left[start + i], b = right[start + i];
      if (a != 0.0F && b != 0.0F) maximum = std::max(maximum, exponent_of(a) + exponent_of(b));
    }
    std::int32_t sum = accumulator == 0.0F
                           ? 0
                           : align(accumulator, exponent_of(accumulator), maximum, false);
    for (std::size_t i = 0; i < 32; ++i) {
      const float a = left[start + i], b = right[start + i];
      if (a != 0.0F && b != 0.0F)
        sum += align(a * b, exponent_of(a) + exponent_of(b), maximum, true);
    }
    accumulator = sum == 0 ? 0.0F
                           : u2f(f2u(std::ldexp(static_cast<float>(sum), maximum - 13)) &
                                 0xfffffc00U);
  }
  return accumulator;
}

// ---- GELU (src/cuda/ops.cu:115-143)
inline u16 gelu_bits(const u16 input) {
  switch (input) {
    case 0xc049: return 0xbb2d;
    case 0xc081: return 0xb8eb;
    case 0xc089: return 0xb827;
    case 0xc092: return 0xb742;
    case 0xc0a0: return 0xb5c8;
    case 0xc0a8: return 0xb4fc;
    case 0xc0ab: return 0xb4ab;
    default: break;
  }
  const float value = bf(input);
  return to_bf16(value * 0.5F * (1.0F + std::erf(value * 0.70710678118654752440F)));
}

inline float filter_at(const void *filter, const int is_f32, const std::size_t index) {
  return is_f32 ? static_cast<const float *>(filter)[index]
                : bf(static_cast<const u16 *>(filter)[index]);
}

}  // namespace

ORC_API u8 orc_e4m3_encode(const float value) { return e4m3_encode(value); }
ORC_API float orc_e4m3_decode(const u8 code) { return e4m3_decode(code); }

// software_lowp_kernel / _codes_kernel (src/cuda/ops.cu:232-262)
ORC_API void orc_quantize_bf16(const u16 *input, const std::size_t elements,
                               const float scale, u8 *codes, float *dequantized) {
  const float inverse = 1.0F / scale;
  for (std::size_t i = 0; i < elements; ++i) {
    const u8 code = e4m3_encode(bf(input[i]) * scale);
    if (codes) codes[i] = code;
    if (dequantized) dequantized[i] = e4m3_decode(code) * inverse;
  }
}
ORC_API void orc_quantize_f32(const float *input, const std::size_t elements,
                              const float scale, u8 *codes) {
  for (std::size_t i = 0; i < elements; ++i) codes[i] = e4m3_encode(input[i] * scale);
}

// software_e4m3_h100_linear on codes (src/cuda/ops.cu:353-441)
ORC_API void orc_qgmma_codes(const u8 *input_codes, const u8 *weight_codes,
                             const std::size_t rows, const std::size_t inner,
                             const std::size_t columns, const float output_scale,
                             u16 *output) {
  std::vector<float> left(rows * inner), right(columns * inner);
  for (std::size_t i = 0; i < left.size(); ++i) left[i] = e4m3_decode(input_codes[i]);
  for (std::size_t i = 0; i < right.size(); ++i) right[i] = e4m3_decode(weight_codes[i]);
  for (std::size_t r = 0; r < rows; ++r)
    for (std::size_t c = 0; c < columns; ++c)
      output[r * columns + c] =
          to_bf16(qgmma_dot(&left[r * inner], &right[c * inner], inner) * output_scale);
}
// quantise + emulate (src/cuda/ops.cu:916-1006)
ORC_API void orc_qgmma_linear(const u16 *input, const u8 *weight_codes,
                              const std::size_t rows, const std::size_t inner,
                              const std::size_t columns, const float input_scale,
                              const float output_scale, u16 *output) {
  std::vector<u8> codes(rows * inner);
  orc_quantize_bf16(input, codes.size(), input_scale, codes.data(), nullptr);
  orc_qgmma_codes(codes.data(), weight_codes, rows, inner, columns, output_scale, output);
}
// Exact-product reference for the tensor-core profile: true E4M3 products
// summed in double, one rounding.  (No upstream counterpart: tolerance oracle.)
ORC_API void orc_e4m3_exact_linear(const u16 *input, const u8 *weight_codes,
                                   const std::size_t rows, const std::size_t inner,
                                   const std::size_t columns, const float input_scale,
                                   const float output_scale, u16 *output) {
  std::vector<float> left(rows * inner), right(columns * inner);
  for (std::size_t i = 0; i < left.size(); ++i)
    left[i] = e4m3_decode(e4m3_encode(bf(input[i]) * input_scale));
  for (std::size_t i = 0; i < right.size(); ++i) right[i] = e4m3_decode(weight_codes[i]);
  for (std::size_t r = 0; r < rows; ++r)
    for (std::size_t c = 0; c < columns; ++c) {
      double sum = 0.0;
      for (std::size_t k = 0; k < inner; ++k)
        sum += static_cast<double>(left[r * inner + k]) * right[c * inner + k];
      output[r * columns + c] = to_bf16(static_cast<float>(sum) * output_scale);
    }
}

// rms_norm_kernel (src/cuda/ops.cu:72-113): 256 strided lanes, shuffle-down
// trees, BF16 chain norm -> *rsqrt(width) -> +eps, then x/den and *scale.
ORC_API void orc_rms_norm(const u16 *input, const float *scale, const std::size_t rows,
                          const std::size_t width, const float epsilon, u16 *output) {
  for (std::size_t row = 0; row < rows; ++row) {
    float lanes[256];
    for (int t = 0; t < 256; ++t) {
      float sum = 0.0F;
      for (std::size_t c = t; c < width; c += 256) {
        const float v = bf(input[row * width + c]);
        sum = std::fmaf(v, v, sum);
      }
      lanes[t] = sum;
    }
    float partial[32] = {};
    for (int w = 0; w < 8; ++w) {
      float v[32];
      for (int l = 0; l < 32; ++l) v[l] = lanes[w * 32 + l];
      for (int offset = 16; offset > 0; offset /= 2)
        for (int l = 0; l < 32; ++l) v[l] = v[l] + (l + offset < 32 ? v[l + offset] : v[l]);
      partial[w] = v[0];
    }
    // The upstream shuffle-down reads lanes >= 32-offset from themselves; only
    // lane 0 is consumed and it never depends on those lanes.
    float v[32];
    for (int l = 0; l < 32; ++l) v[l] = l < 8 ? partial[l] : 0.0F;
    for (int offset = 16; offset > 0; offset /= 2)
      for (int l = 0; l + offset < 32; ++l) v[l] = v[l] + v[l + offset];
    const float norm = rbf(std::sqrt(v[0]));
    const float scaled = rbf(norm * (1.0F / std::sqrt(static_cast<float>(width))));
    const float denominator = rbf(scaled + epsilon);
    for (std::size_t c = 0; c < width; ++c) {
      const float normalized = rbf(bf(input[row * width + c]) / denominator);
      output[row * width + c] = to_bf16(normalized * rbf(scale[c]));
    }
  }
}

// bf16_linear (src/cuda/ops.cu:535-748) + add_bias / add kernels (175-198):
// F32 accumulation (here: double, rounded once), bias_mode 1 fused / 2 separate.
ORC_API void orc_linear_bf16(const u16 *input, const u16 *weight, const u16 *bias,
                             const u16 *residual, const std::size_t rows,
                             const std::size_t inner, const std::size_t columns,
                             const int bias_mode, u16 *output) {
  for (std::size_t r = 0; r < rows; ++r)
    for (std::size_t c = 0; c < columns; ++c) {
      double sum = 0.0;
      for (std::size_t k = 0; k < inner; ++k)
        sum += static_cast<double>(bf(input[r * inner + k])) * bf(weight[c * inner + k]);
      float value = static_cast<float>(sum);
      if (bias && bias_mode == 1) value += bf(bias[c]);
      value = rbf(value);
      if (bias && bias_mode == 2) value = rbf(value + bf(bias[c]));
      if (residual) value = rbf(value + bf(residual[r * columns + c]));
      output[r * columns + c] = to_bf16(value);
    }
}

ORC_API void orc_gelu(const u16 *input, const std::size_t n, u16 *output) {
  for (std::size_t i = 0; i < n; ++i) output[i] = gelu_bits(input[i]);
}
// gated_kernel (src/cuda/ops.cu:145-162)
ORC_API void orc_gate(const u16 *first, const u16 *second, const std::size_t n,
                      const int gelu, u16 *output) {
  for (std::size_t i = 0; i < n; ++i) {
    const float a = gelu ? bf(gelu_bits(first[i])) : bf(first[i]);
    output[i] = to_bf16(a * bf(second[i]));
  }
}
ORC_API void orc_add(const u16 *a, const u16 *b, const std::size_t n, u16 *output) {
  for (std::size_t i = 0; i < n; ++i) output[i] = to_bf16(bf(a[i]) + bf(b[i]));
}

// split_projection_kernel (src/cuda/hyena.cu:194-208)
ORC_API void orc_split(const u16 *projection, const std::size_t elements, u16 *x2,
                       u16 *x1, u16 *value) {
  for (std::size_t i = 0; i < elements; ++i) {
    x2[i] = projection[3 * i];
    x1[i] = projection[3 * i + 1];
    value[i] = projection[3 * i + 2];
  }
}

// fir_prefill_kernel (src/cuda/hyena.cu:243-272): F32 serial FMA over taps
// 0..k-1, optional +bias or +bias*x, one BF16 rounding.
ORC_API void orc_fir_prefill(const u16 *input, const void *filter, const int filter_is_f32,
                             const u16 *bias, const int multiply_bias,
                             const std::size_t length, const std::size_t channels,
                             const std::size_t groups, const std::size_t taps,
                             const int cross_correlation, u16 *output, float *cache) {
  const std::size_t per_group = channels / groups;
  for (std::size_t t = 0; t < length; ++t)
    for (std::size_t c = 0; c < channels; ++c) {
      float total = 0.0F;
      for (std::size_t tap = 0; tap < taps; ++tap) {
        const std::size_t delay = cross_correlation ? taps - 1 - tap : tap;
        if (t >= delay)
          total = std::fmaf(bf(input[(t - delay) * channels + c]),
                            filter_at(filter, filter_is_f32, (c / per_group) * taps + tap),
                            total);
      }
      if (bias) {
        const float b = bf(bias[c]);
        total = multiply_bias ? std::fmaf(b, bf(input[t * channels + c]), total) : total + b;
      }
      output[t * channels + c] = to_bf16(total);
    }
  if (cache && taps > 1) {  // fill_fir_cache_kernel (src/cuda/hyena.cu:210-232)
    const std::size_t size = taps - 1, valid = std::min(length, size), lead = size - valid;
    for (std::size_t c = 0; c < channels; ++c)
      for (std::size_t s = 0; s < size; ++s)
        cache[c * size + s] =
            s < lead ? 0.0F : bf(input[(length - valid + s - lead) * channels + c]);
  }
}

// fir_continue_kernel / fir_decode_kernel + advance_fir_cache_kernel
// (src/cuda/hyena.cu:275-416): separately rounded products into 32 strided
// lanes, 16/8/4/2/1 tree, then current tap, then bias.
ORC_API void orc_fir_step(const u16 *input, const void *filter, const int filter_is_f32,
                          const u16 *bias, const int multiply_bias,
                          const std::size_t length, const std::size_t channels,
                          const std::size_t groups, const std::size_t taps,
                          const int cross_correlation, float *cache,
                          const std::size_t cached, u16 *output) {
  const std::size_t per_group = channels / groups, size = taps - 1;
  for (std::size_t t = 0; t < length; ++t)
    for (std::size_t c = 0; c < channels; ++c) {
      const std::size_t group = c / per_group;
      const std::size_t history_total = cached + t;
      const std::size_t active = std::min(history_total, size);
      const std::size_t begin = history_total - active;
      float terms[32] = {};
      for (std::size_t a = 0; a < active; ++a) {
        const std::size_t h = begin + a;
        const float source = h < cached ? cache[c * size + size - cached + h]
                                        : bf(input[(h - cached) * channels + c]);
        const std::size_t tap = cross_correlation ? a : active - a;
        const float product = source * filter_at(filter, filter_is_f32, group * taps + tap);
        terms[a % 32] = terms[a % 32] + product;
      }
      for (int offset = 16; offset != 0; offset /= 2)
        for (int lane = 0; lane < offset; ++lane) terms[lane] = terms[lane] + terms[lane + offset];
      const float current = bf(input[t * channels + c]);
      const std::size_t current_tap = cross_correlation ? active : 0;
      float total =
          current * filter_at(filter, filter_is_f32, group * taps + current_tap) + terms[0];
      if (bias) {
        const float b = bf(bias[c]);
        total = total + (multiply_bias ? b * current : b);
      }
      output[t * channels + c] = to_bf16(total);
    }
  for (std::size_t c = 0; c < channels; ++c) {
    float *row = cache + c * size;
    if (length >= size) {
      for (std::size_t s = 0; s < size; ++s) row[s] = bf(input[(length - size + s) * channels + c]);
    } else {
      const std::size_t retained = size - length;
      for (std::size_t s = 0; s < retained; ++s) row[s] = row[s + length];
      for (std::size_t t = 0; t < length; ++t) row[retained + t] = bf(input[t * channels + c]);
    }
  }
}

// bf16_hcs_prefill / bf16_hcm_prefill_direct (src/cuda/hyena.cu:1792-1992):
// u = bf16(x1*v); y = bf16(fir(u) [+ D*u]); out = bf16(y*x2).  HCM upstream
// prefill runs this convolution through an n=2T FFT (tolerance-level equal).
ORC_API void orc_gated_fir(const u16 *x2, const u16 *x1, const u16 *value,
                           const void *filter, const int filter_is_f32, const u16 *direct,
                           const std::size_t length, const std::size_t width,
                           const std::size_t groups, const std::size_t taps,
                           const int cross_correlation, u16 *pregate, float *cache,
                           u16 *output) {
  std::vector<u16> u(length * width), y(length * width);
  for (std::size_t i = 0; i < u.size(); ++i) u[i] = to_bf16(bf(x1[i]) * bf(value[i]));
  orc_fir_prefill(u.data(), filter, filter_is_f32, direct, 1, length, width, groups, taps,
                  cross_correlation, y.data(), cache);
  for (std::size_t i = 0; i < u.size(); ++i) output[i] = to_bf16(bf(y[i]) * bf(x2[i]));
  if (pregate) std::memcpy(pregate, u.data(), u.size() * sizeof(u16));
}

// hcl_filter_kernel (src/cuda/hyena.cu:562-592): four accumulators by mode%4.
static float modal_filter(const float *log_poles, const float *residues, const std::size_t modes,
                          const std::size_t t) {
  float partial[4] = {0, 0, 0, 0};
  for (std::size_t m = 0; m < modes; ++m)
    partial[m % 4] = partial[m % 4] + residues[m] * std::exp(log_poles[m] * static_cast<float>(t));
  return ((partial[0] + partial[1]) + partial[2]) + partial[3];
}

// bf16_hcl_prefill (src/cuda/hyena.cu:1994-2124).  mode 0: FFT-path contract
// evaluated as an exact (double) causal convolution with the materialised
// filter, then the four BF16 roundings; state = sum_t exp(lp (T-1-t)) u[t].
// mode 1: recurrence continuation (src/cuda/hyena.cu:534-560), single rounding.
ORC_API void orc_hcl_prefill(const u16 *x2, const u16 *x1, const u16 *value, const u16 *direct,
                             const float *log_poles, const float *residues,
                             const std::size_t length, const std::size_t width,
                             const std::size_t modes, const int mode, float *state,
                             u16 *pregate, u16 *output) {
  std::vector<u16> u(length * width);
  for (std::size_t i = 0; i < u.size(); ++i) u[i] = to_bf16(bf(x1[i]) * bf(value[i]));
  if (pregate) std::memcpy(pregate, u.data(), u.size() * sizeof(u16));
  if (mode == 1) {
    for (std::size_t c = 0; c < width; ++c)
      for (std::size_t t = 0; t < length; ++t) {
        const float in = bf(u[t * width + c]);
        float modal = 0.0F;
        for (std::size_t m = 0; m < modes; ++m) {
          const std::size_t q = c * modes + m;
          const float updated = std::fmaf(std::exp(log_poles[q]), state[q], in);
          state[q] = updated;
          modal = std::fmaf(residues[q], updated, modal);
        }
        output[t * width + c] =
            to_bf16(bf(x2[t * width + c]) * std::fmaf(bf(direct[c]), in, modal));
      }
    return;
  }
  for (std::size_t c = 0; c < width; ++c) {
    std::vector<float> h(length);
    for (std::size_t t = 0; t < length; ++t)
      h[t] = modal_filter(log_poles + c * modes, residues + c * modes, modes, t);
    for (std::size_t t = 0; t < length; ++t) {
      double conv = 0.0;
      for (std::size_t s = 0; s <= t; ++s)
        conv += static_cast<double>(h[t - s]) * bf(u[s * width + c]);
      const float y = rbf(static_cast<float>(conv));
      const float d = rbf(bf(u[t * width + c]) * bf(direct[c]));
      const float mixed = rbf(y + d);
      output[t * width + c] = to_bf16(mixed * bf(x2[t * width + c]));
    }
    if (state)
      for (std::size_t m = 0; m < modes; ++m) {
        double sum = 0.0;
        for (std::size_t t = 0; t < length; ++t)
          sum += std::exp(static_cast<double>(log_poles[c * modes + m]) *
                          static_cast<double>(length - 1 - t)) *
                 bf(u[t * width + c]);
        state[c * modes + m] = static_cast<float>(sum);
      }
  }
}

// hcl_decode_kernel (src/cuda/hyena.cu:718-761)
ORC_API void orc_hcl_decode(const u16 *x2, const u16 *x1, const u16 *value, const u16 *direct,
                            const float *log_poles, const float *residues,
                            const std::size_t width, const std::size_t modes, float *state,
                            u16 *pregate, u16 *output) {
  for (std::size_t c = 0; c < width; ++c) {
    const u16 gated_bits = to_bf16(bf(x1[c]) * bf(value[c]));
    if (pregate) pregate[c] = gated_bits;
    const float gated = bf(gated_bits);
    float terms[32] = {};
    for (std::size_t m = 0; m < modes; ++m) {
      const std::size_t q = c * modes + m;
      const float decayed = std::exp(log_poles[q]) * state[q];
      const float updated = decayed + gated;
      state[q] = updated;
      terms[m] = residues[q] * updated;
    }
    for (int offset = 16; offset != 0; offset /= 2)
      for (int lane = 0; lane < 32 - offset; ++lane) terms[lane] = terms[lane] + terms[lane + offset];
    const float direct_product = rbf(bf(direct[c]) * gated);
    const float mixed = terms[0] + direct_product;
    output[c] = to_bf16(bf(x2[c]) * mixed);
  }
}

// split_qkv_kernel + rope_kernel + KV append (src/cuda/attention.cu:210-281)
ORC_API void orc_split_rope_append(const u16 *qkv, const float *inverse_frequency,
                                   const std::size_t rows, const std::size_t heads,
                                   const std::size_t head_dim, const std::size_t offset,
                                   const float position_scale, const int head_major,
                                   u16 *query, u16 *key_cache, u16 *value_cache) {
  const std::size_t width = heads * head_dim, half = head_dim / 2;
  for (std::size_t t = 0; t < rows; ++t)
    for (std::size_t h = 0; h < heads; ++h) {
      const u16 *source = qkv + t * width * 3;
      const std::size_t q_at = head_major ? h * 3 * head_dim : h * head_dim;
      const std::size_t k_at = head_major ? q_at + head_dim : width + q_at;
      const std::size_t v_at = head_major ? k_at + head_dim : 2 * width + q_at;
      const std::size_t out = t * width + h * head_dim;
      const std::size_t cache = (offset + t) * width + h * head_dim;
      for (std::size_t p = 0; p < half; ++p) {
        const float position = static_cast<float>(offset + t) / position_scale;
        const float angle = position * inverse_frequency[p];
        const float sine = rbf(std::sin(angle)), cosine = rbf(std::cos(angle));
        const float q1 = bf(source[q_at + p]), q2 = bf(source[q_at + half + p]);
        query[out + p] = to_bf16(std::fmaf(q1, cosine, -(q2 * sine)));
        query[out + half + p] = to_bf16(std::fmaf(q2, cosine, q1 * sine));
        const float k1 = bf(source[k_at + p]), k2 = bf(source[k_at + half + p]);
        key_cache[cache + p] = to_bf16(std::fmaf(k1, cosine, -(k2 * sine)));
        key_cache[cache + half + p] = to_bf16(std::fmaf(k2, cosine, k1 * sine));
        value_cache[cache + p] = source[v_at + p];
        value_cache[cache + half + p] = source[v_at + half + p];
      }
    }
}

// Causal softmax(QK^T/sqrt(d))V, F32/double math, one BF16 rounding
// (contract of src/cuda/flash_attention.cu:199-441 and
// src/cuda/attention.cu:879-968; upstream tests compare at tolerance).
ORC_API void orc_causal_attention(const u16 *query, const u16 *keys, const u16 *values,
                                  const std::size_t rows, const std::size_t total,
                                  const std::size_t heads, const std::size_t head_dim,
                                  u16 *output) {
  const std::size_t width = heads * head_dim;
  const double scale = 1.0 / std::sqrt(static_cast<double>(head_dim));
  std::vector<double> scores(total);
  for (std::size_t r = 0; r < rows; ++r)
    for (std::size_t h = 0; h < heads; ++h) {
      const std::size_t visible = total - rows + r + 1;
      double maximum = -1e300;
      for (std::size_t j = 0; j < visible; ++j) {
        double dot = 0.0;
        for (std::size_t d = 0; d < head_dim; ++d)
          dot += static_cast<double>(bf(query[r * width + h * head_dim + d])) *
                 bf(keys[j * width + h * head_dim + d]);
        scores[j] = dot * scale;
        maximum = std::max(maximum, scores[j]);
      }
      double total_weight = 0.0;
      for (std::size_t j = 0; j < visible; ++j) {
        scores[j] = std::exp(scores[j] - maximum);
        total_weight += scores[j];
      }
      for (std::size_t d = 0; d < head_dim; ++d) {
        double acc = 0.0;
        for (std::size_t j = 0; j < visible; ++j)
          acc += scores[j] * bf(values[j * width + h * head_dim + d]);
        output[r * width + h * head_dim + d] = to_bf16(static_cast<float>(acc / total_weight));
      }
    }
}

// bf16_cached_cross_attention (src/cuda/attention.cu:283-784,1669-1799):
// K*scale -> BF16, scores -> BF16, masked, F32 softmax -> BF16 probabilities,
// P.V with F32 accumulation -> BF16.
ORC_API void orc_cached_attention(const u16 *query, const u16 *keys, const u16 *values,
                                  const std::size_t rows, const std::size_t total,
                                  const std::size_t heads, const std::size_t head_dim,
                                  u16 *output) {
  const std::size_t width = heads * head_dim;
  const float scale = 1.0F / std::sqrt(static_cast<float>(head_dim));
  std::vector<float> scores(total);
  for (std::size_t r = 0; r < rows; ++r)
    for (std::size_t h = 0; h < heads; ++h) {
      const std::size_t visible = total - rows + r + 1;
      float maximum = -std::numeric_limits<float>::infinity();
      for (std::size_t j = 0; j < visible; ++j) {
        float dot = 0.0F;
        for (std::size_t d = 0; d < head_dim; ++d)
          dot = std::fmaf(bf(query[r * width + h * head_dim + d]),
                          rbf(bf(keys[j * width + h * head_dim + d]) * scale), dot);
        scores[j] = rbf(dot);
        maximum = std::max(maximum, scores[j]);
      }
      float sum = 0.0F;
      for (std::size_t j = 0; j < visible; ++j) {
        scores[j] = std::exp(scores[j] - maximum);
        sum += scores[j];
      }
      for (std::size_t d = 0; d < head_dim; ++d) {
        float acc = 0.0F;
        for (std::size_t j = 0; j < visible; ++j)
          acc = std::fmaf(rbf(scores[j] / sum), bf(values[j * width + h * head_dim + d]), acc);
        output[r * width + h * head_dim + d] = to_bf16(acc);
      }
    }
}

ORC_API void orc_embedding(const std::uint32_t *tokens, const u16 *table,
                           const std::size_t rows, const std::size_t width, u16 *output) {
  for (std::size_t r = 0; r < rows; ++r)
    std::memcpy(output + r * width, table + static_cast<std::size_t>(tokens[r]) * width,
                width * sizeof(u16));
}
