// TEST INFRASTRUCTURE ONLY - flat C entry points over upstream's own CPU math
// (namespace evo::fp8 in src/fp8.cpp and namespace evo::cpu in
// src/cpu_reference.cpp), compiled unmodified from the upstream tree by
// oracle/Makefile.  Used to pin oracle/evo_oracle.cpp; never shipped.
#include <cstddef>
#include <cstdint>
#include <vector>

#include "evo/cpu_reference.hpp"
#include "evo/fp8.hpp"

#define SHIM extern "C" __attribute__((visibility("default")))

namespace {
std::vector<float> vec(const float *p, std::size_t n) { return std::vector<float>(p, p + n); }
int finish(const evo::Status &status, const std::vector<float> &result, float *out) {
  if (!status.ok()) return static_cast<int>(status.code());
  for (std::size_t i = 0; i < result.size(); ++i) out[i] = result[i];
  return 0;
}
}  // namespace

SHIM std::uint8_t ref_encode_e4m3fn(float v) { return evo::fp8::encode_e4m3fn(v); }
SHIM float ref_decode_e4m3fn(std::uint8_t b) { return evo::fp8::decode_e4m3fn(b); }
SHIM float ref_scaled_roundtrip(float v, float s) { return evo::fp8::scaled_e4m3fn_roundtrip(v, s); }

SHIM int ref_rms_norm(const float *x, std::size_t rows, std::size_t width, const float *scale,
                      float eps, float *out) {
  std::vector<float> r;
  return finish(evo::cpu::rms_norm(vec(x, rows * width), rows, width, vec(scale, width), eps, &r), r, out);
}
SHIM int ref_linear(const float *x, std::size_t rows, std::size_t in, const float *w,
                    std::size_t outf, const float *bias, float *out) {
  std::vector<float> r, b;
  if (bias) b = vec(bias, outf);
  return finish(evo::cpu::linear(vec(x, rows * in), rows, in, vec(w, in * outf), outf,
                                 bias ? &b : nullptr, &r), r, out);
}
SHIM int ref_gated_mlp(const float *x, std::size_t rows, std::size_t width, std::size_t inner,
                       const float *l1, const float *l2, const float *l3, int gelu, float *out) {
  std::vector<float> r;
  return finish(evo::cpu::gated_mlp(vec(x, rows * width), rows, width, inner,
                                    vec(l1, inner * width), vec(l2, inner * width),
                                    vec(l3, inner * width),
                                    gelu ? evo::cpu::MlpActivation::kGelu
                                         : evo::cpu::MlpActivation::kIdentity, &r), r, out);
}
SHIM int ref_fir(const float *x, std::size_t length, std::size_t channels, const float *w,
                 std::size_t taps, const float *bias, int convolution, int multiply, float *out) {
  std::vector<float> r, b;
  if (bias) b = vec(bias, channels);
  return finish(evo::cpu::causal_depthwise_fir(
                    vec(x, length * channels), length, channels, vec(w, channels * taps), taps,
                    bias ? &b : nullptr, &r,
                    convolution ? evo::cpu::FirOrientation::kCausalConvolution
                                : evo::cpu::FirOrientation::kCrossCorrelation,
                    multiply ? evo::cpu::FirBiasMode::kMultiplyInput
                             : evo::cpu::FirBiasMode::kAdd), r, out);
}
SHIM int ref_hcl_recurrence(const float *x2, const float *x1, const float *v, std::size_t length,
                            std::size_t width, const float *direct, const float *log_poles,
                            const float *residues, std::size_t modes, float *state, float *out) {
  std::vector<float> r, s = vec(state, width * modes);
  const auto status = evo::cpu::hcl_recurrence(
      vec(x2, length * width), vec(x1, length * width), vec(v, length * width), length, width,
      vec(direct, width), vec(log_poles, width * modes), vec(residues, width * modes), modes, &s, &r);
  for (std::size_t i = 0; i < s.size(); ++i) state[i] = s[i];
  return finish(status, r, out);
}
SHIM int ref_rope(float *q, float *k, std::size_t length, std::size_t heads, std::size_t head_dim,
                  const float *inv_freq, std::size_t offset, float scale) {
  const std::size_t n = length * heads * head_dim;
  std::vector<float> qv = vec(q, n), kv = vec(k, n);
  const auto status = evo::cpu::apply_rope(&qv, &kv, length, heads, head_dim,
                                           vec(inv_freq, head_dim / 2), offset, scale);
  if (!status.ok()) return static_cast<int>(status.code());
  for (std::size_t i = 0; i < n; ++i) { q[i] = qv[i]; k[i] = kv[i]; }
  return 0;
}
SHIM int ref_attention(const float *q, const float *k, const float *v, std::size_t length,
                       std::size_t heads, std::size_t head_dim, float *out) {
  const std::size_t n = length * heads * head_dim;
  std::vector<float> r;
  return finish(evo::cpu::causal_attention(vec(q, n), vec(k, n), vec(v, n), length, heads,
                                           head_dim, &r), r, out);
}
