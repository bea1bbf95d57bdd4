// Host-side E4M3FN codec with upstream's contract (include/evo/fp8.hpp:9-18,
// src/fp8.cpp:26-77): round-to-nearest-even, NVIDIA satfinite overflow (every
// finite or infinite magnitude >= 448 encodes as 448), NaN -> 0x7f with the
// sign kept.  Upstream searches the 127 positive codes; this version rounds
// the float's own bit pattern, which gives the same code for every input.
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>

#include "ops_internal.hpp"

namespace evob {
namespace fp8 {

std::uint8_t encode_e4m3fn(const float value) noexcept {
  std::uint32_t bits;
  std::memcpy(&bits, &value, sizeof(bits));
  const std::uint8_t sign = static_cast<std::uint8_t>((bits >> 24U) & 0x80U);
  const std::uint32_t magnitude = bits & 0x7fffffffU;
  if (magnitude > 0x7f800000U) return sign | 0x7fU;   // NaN
  if (magnitude >= 0x43e00000U) return sign | 0x7eU;  // >= 448, infinities included
  if (magnitude >= 0x3c800000U) {
    // normal E4M3 range [2^-6, 448): keep 3 of the 23 fraction bits, ties to even;
    // a carry out of the fraction moves into the exponent field by itself
    const std::uint32_t rounded = (magnitude + 0x7ffffU + ((magnitude >> 20U) & 1U)) >> 20U;
    return sign | static_cast<std::uint8_t>(rounded - ((127U - 7U) << 3U));
  }
  // subnormal range: multiples of 2^-9; nearbyint rounds ties to even in the
  // default rounding mode, and 8 * 2^-9 is the code of the smallest normal
  float scaled;
  std::memcpy(&scaled, &magnitude, sizeof(scaled));
  return sign | static_cast<std::uint8_t>(std::nearbyint(scaled * 512.0F));
}

float decode_e4m3fn(const std::uint8_t code) noexcept {
  const unsigned magnitude = code & 0x7fU;
  const float sign = (code & 0x80U) != 0 ? -1.0F : 1.0F;
  if (magnitude == 0x7fU) return std::copysign(std::numeric_limits<float>::quiet_NaN(), sign);
  const unsigned exponent = magnitude >> 3U, fraction = magnitude & 7U;
  const float positive = exponent == 0 ? std::ldexp(static_cast<float>(fraction), -9)
                                       : std::ldexp(static_cast<float>(8U + fraction), static_cast<int>(exponent) - 10);
  return sign * positive;
}

bool valid_scale(const float scale) noexcept { return scale > 0.0F && std::isfinite(scale); }

float scaled_e4m3fn_roundtrip(const float value, const float scale) noexcept {
  if (!valid_scale(scale)) return std::numeric_limits<float>::quiet_NaN();
  return decode_e4m3fn(encode_e4m3fn(value * scale)) * (1.0F / scale);
}

}  // namespace fp8
}  // namespace evob
