// Shared device/host helpers for the sm_100a StripedHyena2 hot path.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <string>

namespace evob {

// Status codes shared with the public C ABI (same numeric values as
// evo_status in include/evo/evo.h).
enum : int {
  kOk = 0,
  kInvalidArgument = 2,
  kIo = 3,
  kModelFormat = 4,
  kUnsupported = 5,
  kCuda = 6,
  kInternal = 70,
};

// Thread-local error text for the operator-level C ABI.
void set_error(int code, const std::string &message);
const char *last_error();
int fail(int code, const std::string &message);
int check_launch(const char *what);

using bf16 = __nv_bfloat16;

__host__ __device__ __forceinline__ unsigned int ceil_div_u(
    const std::size_t a, const std::size_t b) {
  return static_cast<unsigned int>((a + b - 1) / b);
}

__device__ __forceinline__ float bf2f(const bf16 v) {
  return __bfloat162float(v);
}
__device__ __forceinline__ bf16 f2bf(const float v) {
  return __float2bfloat16_rn(v);
}
// Round an F32 value to BF16 precision and widen it again.
__device__ __forceinline__ float rbf(const float v) {
  // one instruction: the packed convert puts bf16(v) in the upper half and
  // bf16(+0) in the lower half, which is the F32 bit pattern of the result
  unsigned int bits;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(bits) : "f"(v), "f"(0.0F));
  return __uint_as_float(bits);
}
__device__ __forceinline__ float bits2f_bf16(const unsigned short bits) {
  return __uint_as_float(static_cast<unsigned int>(bits) << 16U);
}

// 8 BF16 values in one 128-bit register quad.
struct alignas(16) Bf16x8 {
  uint4 raw;
  __device__ __forceinline__ float get(const int i) const {
    const unsigned int word = (&raw.x)[i >> 1];
    return __uint_as_float((i & 1) ? (word & 0xffff0000U) : (word << 16U));
  }
};

__device__ __forceinline__ unsigned int pack_bf16x2(const float lo,
                                                    const float hi) {
  const unsigned int l = __bfloat16_as_ushort(__float2bfloat16_rn(lo));
  const unsigned int h = __bfloat16_as_ushort(__float2bfloat16_rn(hi));
  return l | (h << 16U);
}

constexpr int kSmCount = 148;

}  // namespace evob
