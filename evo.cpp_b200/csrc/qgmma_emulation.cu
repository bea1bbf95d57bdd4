// Bit-exact integer emulation of the Hopper FP8 tensor-core accumulation
// that upstream's "exact" profile pins for the E4M3 Hyena projections
// (src/cuda/ops.cu:277-441, docs/software-fp8.md).  Per output element and
// per group of 32 K values:
//   E     = max(exponent(acc) if acc != 0, max over non-zero products of
//           (e_a + e_b))
//   sum   = trunc(sig14(acc) >> (E - e_acc))
//           + sum_k sign * ((|s_a| * |s_b| * 128) >> (E - e_a - e_b))
//   acc   = truncate_to_13_fraction_bits(ldexp(sum, E - 13))
// and finally out = bf16(acc * output_scale).
//
// This is an integer-ALU kernel by construction (no tensor-core mapping
// reproduces the per-group alignment), so it is register-tiled instead: a
// 256-thread CTA owns a 64x64 output tile, each thread a 4x4 sub-tile, and the
// operands of one K group are staged in shared memory already unpacked into
// (exponent, signed significand) pairs so the inner loops are pure
// add/max/mul/shift.
#include "common.cuh"
#include "ops_internal.hpp"

namespace evob {
namespace {

constexpr int kTile = 64;
constexpr int kGroup = 32;
constexpr int kZeroExponent = -64;  // never wins a max against a real product

// (exponent << 16) | (signed 5-bit significand & 0xffff); zero operands carry
// kZeroExponent so they drop out of the exponent maximum and contribute
// a zero product.  Subnormal codes are normalised (src/cuda/ops.cu:310-332).
__device__ __forceinline__ std::uint32_t unpack_e4m3(const std::uint8_t code) {
  const unsigned int magnitude = code & 0x7fU;
  const unsigned int exponent_field = (magnitude >> 3U) & 0x0fU;
  const unsigned int mantissa = magnitude & 0x07U;
  int exponent;
  int significand;
  if (exponent_field == 0U) {
    if (mantissa == 0U)
      return static_cast<std::uint32_t>(kZeroExponent) << 16U;
    const int leading = 31 - __clz(static_cast<int>(mantissa));
    exponent = -9 + leading;
    significand = static_cast<int>(mantissa << (3 - leading));
  } else {
    exponent = static_cast<int>(exponent_field) - 7;
    significand = static_cast<int>(8U + mantissa);
  }
  if ((code & 0x80U) != 0U) significand = -significand;
  return (static_cast<std::uint32_t>(exponent) << 16U) |
         (static_cast<std::uint32_t>(significand) & 0xffffU);
}

__device__ __forceinline__ int exponent_of(const std::uint32_t packed) {
  return static_cast<int>(packed) >> 16;
}
__device__ __forceinline__ int significand_of(const std::uint32_t packed) {
  return static_cast<int>(static_cast<short>(packed & 0xffffU));
}

__global__ void __launch_bounds__(256)
qgmma_emulation_kernel(const std::uint8_t *__restrict__ input_codes,
                       const std::uint8_t *__restrict__ weight_codes,
                       bf16 *__restrict__ output, const std::size_t rows,
                       const std::size_t in_features,
                       const std::size_t out_features,
                       const float output_scale) {
  // [k][row] / [k][column] so a thread's four rows (columns) are one
  // 128-bit shared-memory load.
  __shared__ __align__(16) std::uint32_t a_tile[kGroup][kTile];
  __shared__ __align__(16) std::uint32_t b_tile[kGroup][kTile];
  const unsigned int tid = threadIdx.x;
  const unsigned int ty = tid / 16;
  const unsigned int tx = tid % 16;
  const std::size_t row0 = static_cast<std::size_t>(blockIdx.y) * kTile;
  const std::size_t col0 = static_cast<std::size_t>(blockIdx.x) * kTile;

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0F;

  // Each thread stages 8 consecutive K codes of one row and one column.
  const unsigned int load_line = tid / 4;        // 0..63
  const unsigned int load_k = (tid % 4) * 8;     // 0,8,16,24
  for (std::size_t k0 = 0; k0 < in_features; k0 += kGroup) {
    {
      uint2 raw = make_uint2(0U, 0U);
      if (row0 + load_line < rows)
        raw = *reinterpret_cast<const uint2 *>(
            input_codes + (row0 + load_line) * in_features + k0 + load_k);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        a_tile[load_k + j][load_line] = unpack_e4m3(static_cast<std::uint8_t>(
            ((j < 4 ? raw.x : raw.y) >> (8 * (j & 3))) & 0xffU));
      raw = make_uint2(0U, 0U);
      if (col0 + load_line < out_features)
        raw = *reinterpret_cast<const uint2 *>(
            weight_codes + (col0 + load_line) * in_features + k0 + load_k);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        b_tile[load_k + j][load_line] = unpack_e4m3(static_cast<std::uint8_t>(
            ((j < 4 ? raw.x : raw.y) >> (8 * (j & 3))) & 0xffU));
    }
    __syncthreads();

    int maximum[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j)
        maximum[i][j] =
            acc[i][j] == 0.0F
                ? -1024
                : static_cast<int>((__float_as_uint(acc[i][j]) >> 23U) & 0xffU) -
                      127;
#pragma unroll 4
    for (int k = 0; k < kGroup; ++k) {
      const uint4 a = *reinterpret_cast<const uint4 *>(&a_tile[k][ty * 4]);
      const uint4 b = *reinterpret_cast<const uint4 *>(&b_tile[k][tx * 4]);
      const int ea[4] = {exponent_of(a.x), exponent_of(a.y), exponent_of(a.z),
                         exponent_of(a.w)};
      const int eb[4] = {exponent_of(b.x), exponent_of(b.y), exponent_of(b.z),
                         exponent_of(b.w)};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
          maximum[i][j] = max(maximum[i][j], ea[i] + eb[j]);
    }

    int sum[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        int aligned = 0;
        if (acc[i][j] != 0.0F) {
          const std::uint32_t bits = __float_as_uint(acc[i][j]);
          const int exponent = static_cast<int>((bits >> 23U) & 0xffU) - 127;
          std::uint32_t significand = ((bits & 0x7fffffU) | 0x800000U) >> 10U;
          const int shift = maximum[i][j] - exponent;
          significand = shift > 31 ? 0U : significand >> shift;
          aligned = (bits & 0x80000000U) == 0U
                        ? static_cast<int>(significand)
                        : -static_cast<int>(significand);
        }
        sum[i][j] = aligned;
      }
#pragma unroll 4
    for (int k = 0; k < kGroup; ++k) {
      const uint4 a = *reinterpret_cast<const uint4 *>(&a_tile[k][ty * 4]);
      const uint4 b = *reinterpret_cast<const uint4 *>(&b_tile[k][tx * 4]);
      const std::uint32_t ap[4] = {a.x, a.y, a.z, a.w};
      const std::uint32_t bp[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int product = significand_of(ap[i]) * significand_of(bp[j]);
          const int sign = product >> 31;
          const unsigned int magnitude =
              static_cast<unsigned int>((product ^ sign) - sign) << 7U;
          const int shift =
              min(maximum[i][j] - exponent_of(ap[i]) - exponent_of(bp[j]), 31);
          const int shifted = static_cast<int>(magnitude >> shift);
          sum[i][j] += (shifted ^ sign) - sign;
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j)
        acc[i][j] =
            sum[i][j] == 0
                ? 0.0F
                : __uint_as_float(
                      __float_as_uint(ldexpf(static_cast<float>(sum[i][j]),
                                             maximum[i][j] - 13)) &
                      0xfffffc00U);
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const std::size_t row = row0 + ty * 4 + i;
    if (row >= rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const std::size_t column = col0 + tx * 4 + j;
      if (column < out_features)
        output[row * out_features + column] =
            f2bf(acc[i][j] * output_scale);
    }
  }
}

// One or two rows (cached decode): four lanes share one output column and
// split each 32-product group between them (8 weight bytes per lane, so a
// quad reads the group's 32 bytes as one sector).  The group maximum and the
// aligned integer sum are combined across the quad with shuffles - integer
// addition is exact, so the result is the one accumulator chain of the tiled
// kernel above, bit for bit.  Unpacked activation rows sit in shared memory.
constexpr int kRowKernelThreads = 128;
constexpr int kQuad = 4;

template <int kRows>
__global__ void __launch_bounds__(kRowKernelThreads)
qgmma_emulation_rows_kernel(const std::uint8_t *__restrict__ input_codes,
                            const std::uint8_t *__restrict__ weight_codes,
                            bf16 *__restrict__ output, const std::size_t in_features,
                            const std::size_t out_features, const float output_scale) {
  extern __shared__ std::uint32_t x_unpacked[];  // [kRows][in_features]
  __shared__ std::uint32_t unpacked_code[256];   // unpack_e4m3 of every code: one load per weight
  for (int i = threadIdx.x; i < 256; i += kRowKernelThreads)
    unpacked_code[i] = unpack_e4m3(static_cast<std::uint8_t>(i));
  for (std::size_t i = threadIdx.x; i < kRows * in_features; i += kRowKernelThreads)
    x_unpacked[i] = unpack_e4m3(input_codes[i]);
  __syncthreads();
  const int quad_lane = threadIdx.x % kQuad;
  const std::size_t column =
      static_cast<std::size_t>(blockIdx.x) * (kRowKernelThreads / kQuad) + threadIdx.x / kQuad;
  // whole quads are in or out together, so the shuffles below stay converged
  const bool active = column < out_features;
  const uint2 *const weights = reinterpret_cast<const uint2 *>(
      weight_codes + (active ? column : 0) * in_features + quad_lane * (kGroup / kQuad));
  float acc[kRows];
#pragma unroll
  for (int r = 0; r < kRows; ++r) acc[r] = 0.0F;
  const std::size_t groups = in_features / kGroup;
  uint2 next = __ldcs(weights);
  for (std::size_t group = 0; group < groups; ++group) {
    const uint2 raw = next;
    if (group + 1 < groups) next = __ldcs(weights + (group + 1) * (kGroup / 8));
    std::uint32_t w[kGroup / kQuad];
#pragma unroll
    for (int k = 0; k < kGroup / kQuad; ++k)
      w[k] = unpacked_code[((k < 4 ? raw.x : raw.y) >> (8 * (k % 4))) & 0xffU];
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      const std::uint32_t *const x =
          x_unpacked + r * in_features + group * kGroup + quad_lane * (kGroup / kQuad);
      int maximum = acc[r] == 0.0F
                        ? -1024
                        : static_cast<int>((__float_as_uint(acc[r]) >> 23U) & 0xffU) - 127;
#pragma unroll
      for (int k = 0; k < kGroup / kQuad; ++k) maximum = max(maximum, exponent_of(x[k]) + exponent_of(w[k]));
      maximum = max(maximum, __shfl_xor_sync(0xffffffffU, maximum, 1));
      maximum = max(maximum, __shfl_xor_sync(0xffffffffU, maximum, 2));
      int sum = 0;
      if (quad_lane == 0 && acc[r] != 0.0F) {
        const std::uint32_t bits = __float_as_uint(acc[r]);
        const int exponent = static_cast<int>((bits >> 23U) & 0xffU) - 127;
        std::uint32_t significand = ((bits & 0x7fffffU) | 0x800000U) >> 10U;
        const int shift = maximum - exponent;
        significand = shift > 31 ? 0U : significand >> shift;
        sum = (bits & 0x80000000U) == 0U ? static_cast<int>(significand)
                                         : -static_cast<int>(significand);
      }
#pragma unroll
      for (int k = 0; k < kGroup / kQuad; ++k) {
        const int product = significand_of(x[k]) * significand_of(w[k]);
        const int sign = product >> 31;
        const unsigned int magnitude = static_cast<unsigned int>((product ^ sign) - sign) << 7U;
        const int shift = min(maximum - exponent_of(x[k]) - exponent_of(w[k]), 31);
        sum += (static_cast<int>(magnitude >> shift) ^ sign) - sign;
      }
      sum += __shfl_xor_sync(0xffffffffU, sum, 1);
      sum += __shfl_xor_sync(0xffffffffU, sum, 2);
      acc[r] = sum == 0 ? 0.0F
                        : __uint_as_float(
                              __float_as_uint(ldexpf(static_cast<float>(sum), maximum - 13)) &
                              0xfffffc00U);
    }
  }
  if (active && quad_lane == 0) {
#pragma unroll
    for (int r = 0; r < kRows; ++r)
      output[r * out_features + column] = f2bf(acc[r] * output_scale);
  }
}

}  // namespace

int e4m3_emulated_gemm(const void *input_codes, const void *weight_codes,
                       const std::size_t rows, const std::size_t in_features,
                       const std::size_t out_features,
                       const float output_scale, void *output,
                       cudaStream_t stream) {
  if (input_codes == nullptr || weight_codes == nullptr || output == nullptr ||
      in_features == 0 || out_features == 0 || in_features % kGroup != 0 ||
      !isfinite(output_scale))
    return fail(kInvalidArgument,
                "software E4M3 linear needs K to be a multiple of 32 and "
                "valid buffers");
  if (rows == 0) return kOk;
  if ((reinterpret_cast<std::uintptr_t>(input_codes) & 7U) != 0 ||
      (reinterpret_cast<std::uintptr_t>(weight_codes) & 7U) != 0)
    return fail(kInvalidArgument,
                "software E4M3 linear code buffers must be 8-byte aligned");
  if (rows <= 2 && in_features * rows * sizeof(std::uint32_t) <= 96 * 1024 &&
      (reinterpret_cast<std::uintptr_t>(weight_codes) & 15U) == 0) {
    const std::size_t smem = in_features * rows * sizeof(std::uint32_t);
    const unsigned int blocks = ceil_div_u(out_features, kRowKernelThreads / kQuad);
    auto *const kernel = rows == 1 ? qgmma_emulation_rows_kernel<1> : qgmma_emulation_rows_kernel<2>;
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
      return fail(kCuda, "cannot raise the emulation kernel shared-memory limit");
    kernel<<<blocks, kRowKernelThreads, smem, stream>>>(
        static_cast<const std::uint8_t *>(input_codes),
        static_cast<const std::uint8_t *>(weight_codes), static_cast<bf16 *>(output),
        in_features, out_features, output_scale);
    return check_launch("software E4M3 QGMMA emulation row kernel");
  }
  const dim3 grid(ceil_div_u(out_features, kTile), ceil_div_u(rows, kTile));
  if (grid.y > 65535)
    return fail(kInvalidArgument, "software E4M3 linear has too many rows");
  qgmma_emulation_kernel<<<grid, 256, 0, stream>>>(
      static_cast<const std::uint8_t *>(input_codes),
      static_cast<const std::uint8_t *>(weight_codes),
      static_cast<bf16 *>(output), rows, in_features, out_features,
      output_scale);
  return check_launch("software E4M3 QGMMA emulation kernel");
}

}  // namespace evob
