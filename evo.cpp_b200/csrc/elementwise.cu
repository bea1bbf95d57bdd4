// Element-wise and row-wise kernels of the StripedHyena2 block graph:
// E4M3 quantisation, RMSNorm (optionally emitting E4M3 codes in the same
// pass), GELU, gating, residual / bias adds, embedding gather and the
// interleaved-triple split.  All are HBM-bound; every kernel moves 128-bit
// vectors where the shape allows and sizes its grid in SM multiples.
//
// Numerics follow the upstream CUDA operators one rounding at a time
// (src/cuda/ops.cu:72-198, 232-275; src/cuda/hyena.cu:194-208;
// src/cuda/model.cu:269-284).
#include <cuda_fp8.h>

#include <algorithm>

#include "common.cuh"
#include "ops_internal.hpp"

namespace evob {
namespace {

constexpr int kThreads = 256;

__host__ unsigned int grid_for(const std::size_t work_items,
                               const int per_block = kThreads) {
  const std::size_t blocks = (work_items + per_block - 1) / per_block;
  const std::size_t cap = static_cast<std::size_t>(kSmCount) * 16;
  return static_cast<unsigned int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

__device__ __forceinline__ std::uint8_t e4m3_code(const float scaled) {
  // RNE with saturate-to-finite, the conversion upstream uses
  // (src/cuda/ops.cu:258-260).
  return static_cast<std::uint8_t>(
      __nv_cvt_float_to_fp8(scaled, __NV_SATFINITE, __NV_E4M3));
}

__device__ __forceinline__ float e4m3_value(const std::uint8_t code) {
  const __half_raw half = __nv_cvt_fp8_to_halfraw(code, __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half *>(&half));
}

// ---------------------------------------------------------------- quantise
template <typename In>
__global__ void quantize_kernel(const In *__restrict__ input,
                                std::uint8_t *__restrict__ codes,
                                float *__restrict__ dequantized,
                                const std::size_t elements, const float scale) {
  const float inverse = __frcp_rn(scale);
  const std::size_t stride = static_cast<std::size_t>(blockDim.x) * gridDim.x;
  for (std::size_t i = static_cast<std::size_t>(blockIdx.x) * blockDim.x +
                       threadIdx.x;
       i < elements; i += stride) {
    float value;
    if constexpr (sizeof(In) == 2) {
      value = bf2f(input[i]);
    } else {
      value = input[i];
    }
    const std::uint8_t code = e4m3_code(value * scale);
    if (codes != nullptr) codes[i] = code;
    if (dequantized != nullptr) dequantized[i] = e4m3_value(code) * inverse;
  }
}

// 16 BF16 values -> 16 codes per thread per step (2x128-bit in, 128-bit out).
__global__ void quantize_bf16_vec_kernel(const uint4 *__restrict__ input,
                                         uint4 *__restrict__ codes,
                                         const std::size_t vectors,
                                         const float scale) {
  const std::size_t stride = static_cast<std::size_t>(blockDim.x) * gridDim.x;
  for (std::size_t i = static_cast<std::size_t>(blockIdx.x) * blockDim.x +
                       threadIdx.x;
       i < vectors; i += stride) {
    Bf16x8 a, b;
    a.raw = input[2 * i];
    b.raw = input[2 * i + 1];
    unsigned int out[4];
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      unsigned int word = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int k = w * 4 + j;
        const float v = k < 8 ? a.get(k) : b.get(k - 8);
        word |= static_cast<unsigned int>(e4m3_code(v * scale)) << (8 * j);
      }
      out[w] = word;
    }
    codes[i] = make_uint4(out[0], out[1], out[2], out[3]);
  }
}

// ---- per-row dynamic quantisation (FP8 FFN profile)
// codes[r, :] = E4M3(x[r, :] * q_r) with q_r = 448 / max|x[r, :]|, and
// row_scale[r] = 1 / q_r for the consuming GEMM's epilogue.  Persistent blocks
// walk rows; a row is copied into shared memory once (cp.async, the next row in
// flight while the current one is reduced and converted), so HBM sees 2 bytes
// in and 1 byte out per element.  The magnitude maximum is taken on the packed
// bit patterns (for BF16 magnitudes, integer order is value order).
__global__ void __launch_bounds__(kThreads)
quantize_rows_kernel(const bf16 *__restrict__ input, std::uint8_t *__restrict__ codes,
                     float *__restrict__ row_scale, const std::size_t rows, const std::size_t width) {
  extern __shared__ __align__(16) unsigned short row_cache[];  // 2 x width BF16 values
  __shared__ unsigned int partial[kThreads / 32];
  const auto fetch = [&](const std::size_t row, unsigned short *target) {
    const uint4 *const source = reinterpret_cast<const uint4 *>(input + row * width);
    for (std::size_t v = threadIdx.x; v < width / 8; v += kThreads) {
      const std::uint32_t address =
          static_cast<std::uint32_t>(__cvta_generic_to_shared(reinterpret_cast<uint4 *>(target) + v));
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(address), "l"(source + v) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  std::size_t row = blockIdx.x;
  if (row >= rows) return;
  fetch(row, row_cache);
  const int vectors = static_cast<int>(width / 8);
  for (int parity = 0; row < rows; row += gridDim.x, parity ^= 1) {
    const unsigned short *const current = row_cache + parity * width;
    const std::size_t next = row + gridDim.x;
    if (next < rows) {
      fetch(next, row_cache + (parity ^ 1) * width);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    // a thread reads back exactly the 16-byte chunks it copied, so no barrier is needed before
    // the reduction; the barriers inside it order this row's reads against the next refill
    unsigned int high = 0U;
    for (int v = threadIdx.x; v < vectors; v += kThreads) {
      const uint4 raw = reinterpret_cast<const uint4 *>(current)[v];
      high = __vmaxu2(high, __vmaxu2(__vmaxu2(raw.x & 0x7fff7fffU, raw.y & 0x7fff7fffU),
                                     __vmaxu2(raw.z & 0x7fff7fffU, raw.w & 0x7fff7fffU)));
    }
    high = max(high & 0xffffU, high >> 16U);
#pragma unroll
    for (int offset = 16; offset > 0; offset /= 2) high = max(high, __shfl_xor_sync(0xffffffffU, high, offset));
    if (threadIdx.x % 32 == 0) partial[threadIdx.x / 32] = high;
    __syncthreads();
    unsigned int magnitude = 0U;
#pragma unroll
    for (int w = 0; w < kThreads / 32; ++w) magnitude = max(magnitude, partial[w]);
    magnitude = min(magnitude, 0x7f7fU);  // infinities and NaNs saturate
    const float amax = __uint_as_float(magnitude << 16U);
    const float quant = amax > 0.0F ? __fdiv_rn(448.0F, amax) : 1.0F;
    if (threadIdx.x == 0) row_scale[row] = __fdiv_rn(1.0F, quant);
    std::uint8_t *const out = codes + row * width;
    for (int v = threadIdx.x; v < vectors; v += kThreads) {
      Bf16x8 values;
      values.raw = reinterpret_cast<const uint4 *>(current)[v];
      unsigned int words[2] = {0U, 0U};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 scaled = make_float2(values.get(2 * j) * quant, values.get(2 * j + 1) * quant);
        const unsigned int two = __nv_cvt_float2_to_fp8x2(scaled, __NV_SATFINITE, __NV_E4M3);
        words[j / 2] |= two << (16 * (j % 2));
      }
      reinterpret_cast<uint2 *>(out)[v] = make_uint2(words[0], words[1]);
    }
    __syncthreads();  // partial[] and this half of the row cache are free again
  }
}

// Largest magnitude of a BF16 tensor as a bit pattern (atomicMax on the patterns;
// *result must start at zero).
__global__ void amax_bf16_kernel(const uint4 *__restrict__ input, const std::size_t vectors,
                                 unsigned int *__restrict__ result) {
  unsigned int high = 0U;
  const std::size_t stride = static_cast<std::size_t>(blockDim.x) * gridDim.x;
  for (std::size_t i = static_cast<std::size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < vectors; i += stride) {
    const uint4 raw = input[i];
    high = __vmaxu2(high, __vmaxu2(__vmaxu2(raw.x & 0x7fff7fffU, raw.y & 0x7fff7fffU),
                                   __vmaxu2(raw.z & 0x7fff7fffU, raw.w & 0x7fff7fffU)));
  }
  high = max(high & 0xffffU, high >> 16U);
#pragma unroll
  for (int offset = 16; offset > 0; offset /= 2) high = max(high, __shfl_xor_sync(0xffffffffU, high, offset));
  if (threadIdx.x % 32 == 0 && high != 0U) atomicMax(result, high);
}

// ---------------------------------------------------------------- RMSNorm
// One 256-thread block per row.  The F32 sum of squares is taken in the same
// order as upstream (thread-strided columns, shuffle-down tree, 8 warp
// partials through a second tree; src/cuda/ops.cu:72-96) so that the BF16
// rounding chain sees bit-identical sums.
// BF16 of two F32 values in one instruction: `low` in bits 0-15, `high` in bits 16-31.
__device__ __forceinline__ std::uint32_t round_pair(const float low, const float high) {
  std::uint32_t packed;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(packed) : "f"(high), "f"(low));
  return packed;
}

__device__ __forceinline__ float warp_sum_down(float value) {
#pragma unroll
  for (int offset = 16; offset > 0; offset /= 2)
    value += __shfl_down_sync(0xffffffffU, value, offset);
  return value;
}

// Packs two values that are already BF16-representable (no rounding needed).
__device__ __forceinline__ std::uint32_t pack_exact_pair(const float low, const float high) {
  return (__float_as_uint(low) >> 16U) | (__float_as_uint(high) & 0xffff0000U);
}

// Sum of squares of the cached row in the pinned order, then the BF16 chain
// down to the denominator.  Two block-wide barriers; every thread returns it.
// kWidth: the row width when it is known at compile time (the loops then unroll completely and the
// indices are constants), 0 when it is only known at run time.
template <int kWidth = 0>
__device__ __forceinline__ float row_denominator(const unsigned short *row_cache, const std::size_t width,
                                                 const float epsilon, float *partial) {
  float sum = 0.0F;
  if constexpr (kWidth != 0) {
    static_assert(kWidth % kThreads == 0, "a compile-time width is a multiple of the block size");
#pragma unroll
    for (int k = 0; k < kWidth / kThreads; ++k) {
      const float value = bits2f_bf16(row_cache[threadIdx.x + k * kThreads]);
      sum = fmaf(value, value, sum);
    }
  } else {
    const int columns = static_cast<int>(width);  // <= 24576
#pragma unroll 8
    for (int column = threadIdx.x; column < columns; column += kThreads) {
      const float value = bits2f_bf16(row_cache[column]);
      sum = fmaf(value, value, sum);
    }
  }
  sum = warp_sum_down(sum);
  const int lane = threadIdx.x % 32;
  const int warp = threadIdx.x / 32;
  if (lane == 0) partial[warp] = sum;
  __syncthreads();
  if (warp == 0) {
    float block_sum = lane < kThreads / 32 ? partial[lane] : 0.0F;
    block_sum = warp_sum_down(block_sum);
    if (lane == 0) {
      const float norm = rbf(sqrtf(block_sum));
      const float scaled = rbf(norm * rsqrtf(static_cast<float>(width)));
      partial[0] = rbf(scaled + epsilon);
    }
  }
  __syncthreads();
  return partial[0];
}

// Normalises the cached row 8 columns per thread and step (width % 8 == 0, 16-byte
// aligned pointers) and stores BF16 values and / or E4M3 codes.
template <int kWidth = 0>
__device__ __forceinline__ void store_normalized_row(const unsigned short *row_cache, const float *scale,
                                                     const std::uint32_t *scale_pairs,
                                                     const float denominator, const std::size_t width,
                                                     bf16 *out_row, std::uint8_t *codes_row,
                                                     const float quant_scale) {
  const int vectors = kWidth != 0 ? kWidth / 8 : static_cast<int>(width / 8);
  constexpr int kSteps = kWidth != 0 ? kWidth / 8 / kThreads : 2;  // full unroll when the width is known
  // bf16(x / den) == bf16(x * (1/den)) for every BF16 x and every BF16 den
  // in [1e-30, 1e30] (checked exhaustively on the host: a BF16 quotient is
  // never closer than ~2^-17 relative to a BF16 rounding boundary), so the
  // IEEE division is only kept for denominators outside that range.
  const bool by_reciprocal = denominator >= 1e-30F && denominator <= 1e30F;
  const float reciprocal = __frcp_rn(denominator);
  const auto load = [&](const int v, Bf16x8 &values, float (&scales)[8]) {
    values.raw = reinterpret_cast<const uint4 *>(row_cache)[v];
    const float4 s0 = __ldg(reinterpret_cast<const float4 *>(scale) + 2 * v);
    const float4 s1 = __ldg(reinterpret_cast<const float4 *>(scale) + 2 * v + 1);
    scales[0] = s0.x; scales[1] = s0.y; scales[2] = s0.z; scales[3] = s0.w;
    scales[4] = s1.x; scales[5] = s1.y; scales[6] = s1.z; scales[7] = s1.w;
  };
  if (by_reciprocal && codes_row == nullptr) {
    // no codes wanted: bf16(x / den) two at a time, then one packed BF16 multiply with the
    // BF16 scale pair (a product of BF16 values rounded once, as the scalar chain does)
#pragma unroll kSteps
    for (int v = threadIdx.x; v < vectors; v += kThreads) {
      Bf16x8 values;
      values.raw = reinterpret_cast<const uint4 *>(row_cache)[v];
      const uint4 pairs = reinterpret_cast<const uint4 *>(scale_pairs)[v];
      const std::uint32_t scales[4] = {pairs.x, pairs.y, pairs.z, pairs.w};
      std::uint32_t packed[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const std::uint32_t normalized =
            round_pair(values.get(2 * j) * reciprocal, values.get(2 * j + 1) * reciprocal);
        asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(packed[j]) : "r"(normalized), "r"(scales[j]));
      }
      reinterpret_cast<uint4 *>(out_row)[v] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    }
    return;
  }
  if (by_reciprocal) {
    // with codes: the same packed chain, then two E4M3 codes per conversion
#pragma unroll kSteps
    for (int v = threadIdx.x; v < vectors; v += kThreads) {
      Bf16x8 values;
      values.raw = reinterpret_cast<const uint4 *>(row_cache)[v];
      const uint4 pairs = reinterpret_cast<const uint4 *>(scale_pairs)[v];
      const std::uint32_t scales[4] = {pairs.x, pairs.y, pairs.z, pairs.w};
      std::uint32_t packed[4];
      unsigned int words[2] = {0U, 0U};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const std::uint32_t normalized =
            round_pair(values.get(2 * j) * reciprocal, values.get(2 * j + 1) * reciprocal);
        asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(packed[j]) : "r"(normalized), "r"(scales[j]));
        const float2 scaled = make_float2(__uint_as_float(packed[j] << 16U) * quant_scale,
                                          __uint_as_float(packed[j] & 0xffff0000U) * quant_scale);
        const unsigned int two = __nv_cvt_float2_to_fp8x2(scaled, __NV_SATFINITE, __NV_E4M3);  // .x in the low byte
        words[j / 2] |= two << (16 * (j % 2));
      }
      if (out_row != nullptr)
        reinterpret_cast<uint4 *>(out_row)[v] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
      reinterpret_cast<uint2 *>(codes_row)[v] = make_uint2(words[0], words[1]);
    }
    return;
  }
  for (int v = threadIdx.x; v < vectors; v += kThreads) {
    Bf16x8 values;
    float scales[8], results[8];
    load(v, values, scales);
#pragma unroll
    for (int j = 0; j < 8; ++j)
      results[j] = rbf(rbf(__fdiv_rn(values.get(j), denominator)) * rbf(scales[j]));
    if (out_row != nullptr)
      reinterpret_cast<uint4 *>(out_row)[v] =
          make_uint4(pack_exact_pair(results[0], results[1]), pack_exact_pair(results[2], results[3]),
                     pack_exact_pair(results[4], results[5]), pack_exact_pair(results[6], results[7]));
    if (codes_row != nullptr) {
      unsigned int words[2] = {0U, 0U};
#pragma unroll
      for (int j = 0; j < 8; ++j)
        words[j / 4] |= static_cast<unsigned int>(e4m3_code(results[j] * quant_scale)) << (8 * (j % 4));
      reinterpret_cast<uint2 *>(codes_row)[v] = make_uint2(words[0], words[1]);
    }
  }
}

// Generic form: one block per row, any width and alignment.
__global__ void __launch_bounds__(kThreads)
rms_norm_kernel(const bf16 *__restrict__ input, const float *__restrict__ scale,
                bf16 *__restrict__ output, std::uint8_t *__restrict__ codes,
                const std::size_t width, const float epsilon,
                const float quant_scale) {
  extern __shared__ __align__(16) unsigned short row_cache[];  // width BF16 values
  __shared__ float partial[32];
  const std::size_t row = blockIdx.x;
  const bf16 *const in = input + row * width;
  for (std::size_t column = threadIdx.x; column < width; column += kThreads)
    row_cache[column] = __bfloat16_as_ushort(in[column]);
  __syncthreads();
  const float denominator = row_denominator(row_cache, width, epsilon, partial);
  for (std::size_t column = threadIdx.x; column < width; column += kThreads) {
    const float value = bits2f_bf16(row_cache[column]);
    const float column_scale = rbf(scale[column]);
    const float normalized = rbf(__fdiv_rn(value, denominator));
    const bf16 result = f2bf(normalized * column_scale);
    if (output != nullptr) output[row * width + column] = result;
    if (codes != nullptr)
      codes[row * width + column] = e4m3_code(bf2f(result) * quant_scale);
  }
}

// A few rows (cached decode, very short prompts): one block per row, every load of the row and of the
// gains issued before anything is waited for - one trip to memory where the streaming kernel makes three
// in a row (gains, row, next row) and the generic one two.  A thread owns columns t, t + 256, ... in
// registers: exactly the terms of its partial sum in row_denominator's order, and the columns it
// normalises and stores (neighbouring threads write neighbouring columns).
template <int kPerThread>
__global__ void __launch_bounds__(kThreads)
rms_norm_few_rows_kernel(const bf16 *__restrict__ input, const float *__restrict__ scale,
                         bf16 *__restrict__ output, std::uint8_t *__restrict__ codes, const int width,
                         const float epsilon, const float quant_scale) {
  // lets a one-row projection launched with programmatic stream serialisation start (and fetch its
  // weights) under this kernel; it still waits for this grid to finish before it reads the result
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  __shared__ float partial[32];
  const std::size_t row = blockIdx.x;
  const unsigned short *const in = reinterpret_cast<const unsigned short *>(input) + row * width;
  unsigned short raw[kPerThread];
  float gain[kPerThread];
#pragma unroll
  for (int k = 0; k < kPerThread; ++k) gain[k] = __ldg(scale + threadIdx.x + k * kThreads);
  // launched with programmatic stream serialisation, the gains above were requested while the kernel
  // that writes the row may still be running; otherwise this returns at once
  asm volatile("griddepcontrol.wait;" ::: "memory");
#pragma unroll
  for (int k = 0; k < kPerThread; ++k) raw[k] = in[threadIdx.x + k * kThreads];
  float sum = 0.0F;
#pragma unroll
  for (int k = 0; k < kPerThread; ++k) {
    const float value = bits2f_bf16(raw[k]);
    sum = fmaf(value, value, sum);
  }
  // the rest of row_denominator: shuffle-down tree, the warps' sums, the three roundings
  sum = warp_sum_down(sum);
  const int lane = threadIdx.x % 32, warp = threadIdx.x / 32;
  if (lane == 0) partial[warp] = sum;
  __syncthreads();
  if (warp == 0) {
    float block_sum = lane < kThreads / 32 ? partial[lane] : 0.0F;
    block_sum = warp_sum_down(block_sum);
    if (lane == 0) {
      const float norm = rbf(sqrtf(block_sum));
      const float scaled = rbf(norm * rsqrtf(static_cast<float>(width)));
      partial[0] = rbf(scaled + epsilon);
    }
  }
  __syncthreads();
  const float denominator = partial[0];
#pragma unroll
  for (int k = 0; k < kPerThread; ++k) {
    const std::size_t column = threadIdx.x + k * kThreads;
    const bf16 result = f2bf(rbf(__fdiv_rn(bits2f_bf16(raw[k]), denominator)) * rbf(gain[k]));
    if (output != nullptr) output[row * width + column] = result;
    if (codes != nullptr) codes[row * width + column] = e4m3_code(bf2f(result) * quant_scale);
  }
}

// Vector form (width % 8 == 0, 16-byte aligned pointers): persistent blocks, each
// walking rows blockIdx.x, blockIdx.x + gridDim.x, ...  The next row of a block
// is copied into the other half of the shared row cache with cp.async while
// the current one is reduced and normalised, so a block always has a row of
// loads in flight instead of waiting for them at the start of every row.
template <int kWidth>
__global__ void __launch_bounds__(kThreads)
rms_norm_stream_kernel(const bf16 *__restrict__ input, const float *__restrict__ scale,
                       bf16 *__restrict__ output, std::uint8_t *__restrict__ codes, const std::size_t rows,
                       const std::size_t runtime_width, const float epsilon, const float quant_scale) {
  extern __shared__ __align__(16) unsigned short row_cache[];  // 2 x width BF16 values, then width BF16 scales
  __shared__ float partial[32];
  const std::size_t width = kWidth != 0 ? static_cast<std::size_t>(kWidth) : runtime_width;
  std::uint32_t *const scale_pairs = reinterpret_cast<std::uint32_t *>(row_cache + 2 * width);
  for (std::size_t i = threadIdx.x; i < width / 2; i += kThreads)
    scale_pairs[i] = round_pair(scale[2 * i], scale[2 * i + 1]);  // visible after the first barrier below
  const std::uint32_t cache_address = static_cast<std::uint32_t>(__cvta_generic_to_shared(row_cache));
  const auto fetch = [&](const std::size_t row, const int half) {
    const uint4 *const source = reinterpret_cast<const uint4 *>(input + row * width) + threadIdx.x;
    const std::uint32_t target =
        cache_address + static_cast<std::uint32_t>(half) * static_cast<std::uint32_t>(width) * 2U + threadIdx.x * 16U;
    if constexpr (kWidth != 0) {
#pragma unroll
      for (int k = 0; k < kWidth / 8 / kThreads; ++k)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(target + k * kThreads * 16),
                     "l"(source + k * kThreads)
                     : "memory");
    } else {
      const int vectors = static_cast<int>(width / 8);
      for (int v = threadIdx.x, k = 0; v < vectors; v += kThreads, ++k)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(target + k * kThreads * 16),
                     "l"(source + k * kThreads)
                     : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  std::size_t row = blockIdx.x;
  if (row >= rows) return;
  fetch(row, 0);
  for (int parity = 0; row < rows; row += gridDim.x, parity ^= 1) {
    unsigned short *const current = row_cache + parity * width;
    const std::size_t next = row + gridDim.x;
    // A thread's copies land in the chunks that only this thread reads in the
    // store phase; the strided reads of the reduction are fenced by its barriers.
    if (next < rows) {
      fetch(next, parity ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const float denominator = row_denominator<kWidth>(current, width, epsilon, partial);
    store_normalized_row<kWidth>(current, scale, scale_pairs, denominator, width,
                                 output == nullptr ? nullptr : output + row * width,
                                 codes == nullptr ? nullptr : codes + row * width, quant_scale);
  }
}

// ---------------------------------------------------------------- pointwise
__device__ __forceinline__ bf16 gelu_bf16(const bf16 input) {
  const float value = bf2f(input);
  constexpr float kAlpha = 0.70710678118654752440F;
  const bf16 computed = f2bf(value * 0.5F * (1.0F + ::erff(value * kAlpha)));
  // Seven inputs whose rounding depends on the libdevice erf revision are
  // pinned to fixed outputs upstream (src/cuda/ops.cu:125-139).
  switch (__bfloat16_as_ushort(input)) {
    case 0xc049: return __ushort_as_bfloat16(0xbb2d);
    case 0xc081: return __ushort_as_bfloat16(0xb8eb);
    case 0xc089: return __ushort_as_bfloat16(0xb827);
    case 0xc092: return __ushort_as_bfloat16(0xb742);
    case 0xc0a0: return __ushort_as_bfloat16(0xb5c8);
    case 0xc0a8: return __ushort_as_bfloat16(0xb4fc);
    case 0xc0ab: return __ushort_as_bfloat16(0xb4ab);
    default: return computed;
  }
}

enum class Pointwise { kGelu, kGate, kGeluGate, kAdd };

template <Pointwise Op>
__device__ __forceinline__ float pointwise(const float a, const float b) {
  if constexpr (Op == Pointwise::kGelu) {
    return bf2f(gelu_bf16(f2bf(a)));
  } else if constexpr (Op == Pointwise::kGate) {
    return a * b;
  } else if constexpr (Op == Pointwise::kGeluGate) {
    return bf2f(gelu_bf16(f2bf(a))) * b;
  } else {
    return a + b;
  }
}

template <Pointwise Op>
__global__ void pointwise_kernel(const bf16 *__restrict__ first,
                                 const bf16 *__restrict__ second,
                                 bf16 *__restrict__ output,
                                 const std::size_t elements) {
  const std::size_t vectors = elements / 8;
  const std::size_t stride = static_cast<std::size_t>(blockDim.x) * gridDim.x;
  const std::size_t tid =
      static_cast<std::size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  for (std::size_t i = tid; i < vectors; i += stride) {
    Bf16x8 a, b;
    a.raw = reinterpret_cast<const uint4 *>(first)[i];
    if constexpr (Op != Pointwise::kGelu)
      b.raw = reinterpret_cast<const uint4 *>(second)[i];
    else
      b.raw = a.raw;
    unsigned int out[4];
#pragma unroll
    for (int w = 0; w < 4; ++w)
      out[w] = pack_bf16x2(pointwise<Op>(a.get(2 * w), b.get(2 * w)),
                           pointwise<Op>(a.get(2 * w + 1), b.get(2 * w + 1)));
    reinterpret_cast<uint4 *>(output)[i] =
        make_uint4(out[0], out[1], out[2], out[3]);
  }
  for (std::size_t i = vectors * 8 + tid; i < elements; i += stride) {
    const float b = Op == Pointwise::kGelu ? 0.0F : bf2f(second[i]);
    output[i] = f2bf(pointwise<Op>(bf2f(first[i]), b));
  }
}

__global__ void add_bias_kernel(bf16 *__restrict__ output,
                                const bf16 *__restrict__ bias,
                                const std::size_t elements,
                                const std::size_t width) {
  const std::size_t stride = static_cast<std::size_t>(blockDim.x) * gridDim.x;
  for (std::size_t i = static_cast<std::size_t>(blockIdx.x) * blockDim.x +
                       threadIdx.x;
       i < elements; i += stride)
    output[i] = f2bf(bf2f(output[i]) + bf2f(bias[i % width]));
}

// An id outside the table is never used as an index: its row is written as
// zeros and bit 1 of the per-device error word is raised, which the next
// gemm_error_state() reports as an invalid argument.
__global__ void embedding_kernel(const std::uint32_t *__restrict__ tokens,
                                 const bf16 *__restrict__ table,
                                 bf16 *__restrict__ output,
                                 const std::size_t rows,
                                 const std::size_t width,
                                 const std::size_t vocabulary,
                                 int *const error_word) {
  const std::size_t elements = rows * width;
  const std::size_t stride = static_cast<std::size_t>(blockDim.x) * gridDim.x;
  for (std::size_t i = static_cast<std::size_t>(blockIdx.x) * blockDim.x +
                       threadIdx.x;
       i < elements; i += stride) {
    const std::size_t row = i / width;
    const std::size_t id = tokens[row];
    if (id < vocabulary) {
      output[i] = table[id * width + i % width];
    } else {
      output[i] = __ushort_as_bfloat16(0);
      if (i % width == 0) atomicOr(error_word, 2);
    }
  }
}

__global__ void split_triples_kernel(const bf16 *__restrict__ projection,
                                     bf16 *__restrict__ x2,
                                     bf16 *__restrict__ x1,
                                     bf16 *__restrict__ value,
                                     const std::size_t elements) {
  const std::size_t stride = static_cast<std::size_t>(blockDim.x) * gridDim.x;
  for (std::size_t i = static_cast<std::size_t>(blockIdx.x) * blockDim.x +
                       threadIdx.x;
       i < elements; i += stride) {
    x2[i] = projection[3 * i];
    x1[i] = projection[3 * i + 1];
    value[i] = projection[3 * i + 2];
  }
}

__global__ void transpose_kernel(const bf16 *__restrict__ input,
                                 bf16 *__restrict__ output,
                                 const std::size_t rows,
                                 const std::size_t columns) {
  __shared__ unsigned short tile[32][33];
  const std::size_t c0 = static_cast<std::size_t>(blockIdx.x) * 32;
  const std::size_t r0 = static_cast<std::size_t>(blockIdx.y) * 32;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const std::size_t r = r0 + j, c = c0 + threadIdx.x;
    if (r < rows && c < columns)
      tile[j][threadIdx.x] = __bfloat16_as_ushort(input[r * columns + c]);
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const std::size_t c = c0 + j, r = r0 + threadIdx.x;
    if (r < rows && c < columns)
      output[c * rows + r] = __ushort_as_bfloat16(tile[threadIdx.x][j]);
  }
}

bool aligned16(const void *p) {
  return (reinterpret_cast<std::uintptr_t>(p) & 15U) == 0;
}

}  // namespace

int quantize_bf16(const void *input, const std::size_t elements,
                  const float scale, void *codes, float *dequantized,
                  cudaStream_t stream) {
  if (input == nullptr || (codes == nullptr && dequantized == nullptr) ||
      !(scale > 0.0F) || !isfinite(scale))
    return fail(kInvalidArgument, "E4M3 quantise arguments are invalid");
  if (elements == 0) return kOk;
  if (dequantized == nullptr && elements % 16 == 0 && aligned16(input) &&
      aligned16(codes)) {
    quantize_bf16_vec_kernel<<<grid_for(elements / 16), kThreads, 0, stream>>>(
        static_cast<const uint4 *>(input), static_cast<uint4 *>(codes),
        elements / 16, scale);
  } else {
    quantize_kernel<bf16><<<grid_for(elements), kThreads, 0, stream>>>(
        static_cast<const bf16 *>(input), static_cast<std::uint8_t *>(codes),
        dequantized, elements, scale);
  }
  return check_launch("E4M3 quantise kernel");
}

int quantize_rows(const void *input, const std::size_t rows, const std::size_t width, void *codes,
                  float *row_scale, cudaStream_t stream) {
  if (input == nullptr || codes == nullptr || row_scale == nullptr || width == 0 || width % 8 != 0 ||
      width > 49152 || !aligned16(input) || (reinterpret_cast<std::uintptr_t>(codes) & 7U) != 0)
    return fail(kInvalidArgument, "row quantise arguments are invalid (width % 8, 16-byte aligned input)");
  if (rows == 0) return kOk;
  const std::size_t smem = 2 * width * sizeof(unsigned short);
  if (smem + 1024 > 48 * 1024 &&
      cudaFuncSetAttribute(quantize_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(smem)) != cudaSuccess)
    return fail(kCuda, "cannot raise the row quantise shared-memory limit");
  int resident = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, quantize_rows_kernel, kThreads, smem) != cudaSuccess ||
      resident < 1)
    resident = 1;
  const std::size_t grid = std::min<std::size_t>(rows, static_cast<std::size_t>(kSmCount) * resident);
  quantize_rows_kernel<<<static_cast<unsigned int>(grid), kThreads, smem, stream>>>(
      static_cast<const bf16 *>(input), static_cast<std::uint8_t *>(codes), row_scale, rows, width);
  return check_launch("row quantise kernel");
}

int amax_bf16(const void *input, const std::size_t elements, unsigned int *result_bits, cudaStream_t stream) {
  if (input == nullptr || result_bits == nullptr || elements % 8 != 0 || !aligned16(input))
    return fail(kInvalidArgument, "amax arguments are invalid (elements % 8, 16-byte aligned input)");
  if (cudaMemsetAsync(result_bits, 0, sizeof(unsigned int), stream) != cudaSuccess)
    return fail(kCuda, "cannot clear the amax word");
  if (elements == 0) return kOk;
  amax_bf16_kernel<<<grid_for(elements / 8), kThreads, 0, stream>>>(static_cast<const uint4 *>(input),
                                                                    elements / 8, result_bits);
  return check_launch("amax kernel");
}

int quantize_f32(const float *input, const std::size_t elements,
                 const float scale, void *codes, cudaStream_t stream) {
  if (input == nullptr || codes == nullptr || !(scale > 0.0F) ||
      !isfinite(scale))
    return fail(kInvalidArgument, "E4M3 quantise arguments are invalid");
  if (elements == 0) return kOk;
  quantize_kernel<float><<<grid_for(elements), kThreads, 0, stream>>>(
      input, static_cast<std::uint8_t *>(codes), nullptr, elements, scale);
  return check_launch("E4M3 F32 quantise kernel");
}

int rms_norm(const void *input, const float *scale, const std::size_t rows,
             const std::size_t width, const float epsilon, void *output,
             void *codes, const float quant_scale, cudaStream_t stream, const bool dependent_launch) {
  if (input == nullptr || scale == nullptr ||
      (output == nullptr && codes == nullptr) || width == 0 ||
      width > 24576 || rows > 0x7fffffffU)
    return fail(kInvalidArgument, "RMSNorm arguments are invalid");
  if (codes != nullptr && (!(quant_scale > 0.0F) || !isfinite(quant_scale)))
    return fail(kInvalidArgument, "RMSNorm quantisation scale is invalid");
  if (rows == 0) return kOk;
  const auto aligned = [](const void *q, const std::uintptr_t mask) {
    return (reinterpret_cast<std::uintptr_t>(q) & mask) == 0;
  };
  const bool vectors = width % 8 == 0 && aligned(input, 15) && aligned(scale, 15) &&
                       (output == nullptr || aligned(output, 15)) && (codes == nullptr || aligned(codes, 7));
  if (rows <= 8 && width % kThreads == 0) {
    const auto launch_few = [&](auto kernel) {
      cudaLaunchAttribute attribute{};
      attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attribute.val.programmaticStreamSerializationAllowed = dependent_launch ? 1 : 0;
      cudaLaunchConfig_t config{};
      config.gridDim = dim3(static_cast<unsigned int>(rows));
      config.blockDim = dim3(kThreads);
      config.stream = stream;
      config.attrs = &attribute;
      config.numAttrs = 1;
      if (cudaLaunchKernelEx(&config, kernel, static_cast<const bf16 *>(input), scale, static_cast<bf16 *>(output),
                             static_cast<std::uint8_t *>(codes), static_cast<int>(width), epsilon,
                             quant_scale) != cudaSuccess)
        return fail(kCuda, "cannot launch the RMSNorm kernel");
      return check_launch("RMSNorm kernel");
    };
    switch (width / kThreads) {
      case 1: return launch_few(rms_norm_few_rows_kernel<1>);
      case 2: return launch_few(rms_norm_few_rows_kernel<2>);
      case 4: return launch_few(rms_norm_few_rows_kernel<4>);
      case 8: return launch_few(rms_norm_few_rows_kernel<8>);     // 2048
      case 16: return launch_few(rms_norm_few_rows_kernel<16>);   // 4096
      case 32: return launch_few(rms_norm_few_rows_kernel<32>);   // 8192
      default: break;
    }
  }
  if (vectors) {
    const std::size_t smem = 3 * width * sizeof(unsigned short);
    const auto launch = [&](auto kernel) {
      if (smem + 1024 > 48 * 1024 &&  // the static reduction buffer counts against the default limit too
          cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) !=
              cudaSuccess)
        return fail(kCuda, "cannot raise the RMSNorm shared-memory limit");
      int resident = 0;
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kernel, kThreads, smem) != cudaSuccess ||
          resident < 1)
        resident = 1;
      const std::size_t grid = std::min<std::size_t>(rows, static_cast<std::size_t>(kSmCount) * resident);
      kernel<<<static_cast<unsigned int>(grid), kThreads, smem, stream>>>(
          static_cast<const bf16 *>(input), scale, static_cast<bf16 *>(output), static_cast<std::uint8_t *>(codes),
          rows, width, epsilon, quant_scale);
      return check_launch("RMSNorm kernel");
    };
    // width 4096 (the 7B shape) gets the fully unrolled kernel: 30.7 against 32.8 us when it writes E4M3
    // codes, no difference for BF16 output; at 8192 the unrolled form measured slower (49 against 45 us)
    if (width == 4096) return launch(rms_norm_stream_kernel<4096>);
    return launch(rms_norm_stream_kernel<0>);
  }
  rms_norm_kernel<<<static_cast<unsigned int>(rows), kThreads,
                    width * sizeof(unsigned short), stream>>>(
      static_cast<const bf16 *>(input), scale, static_cast<bf16 *>(output),
      static_cast<std::uint8_t *>(codes), width, epsilon, quant_scale);
  return check_launch("RMSNorm kernel");
}

template <Pointwise Op>
static int launch_pointwise(const void *a, const void *b, void *out,
                            const std::size_t elements, cudaStream_t stream,
                            const char *what) {
  if (a == nullptr || out == nullptr ||
      (Op != Pointwise::kGelu && b == nullptr))
    return fail(kInvalidArgument, std::string(what) + " arguments are invalid");
  if (elements == 0) return kOk;
  if (!aligned16(a) || !aligned16(out) || (b != nullptr && !aligned16(b)))
    return fail(kInvalidArgument,
                std::string(what) + " buffers must be 16-byte aligned");
  pointwise_kernel<Op><<<grid_for(elements / 8 + 1), kThreads, 0, stream>>>(
      static_cast<const bf16 *>(a), static_cast<const bf16 *>(b),
      static_cast<bf16 *>(out), elements);
  return check_launch(what);
}

int gelu(const void *input, void *output, const std::size_t elements,
         cudaStream_t stream) {
  return launch_pointwise<Pointwise::kGelu>(input, nullptr, output, elements,
                                            stream, "GELU kernel");
}

int gate(const void *first, const void *second, void *output,
         const std::size_t elements, const bool apply_gelu,
         cudaStream_t stream) {
  return apply_gelu ? launch_pointwise<Pointwise::kGeluGate>(
                          first, second, output, elements, stream,
                          "GELU gate kernel")
                    : launch_pointwise<Pointwise::kGate>(
                          first, second, output, elements, stream,
                          "gate kernel");
}

int add(const void *first, const void *second, void *output,
        const std::size_t elements, cudaStream_t stream) {
  return launch_pointwise<Pointwise::kAdd>(first, second, output, elements,
                                           stream, "residual add kernel");
}

int add_bias(void *output, const void *bias, const std::size_t rows,
             const std::size_t width, cudaStream_t stream) {
  if (output == nullptr || bias == nullptr || width == 0)
    return fail(kInvalidArgument, "bias add arguments are invalid");
  if (rows == 0) return kOk;
  add_bias_kernel<<<grid_for(rows * width), kThreads, 0, stream>>>(
      static_cast<bf16 *>(output), static_cast<const bf16 *>(bias),
      rows * width, width);
  return check_launch("bias add kernel");
}

int embedding(const std::uint32_t *tokens, const void *table,
              const std::size_t rows, const std::size_t width,
              const std::size_t vocabulary, void *output, cudaStream_t stream) {
  if (tokens == nullptr || table == nullptr || output == nullptr || width == 0 ||
      vocabulary == 0)
    return fail(kInvalidArgument, "embedding arguments are invalid");
  if (rows == 0) return kOk;
  int status = kOk;
  int *const error_word = device_error_word(&status);
  if (error_word == nullptr) return status;
  embedding_kernel<<<grid_for(rows * width), kThreads, 0, stream>>>(
      tokens, static_cast<const bf16 *>(table), static_cast<bf16 *>(output),
      rows, width, vocabulary, error_word);
  return check_launch("embedding kernel");
}

int split_triples(const void *projection, const std::size_t rows,
                  const std::size_t width, void *x2, void *x1, void *value,
                  cudaStream_t stream) {
  if (projection == nullptr || x2 == nullptr || x1 == nullptr ||
      value == nullptr || width == 0)
    return fail(kInvalidArgument, "projection split arguments are invalid");
  if (rows == 0) return kOk;
  split_triples_kernel<<<grid_for(rows * width), kThreads, 0, stream>>>(
      static_cast<const bf16 *>(projection), static_cast<bf16 *>(x2),
      static_cast<bf16 *>(x1), static_cast<bf16 *>(value), rows * width);
  return check_launch("projection split kernel");
}

int transpose(const void *input, const std::size_t rows,
              const std::size_t columns, void *output, cudaStream_t stream) {
  if (input == nullptr || output == nullptr || rows == 0 || columns == 0)
    return fail(kInvalidArgument, "transpose arguments are invalid");
  const dim3 grid(ceil_div_u(columns, 32), ceil_div_u(rows, 32));
  if (grid.y > 65535)
    return fail(kInvalidArgument, "transpose has too many rows");
  transpose_kernel<<<grid, dim3(32, 8), 0, stream>>>(
      static_cast<const bf16 *>(input), static_cast<bf16 *>(output), rows,
      columns);
  return check_launch("transpose kernel");
}

}  // namespace evob
