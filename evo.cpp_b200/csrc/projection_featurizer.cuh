// 3-tap depthwise featurizer of the Hyena input projection, evaluated from
// shared memory for one 8-channel chunk of one row.
//
// The projection row holds channel triples (x2, x1, v) interleaved: column
// 3c + s is stream s of channel c, so 8 channels are 48 contiguous bytes.  Each
// of the 24 columns has its own 3 taps; z = bf16(sum over taps, oldest first,
// F32 FMAs) per column, then u = bf16(z_x1 * z_v) and the x2 gate g = z_x2
// (upstream: short FIR over [3D] columns, split, x1*v gate;
// src/cuda/model.cu:1431-1470).  Results are produced as packed BF16 pairs of
// neighbouring channels, rounding two values per cvt instruction.
#pragma once

#include "common.cuh"

namespace evob {

__device__ __forceinline__ std::uint32_t round_pair_bf16(const float low, const float high) {
  std::uint32_t packed;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(packed) : "f"(high), "f"(low));
  return packed;
}

// Packed taps of one chunk: 72 BF16 = 36 words, as stored ([column][tap]).
struct PackedTaps {
  std::uint32_t words[36];
  __device__ __forceinline__ void load_global(const bf16 *short_filter, const int c0) {
    const uint4 *w = reinterpret_cast<const uint4 *>(short_filter + static_cast<std::size_t>(c0) * 9);
#pragma unroll
    for (int i = 0; i < 9; ++i) {
      const uint4 v = __ldg(w + i);
      words[4 * i] = v.x; words[4 * i + 1] = v.y; words[4 * i + 2] = v.z; words[4 * i + 3] = v.w;
    }
  }
  __device__ __forceinline__ void load_shared(const std::uint32_t *source) {
#pragma unroll
    for (int i = 0; i < 9; ++i) {
      const uint4 v = *reinterpret_cast<const uint4 *>(source + 4 * i);
      words[4 * i] = v.x; words[4 * i + 1] = v.y; words[4 * i + 2] = v.z; words[4 * i + 3] = v.w;
    }
  }
  __device__ __forceinline__ float tap(const int index) const {
    const std::uint32_t word = words[index >> 1];
    return (index & 1) ? __uint_as_float(word & 0xffff0000U) : __uint_as_float(word << 16U);
  }
};

// rows[k]: the 48 bytes of the chunk at time t-2+k (shared memory, 16-byte
// aligned).  u[j], g[j]: packed BF16 of channels (2j, 2j+1); g is left
// untouched when kNeedGate is false.
template <bool kNeedGate>
__device__ __forceinline__ void featurize_chunk(const unsigned char *const (&rows)[3], const PackedTaps &taps,
                                                std::uint32_t (&u)[4], std::uint32_t (&g)[4]) {
  std::uint32_t x[3][12];
#pragma unroll
  for (int k = 0; k < 3; ++k)
#pragma unroll
    for (int v = 0; v < 3; ++v) {
      const uint4 q = *reinterpret_cast<const uint4 *>(rows[k] + 16 * v);
      x[k][4 * v] = q.x; x[k][4 * v + 1] = q.y; x[k][4 * v + 2] = q.z; x[k][4 * v + 3] = q.w;
    }
  const auto value = [&](const int k, const int column) {
    const std::uint32_t word = x[k][column >> 1];
    return (column & 1) ? __uint_as_float(word & 0xffff0000U) : __uint_as_float(word << 16U);
  };
  const auto column_sum = [&](const int column) {
    // fmaf with +0, not a multiply: the sign of a zero result must match the FMA chain
    float acc = fmaf(value(0, column), taps.tap(column * 3), 0.0F);
    acc = fmaf(value(1, column), taps.tap(column * 3 + 1), acc);
    return fmaf(value(2, column), taps.tap(column * 3 + 2), acc);
  };
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int a = 3 * (2 * j), b = 3 * (2 * j + 1);  // first columns of the two channels
    if constexpr (kNeedGate) g[j] = round_pair_bf16(column_sum(a), column_sum(b));
    const std::uint32_t x1 = round_pair_bf16(column_sum(a + 1), column_sum(b + 1));
    const std::uint32_t v = round_pair_bf16(column_sum(a + 2), column_sum(b + 2));
    u[j] = round_pair_bf16(__uint_as_float(x1 << 16U) * __uint_as_float(v << 16U),
                           __uint_as_float(x1 & 0xffff0000U) * __uint_as_float(v & 0xffff0000U));
  }
}

}  // namespace evob
